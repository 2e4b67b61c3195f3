// MoE routers.  One warp owns one token; experts are striped over lanes (expert e lives in
// lane e % 32, slot e / 32), so E <= 256.
//
//  * softmax router (OLMoE): fp32 softmax over bf16 logits, top-k by repeated warp arg-max
//    (ties -> lowest expert id), optional renormalisation; also emits per-block partial sums
//    for the Switch load-balance loss (selection counts and mean probabilities per expert)
//    and for a z-loss (sum of logsumexp^2).  Reference: optimus/models/olmoe/modeling_olmoe.py
//    :295-299 (routing) and :29-85 (load_balancing_loss_func).
//  * sigmoid router (DeepSeek-V3): sigmoid scores, selection on score+bias restricted to the
//    best `topk_group` of `n_group` groups (group score = sum of its two best), weights are
//    the unbiased scores, renormalised (+1e-20) and scaled.  Reference:
//    optimus/models/deepseek_v3/modeling_deepseek_v3.py:131-192.
#include <cfloat>

#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

constexpr int R_WARPS = 4;
constexpr int R_THREADS = R_WARPS * 32;
constexpr int MAX_SLOTS = 8;  // E <= 256
constexpr int MAX_K = 16;

// Warp-wide arg-max over per-lane candidates (value, index); ties -> smaller index.
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) {
      v = ov;
      idx = oi;
    }
  }
}

__global__ void __launch_bounds__(R_THREADS)
router_softmax_topk_kernel(const __nv_bfloat16* __restrict__ logits, int T, int E, int K, int renorm,
                           float* __restrict__ weights, int* __restrict__ indices, float* __restrict__ cnt_partial,
                           float* __restrict__ prob_partial, float* __restrict__ lse_sq_partial) {
  __shared__ float s_cnt[R_WARPS][256];
  __shared__ float s_prob[R_WARPS][256];
  __shared__ float s_lse[R_WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = (E + 31) / 32;
  float cnt_acc[MAX_SLOTS], prob_acc[MAX_SLOTS];
#pragma unroll
  for (int s = 0; s < MAX_SLOTS; ++s) cnt_acc[s] = prob_acc[s] = 0.f;
  float lse_acc = 0.f;

  for (int t = blockIdx.x * R_WARPS + warp; t < T; t += gridDim.x * R_WARPS) {
    float p[MAX_SLOTS];
    float mx = -FLT_MAX;
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) {
      const int e = s * 32 + lane;
      p[s] = (s < slots && e < E) ? __bfloat162float(logits[static_cast<long long>(t) * E + e]) : -FLT_MAX;
      mx = fmaxf(mx, p[s]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) {
      const int e = s * 32 + lane;
      p[s] = (s < slots && e < E) ? __expf(p[s] - mx) : 0.f;
      sum += p[s];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    const float lse = mx + __logf(sum);
    lse_acc += lse * lse;
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) {
      p[s] *= inv;
      prob_acc[s] += p[s];
    }
    // top-k
    float sel_w = 0.f;  // lane k keeps the k-th weight
    int sel_i = -1;
    float wsum = 0.f;
    unsigned taken = 0;  // bit s set: this lane's slot s already selected
    for (int k = 0; k < K; ++k) {
      float bv = -1.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int s = 0; s < MAX_SLOTS; ++s) {
        const int e = s * 32 + lane;
        if (s < slots && e < E && !(taken & (1u << s)) && (p[s] > bv)) {
          bv = p[s];
          bi = e;
        }
      }
      warp_argmax(bv, bi);
      if ((bi & 31) == lane) {
        taken |= 1u << (bi >> 5);
        cnt_acc[bi >> 5] += 1.f;
      }
      if (lane == k) {
        sel_w = bv;
        sel_i = bi;
      }
      wsum += bv;
    }
    if (lane < K) {
      weights[static_cast<long long>(t) * K + lane] = renorm ? sel_w / wsum : sel_w;
      indices[static_cast<long long>(t) * K + lane] = sel_i;
    }
  }
  if (cnt_partial) {
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) {
      s_cnt[warp][s * 32 + lane] = cnt_acc[s];
      s_prob[warp][s * 32 + lane] = prob_acc[s];
    }
    if (lane == 0) s_lse[warp] = lse_acc;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += R_THREADS) {
      float c = 0.f, q = 0.f;
#pragma unroll
      for (int w = 0; w < R_WARPS; ++w) {
        c += s_cnt[w][e];
        q += s_prob[w][e];
      }
      cnt_partial[static_cast<long long>(blockIdx.x) * E + e] = c;
      prob_partial[static_cast<long long>(blockIdx.x) * E + e] = q;
    }
    if (threadIdx.x == 0 && lse_sq_partial) {
      float z = 0.f;
#pragma unroll
      for (int w = 0; w < R_WARPS; ++w) z += s_lse[w];
      lse_sq_partial[blockIdx.x] = z;
    }
  }
}

__global__ void __launch_bounds__(R_THREADS)
router_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const int* __restrict__ indices,
                  const float* __restrict__ dweights, int T, int E, int K, int renorm, const float* __restrict__ aux_f,
                  const float* __restrict__ aux_scale_dev, float aux_scale, float z_scale,
                  __nv_bfloat16* __restrict__ dlogits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = (E + 31) / 32;
  const float ascale = aux_f ? aux_scale * (aux_scale_dev ? *aux_scale_dev : 1.f) : 0.f;
  const float zscale = z_scale * (aux_scale_dev ? *aux_scale_dev : 1.f);
  for (int t = blockIdx.x * R_WARPS + warp; t < T; t += gridDim.x * R_WARPS) {
    float p[MAX_SLOTS], dp[MAX_SLOTS];
    float mx = -FLT_MAX;
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) {
      const int e = s * 32 + lane;
      p[s] = (s < slots && e < E) ? __bfloat162float(logits[static_cast<long long>(t) * E + e]) : -FLT_MAX;
      mx = fmaxf(mx, p[s]);
      dp[s] = 0.f;
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) {
      const int e = s * 32 + lane;
      p[s] = (s < slots && e < E) ? __expf(p[s] - mx) : 0.f;
      sum += p[s];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    const float lse = mx + __logf(sum);
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) p[s] *= inv;

    if (dweights) {
      // lane k holds the k-th selection
      const int my_i = lane < K ? indices[static_cast<long long>(t) * K + lane] : -1;
      float my_dw = lane < K ? dweights[static_cast<long long>(t) * K + lane] : 0.f;
      if (renorm) {
        // w_k = p_k / S  ->  dp_k = (dw_k - sum_j dw_j w_j) / S
        float my_p = 0.f;
        // gather p at the selected experts: owner lane = i % 32, slot = i / 32
        for (int k = 0; k < K; ++k) {
          const int ik = __shfl_sync(0xffffffffu, my_i, k);
          float v = 0.f;
#pragma unroll
          for (int s = 0; s < MAX_SLOTS; ++s)
            if (s == (ik >> 5)) v = p[s];
          v = __shfl_sync(0xffffffffu, v, ik & 31);
          if (lane == k) my_p = v;
        }
        const float S = warp_sum(lane < K ? my_p : 0.f);
        const float dot = warp_sum(lane < K ? my_dw * my_p / S : 0.f);
        my_dw = (my_dw - dot) / S;
      }
      for (int k = 0; k < K; ++k) {
        const int ik = __shfl_sync(0xffffffffu, my_i, k);
        const float dk = __shfl_sync(0xffffffffu, my_dw, k);
        if ((ik & 31) == lane) {
#pragma unroll
          for (int s = 0; s < MAX_SLOTS; ++s)
            if (s == (ik >> 5)) dp[s] += dk;
        }
      }
    }
    if (ascale != 0.f) {
#pragma unroll
      for (int s = 0; s < MAX_SLOTS; ++s) {
        const int e = s * 32 + lane;
        if (s < slots && e < E) dp[s] += ascale * aux_f[e];
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) dot += dp[s] * p[s];
    dot = warp_sum(dot);
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) {
      const int e = s * 32 + lane;
      if (s < slots && e < E) {
        float g = p[s] * (dp[s] - dot);
        g += zscale * 2.f * lse * p[s];
        dlogits[static_cast<long long>(t) * E + e] = __float2bfloat16_rn(g);
      }
    }
  }
}

// ------------------------------------------------------------------ DeepSeek-V3 sigmoid router
__global__ void __launch_bounds__(R_THREADS)
router_sigmoid_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int K, int n_group,
                      int topk_group, int renorm, float scale, float* __restrict__ weights,
                      int* __restrict__ indices) {
  __shared__ float s_choice[R_WARPS][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = (E + 31) / 32;
  const int gsize = E / n_group;
  for (int t = blockIdx.x * R_WARPS + warp; t < T; t += gridDim.x * R_WARPS) {
    float sc[MAX_SLOTS], ch[MAX_SLOTS];
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) {
      const int e = s * 32 + lane;
      if (s < slots && e < E) {
        sc[s] = 1.f / (1.f + __expf(-logits[static_cast<long long>(t) * E + e]));
        ch[s] = sc[s] + (bias ? bias[e] : 0.f);
        s_choice[warp][e] = ch[s];
      } else {
        sc[s] = 0.f;
        ch[s] = -FLT_MAX;
      }
    }
    __syncwarp();
    // group score = sum of the two best choices in the group (lane g scans group g)
    float gscore = -FLT_MAX;
    if (lane < n_group) {
      float b1 = -FLT_MAX, b2 = -FLT_MAX;
      for (int j = 0; j < gsize; ++j) {
        const float v = s_choice[warp][lane * gsize + j];
        if (v > b1) {
          b2 = b1;
          b1 = v;
        } else if (v > b2) {
          b2 = v;
        }
      }
      gscore = b1 + b2;
    }
    // rank of each group: number of groups that beat it (ties -> lower index wins)
    int rank = 0;
    for (int g = 0; g < n_group; ++g) {
      const float og = __shfl_sync(0xffffffffu, gscore, g);
      if (lane < n_group && (og > gscore || (og == gscore && g < lane))) ++rank;
    }
    const unsigned group_mask = __ballot_sync(0xffffffffu, lane < n_group && rank < topk_group);
    __syncwarp();
#pragma unroll
    for (int s = 0; s < MAX_SLOTS; ++s) {
      const int e = s * 32 + lane;
      if (s < slots && e < E) {
        // experts outside the chosen groups compete with score 0, as masked_fill(~mask, 0.0) does
        if (!((group_mask >> (e / gsize)) & 1u)) ch[s] = 0.f;
      }
    }
    float sel_w = 0.f;
    int sel_i = -1;
    float wsum = 0.f;
    unsigned taken = 0;
    for (int k = 0; k < K; ++k) {
      float bv = -FLT_MAX, bw = 0.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int s = 0; s < MAX_SLOTS; ++s) {
        const int e = s * 32 + lane;
        if (s < slots && e < E && !(taken & (1u << s)) && ch[s] > bv) {
          bv = ch[s];
          bi = e;
          bw = sc[s];
        }
      }
      float v = bv;
      int idx = bi;
      warp_argmax(v, idx);
      const float w = __shfl_sync(0xffffffffu, bw, idx & 31);
      // the owner lane's candidate is its best remaining one, which is the winner itself
      if ((idx & 31) == lane) taken |= 1u << (idx >> 5);
      if (lane == k) {
        sel_w = w;
        sel_i = idx;
      }
      wsum += w;
    }
    if (lane < K) {
      float w = sel_w;
      if (renorm) w = w / (wsum + 1e-20f);
      weights[static_cast<long long>(t) * K + lane] = w * scale;
      indices[static_cast<long long>(t) * K + lane] = sel_i;
    }
    __syncwarp();
  }
}

__global__ void router_sigmoid_bwd_kernel(const float* __restrict__ logits, const int* __restrict__ indices,
                                          const float* __restrict__ dweights, int T, int E, int K, int renorm,
                                          float scale, float* __restrict__ dlogits) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float s[MAX_K], du[MAX_K];
  float S = 0.f;
  for (int k = 0; k < K; ++k) {
    const int e = indices[static_cast<long long>(t) * K + k];
    s[k] = 1.f / (1.f + __expf(-logits[static_cast<long long>(t) * E + e]));
    du[k] = dweights[static_cast<long long>(t) * K + k] * scale;
    S += s[k];
  }
  float dot = 0.f;
  if (renorm) {
    S += 1e-20f;
    for (int k = 0; k < K; ++k) dot += du[k] * s[k] / S;
  }
  for (int k = 0; k < K; ++k) {
    const int e = indices[static_cast<long long>(t) * K + k];
    const float ds = renorm ? (du[k] - dot) / S : du[k];
    dlogits[static_cast<long long>(t) * E + e] = ds * s[k] * (1.f - s[k]);
  }
}

}  // namespace olb

using namespace olb;

extern "C" int olb_router_blocks(int T) {
  int nb = (T + R_WARPS - 1) / R_WARPS;
  return nb < 1 ? 1 : (nb > 592 ? 592 : nb);
}

extern "C" int olb_router_softmax_topk(const void* logits, int T, int E, int K, int renorm, float* weights,
                                       int* indices, float* cnt_partial, float* prob_partial, float* lse_sq_partial,
                                       cudaStream_t stream) {
  if (E > 256 || K > MAX_K || K > E || K > 32) return -1;
  if (T <= 0) return 0;
  router_softmax_topk_kernel<<<olb_router_blocks(T), R_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(logits), T, E, K, renorm, weights, indices, cnt_partial, prob_partial,
      lse_sq_partial);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_router_bwd_ex(const void* logits, const int* indices, const float* dweights, int T, int E, int K,
                                 int renorm, const float* aux_f, const float* aux_scale_dev, float aux_scale,
                                 float z_scale, void* dlogits, cudaStream_t stream) {
  if (E > 256 || K > MAX_K || K > 32) return -1;
  if (T <= 0) return 0;
  router_bwd_kernel<<<olb_router_blocks(T), R_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(logits), indices, dweights, T, E, K, renorm, aux_f, aux_scale_dev, aux_scale,
      z_scale, static_cast<__nv_bfloat16*>(dlogits));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_router_bwd(const void* logits, const int* indices, const float* dweights, int T, int E, int K,
                              int renorm, const float* aux_f, float aux_scale, float z_scale, void* dlogits,
                              cudaStream_t stream) {
  return olb_router_bwd_ex(logits, indices, dweights, T, E, K, renorm, aux_f, nullptr, aux_scale, z_scale, dlogits,
                           stream);
}

extern "C" int olb_router_sigmoid_group_topk(const float* logits, const float* bias, int T, int E, int K, int n_group,
                                             int topk_group, int renorm, float scale, float* weights, int* indices,
                                             cudaStream_t stream) {
  if (E > 256 || K > MAX_K || n_group > 32 || E % n_group || K > 32) return -1;
  if (T <= 0) return 0;
  router_sigmoid_kernel<<<olb_router_blocks(T), R_THREADS, 0, stream>>>(logits, bias, T, E, K, n_group, topk_group,
                                                                         renorm, scale, weights, indices);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_router_sigmoid_bwd(const float* logits, const int* indices, const float* dweights, int T, int E,
                                      int K, int renorm, float scale, float* dlogits, cudaStream_t stream) {
  if (K > MAX_K) return -1;
  if (T <= 0) return 0;
  router_sigmoid_bwd_kernel<<<(T + 127) / 128, 128, 0, stream>>>(logits, indices, dweights, T, E, K, renorm, scale,
                                                                 dlogits);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
