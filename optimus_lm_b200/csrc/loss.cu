// Cross entropy on bf16 logits with fp32 statistics: one block per row, online softmax in a
// single read for the forward, and a backward that may overwrite the logits in place (the
// [tokens, vocab] logits are the largest activation of the step).
// Reference: F.cross_entropy on the shifted logits, optimus/models/olmoe/modeling_olmoe.py:515-524.
//
// Vocabulary-parallel form: a rank holds the logits of the vocabulary slice [v_start, v_start + V) only.  The forward
// then writes the slice's statistics per row - its maximum, its sum of exponentials relative to that maximum and the
// target's logit if the target falls into the slice - which the caller merges over the ranks (one max and one sum
// all-reduce of [rows] floats) into the global log-sum-exp; the backward takes that and writes the slice's gradient.
// The [rows, vocabulary] logits themselves never cross the links (the reference all-reduces them:
// optimus/models/common/parallel_modules.py:75-80).
#include <cfloat>

#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

constexpr int CE_THREADS = 256;

__device__ __forceinline__ void online_merge(float& m, float& s, float om, float os) {
  const float nm = fmaxf(m, om);
  s = s * __expf(m - nm) + os * __expf(om - nm);
  m = nm;
}

__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, long long ldl, const long long* __restrict__ labels,
              float* __restrict__ loss_row, float* __restrict__ lse_out, int rows, int V, int v_start,
              float* __restrict__ part_max, float* __restrict__ part_sum, float* __restrict__ part_tgt) {
  __shared__ float s_m[CE_THREADS / 32], s_s[CE_THREADS / 32];
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + static_cast<long long>(row) * ldl;
  float m = -FLT_MAX, s = 0.f;
  const int nvec = V / 8;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    const uint4 v = *reinterpret_cast<const uint4*>(lr + i * 8);
    float f[8];
    float2 a;
    a = unpack_bf16(v.x); f[0] = a.x; f[1] = a.y;
    a = unpack_bf16(v.y); f[2] = a.x; f[3] = a.y;
    a = unpack_bf16(v.z); f[4] = a.x; f[5] = a.y;
    a = unpack_bf16(v.w); f[6] = a.x; f[7] = a.y;
    float lm = f[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) lm = fmaxf(lm, f[k]);
    const float nm = fmaxf(m, lm);
    float add = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) add += __expf(f[k] - nm);
    s = s * __expf(m - nm) + add;
    m = nm;
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    const float f = __bfloat162float(lr[i]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, om, os);
  }
  if ((threadIdx.x & 31) == 0) {
    s_m[threadIdx.x >> 5] = m;
    s_s[threadIdx.x >> 5] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = s_m[0], ss = s_s[0];
    for (int w = 1; w < CE_THREADS / 32; ++w) online_merge(mm, ss, s_m[w], s_s[w]);
    const long long lab = labels[row] - v_start;
    const bool mine = lab >= 0 && lab < V;
    if (part_max != nullptr) {  // vocabulary slice: statistics for the caller to merge over the ranks
      part_max[row] = mm;
      part_sum[row] = ss;
      part_tgt[row] = mine ? __bfloat162float(lr[lab]) : 0.f;
    } else {
      const float lse = mm + __logf(ss);
      lse_out[row] = lse;
      loss_row[row] = mine ? lse - __bfloat162float(lr[lab]) : 0.f;
    }
  }
}

__global__ void __launch_bounds__(CE_THREADS)
ce_bwd_kernel(const __nv_bfloat16* __restrict__ logits, long long ldl, const long long* __restrict__ labels,
              const float* __restrict__ lse, const float* __restrict__ scale_dev, __nv_bfloat16* __restrict__ dlogits,
              int rows, int V, int v_start, int v_total) {
  const int row = blockIdx.x;
  const bool valid = labels[row] >= 0 && labels[row] < v_total;  // a target anywhere in the whole vocabulary
  const long long lab = labels[row] - v_start;                  // its column in this slice, if it is here
  const float scale = valid ? *scale_dev : 0.f;
  const float l = lse[row];
  const __nv_bfloat16* lr = logits + static_cast<long long>(row) * ldl;
  __nv_bfloat16* dr = dlogits + static_cast<long long>(row) * ldl;
  const int nvec = V / 8;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    const uint4 v = *reinterpret_cast<const uint4*>(lr + i * 8);
    float f[8];
    float2 a;
    a = unpack_bf16(v.x); f[0] = a.x; f[1] = a.y;
    a = unpack_bf16(v.y); f[2] = a.x; f[3] = a.y;
    a = unpack_bf16(v.z); f[4] = a.x; f[5] = a.y;
    a = unpack_bf16(v.w); f[6] = a.x; f[7] = a.y;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float p = __expf(f[k] - l);
      if (i * 8 + k == lab) p -= 1.f;
      f[k] = p * scale;
    }
    uint4 o;
    o.x = pack_bf16(f[0], f[1]);
    o.y = pack_bf16(f[2], f[3]);
    o.z = pack_bf16(f[4], f[5]);
    o.w = pack_bf16(f[6], f[7]);
    *reinterpret_cast<uint4*>(dr + i * 8) = o;
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    float p = __expf(__bfloat162float(lr[i]) - l);
    if (i == lab) p -= 1.f;
    dr[i] = __float2bfloat16_rn(p * scale);
  }
}

}  // namespace olb

using namespace olb;

extern "C" int olb_ce_fwd(const void* logits, long long ldl, const long long* labels, float* loss_row, float* lse,
                          int rows, int V, cudaStream_t stream) {
  if (ldl % 8 || (reinterpret_cast<uintptr_t>(logits) & 15)) return -1;
  if (rows <= 0) return 0;
  ce_fwd_kernel<<<rows, CE_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), ldl, labels, loss_row, lse,
                                                 rows, V, 0, nullptr, nullptr, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_ce_partial_fwd(const void* logits, long long ldl, const long long* labels, int v_start, float* part_max,
                                  float* part_sum, float* part_tgt, int rows, int V, cudaStream_t stream) {
  if (ldl % 8 || (reinterpret_cast<uintptr_t>(logits) & 15)) return -1;
  if (rows <= 0) return 0;
  ce_fwd_kernel<<<rows, CE_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), ldl, labels, nullptr, nullptr,
                                                 rows, V, v_start, part_max, part_sum, part_tgt);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_ce_bwd(const void* logits, long long ldl, const long long* labels, const float* lse,
                          const float* scale_dev, void* dlogits, int rows, int V, cudaStream_t stream) {
  if (ldl % 8 || (reinterpret_cast<uintptr_t>(logits) & 15) || (reinterpret_cast<uintptr_t>(dlogits) & 15)) return -1;
  if (rows <= 0) return 0;
  ce_bwd_kernel<<<rows, CE_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), ldl, labels, lse, scale_dev,
                                                 static_cast<__nv_bfloat16*>(dlogits), rows, V, 0, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_ce_partial_bwd(const void* logits, long long ldl, const long long* labels, int v_start, int v_total,
                                  const float* lse, const float* scale_dev, void* dlogits, int rows, int V,
                                  cudaStream_t stream) {
  if (ldl % 8 || (reinterpret_cast<uintptr_t>(logits) & 15) || (reinterpret_cast<uintptr_t>(dlogits) & 15)) return -1;
  if (rows <= 0) return 0;
  ce_bwd_kernel<<<rows, CE_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), ldl, labels, lse, scale_dev,
                                                 static_cast<__nv_bfloat16*>(dlogits), rows, V, v_start, v_total);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
