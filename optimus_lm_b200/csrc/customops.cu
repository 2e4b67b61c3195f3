// CUDA kernels behind the entry points of the reference's MoE custom-op extension
// (pytorch_xpu_extensions/pcl.xpu.customops/csrc/ops/sparse_moe_block.sycl:538-548), with that extension's data layout:
//
//   TH = ceil(T / 8) "token blocks" of 8 tokens each;
//   partial_token_counts [E_loc, TH]          hits of each local expert inside each token block;
//   expert_counts_ep [T], cum_expert_counts_ep [T + 1]   local-expert hits per token and their exclusive prefix: the
//                                              token-major *slots* of the routed pairs;
//   rows are ordered by (expert, token block, token, k); input_indices [R] maps row -> token, output_indices [R] maps
//   slot -> row, selected_experts_indices [R] maps slot -> k.
//
// The framework's own MoE path uses the padded, tile-aligned index of moe.cu instead; these kernels serve code written
// against the reference's interface.  bf16 and fp32 data, int32 indices, fp32 accumulation.
#include <cuda_bf16.h>

#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

constexpr int TOK_PER_BLOCK = 8;

// K1: one thread per token block; it owns column `th` of partial_token_counts.
__global__ void co_partial_counts_kernel(const int* __restrict__ sel, int T, int K, int e_start, int E_loc, int TH,
                                         int* __restrict__ partial, int* __restrict__ counts_ep) {
  const int th = blockIdx.x * blockDim.x + threadIdx.x;
  if (th >= TH) return;
  for (int e = 0; e < E_loc; ++e) partial[static_cast<long long>(e) * TH + th] = 0;
  for (int t = th * TOK_PER_BLOCK; t < min(T, (th + 1) * TOK_PER_BLOCK); ++t) {
    int hits = 0;
    for (int k = 0; k < K; ++k) {
      const int e = sel[static_cast<long long>(t) * K + k] - e_start;
      if (e >= 0 && e < E_loc) {
        partial[static_cast<long long>(e) * TH + th] += 1;
        ++hits;
      }
    }
    counts_ep[t] = hits;
  }
}

// K3: one thread per token block walks its tokens in (token, k) order; `incr` [E_loc, TH] is its running position inside
// each (expert, token block) bucket, whose first row is partial_cum[e * TH + th].
__global__ void co_indices_kernel(const int* __restrict__ sel, int T, int K, int e_start, int E_loc, int TH,
                                  const int* __restrict__ partial_cum, int* __restrict__ incr,
                                  const int* __restrict__ cum_ep, int* __restrict__ sel_idx, int* __restrict__ in_idx,
                                  int* __restrict__ out_idx) {
  const int th = blockIdx.x * blockDim.x + threadIdx.x;
  if (th >= TH) return;
  for (int e = 0; e < E_loc; ++e) incr[static_cast<long long>(e) * TH + th] = 0;
  for (int t = th * TOK_PER_BLOCK; t < min(T, (th + 1) * TOK_PER_BLOCK); ++t) {
    int slot = cum_ep[t];
    for (int k = 0; k < K; ++k) {
      const int e = sel[static_cast<long long>(t) * K + k] - e_start;
      if (e >= 0 && e < E_loc) {
        const long long b = static_cast<long long>(e) * TH + th;
        const int row = partial_cum[b] + incr[b];
        incr[b] += 1;
        in_idx[row] = t;
        out_idx[slot] = row;
        sel_idx[slot] = k;
        ++slot;
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// K4f: out[o, :] = inp[indices[o], :].  One block per output row.
template <typename T>
__global__ void co_gather_kernel(const T* __restrict__ inp, const int* __restrict__ idx, T* __restrict__ out, int cols) {
  const long long o = blockIdx.x;
  const T* s = inp + static_cast<long long>(idx[o]) * cols;
  T* d = out + o * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) d[c] = s[c];
}

// K4b / K6f: out[t, :] (+)= sum over the slots s of token t of w(s) * y[out_idx[s], :], w = 1 (K4b) or the routing weight.
template <typename T>
__global__ void co_reduce_kernel(const T* __restrict__ y, const T* __restrict__ weights, int K,
                                 const int* __restrict__ cum_ep, const int* __restrict__ sel_idx,
                                 const int* __restrict__ out_idx, T* __restrict__ out, int cols, int accumulate) {
  const int t = blockIdx.x;
  const int s0 = cum_ep[t], s1 = cum_ep[t + 1];
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float acc = accumulate ? to_f(out[static_cast<long long>(t) * cols + c]) : 0.f;
    for (int s = s0; s < s1; ++s) {
      const float w = weights ? to_f(weights[static_cast<long long>(t) * K + sel_idx[s]]) : 1.f;
      acc += w * to_f(y[static_cast<long long>(out_idx[s]) * cols + c]);
    }
    out[static_cast<long long>(t) * cols + c] = from_f<T>(acc);
  }
}

// K6b: one warp per slot: dY[row] = w[t, k] * dOut[t], dw[t, k] = <Y[row], dOut[t]>.
template <typename T>
__global__ void co_reduce_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ y, const T* __restrict__ weights,
                                     int K, const int* __restrict__ cum_ep, const int* __restrict__ sel_idx,
                                     const int* __restrict__ out_idx, T* __restrict__ dy, T* __restrict__ dw, int Tn,
                                     int cols) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= Tn) return;
  const int t = warp;
  for (int s = cum_ep[t]; s < cum_ep[t + 1]; ++s) {
    const int k = sel_idx[s];
    const long long row = out_idx[s];
    const float w = to_f(weights[static_cast<long long>(t) * K + k]);
    float dot = 0.f;
    for (int c = lane; c < cols; c += 32) {
      const float g = to_f(dout[static_cast<long long>(t) * cols + c]);
      dot += to_f(y[row * cols + c]) * g;
      dy[row * cols + c] = from_f<T>(w * g);
    }
    dot = warp_sum(dot);
    if (lane == 0) dw[static_cast<long long>(t) * K + k] = from_f<T>(dot);
  }
}

// K7: final[indices[c], :] += expert_output[c, :].  Atomic, so repeated indices are summed (in no fixed order).
__global__ void co_index_add_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, const int* __restrict__ idx,
                                        int cols) {
  const long long c = blockIdx.x;
  float* d = dst + static_cast<long long>(idx[c]) * cols;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) atomicAdd(d + i, src[c * cols + i]);
}
__global__ void co_index_add_bf16_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                         const int* __restrict__ idx, int cols) {
  const long long c = blockIdx.x;
  __nv_bfloat162* d = reinterpret_cast<__nv_bfloat162*>(dst + static_cast<long long>(idx[c]) * cols);
  const __nv_bfloat162* s = reinterpret_cast<const __nv_bfloat162*>(src + c * cols);
  for (int i = threadIdx.x; i < cols / 2; i += blockDim.x) atomicAdd(d + i, s[i]);
}

}  // namespace olb

using namespace olb;

static inline bool launch_ok() { return cudaGetLastError() == cudaSuccess; }

extern "C" int olb_co_partial_token_counts(const int* sel, int T, int K, int e_start, int E_loc, int* partial,
                                           int* counts_ep, cudaStream_t stream) {
  if (T <= 0 || E_loc <= 0) return 0;
  const int TH = (T + TOK_PER_BLOCK - 1) / TOK_PER_BLOCK;
  co_partial_counts_kernel<<<(TH + 127) / 128, 128, 0, stream>>>(sel, T, K, e_start, E_loc, TH, partial, counts_ep);
  return launch_ok() ? 0 : -2;
}

extern "C" int olb_co_input_output_indices(const int* sel, int T, int K, int e_start, int E_loc, const int* partial_cum,
                                           int* incr, const int* cum_ep, int* sel_idx, int* in_idx, int* out_idx,
                                           cudaStream_t stream) {
  if (T <= 0 || E_loc <= 0) return 0;
  const int TH = (T + TOK_PER_BLOCK - 1) / TOK_PER_BLOCK;
  co_indices_kernel<<<(TH + 127) / 128, 128, 0, stream>>>(sel, T, K, e_start, E_loc, TH, partial_cum, incr, cum_ep, sel_idx,
                                                         in_idx, out_idx);
  return launch_ok() ? 0 : -2;
}

extern "C" int olb_co_index_gather(const void* inp, const int* idx, void* out, int rows_out, int cols, int fp32,
                                   cudaStream_t stream) {
  if (rows_out <= 0) return 0;
  if (fp32)
    co_gather_kernel<float><<<rows_out, 256, 0, stream>>>(static_cast<const float*>(inp), idx, static_cast<float*>(out), cols);
  else
    co_gather_kernel<__nv_bfloat16><<<rows_out, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(inp), idx,
                                                                   static_cast<__nv_bfloat16*>(out), cols);
  return launch_ok() ? 0 : -2;
}

extern "C" int olb_co_reduce(const void* y, const void* weights, int K, const int* cum_ep, const int* sel_idx,
                             const int* out_idx, void* out, int T, int cols, int accumulate, int fp32,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  if (fp32)
    co_reduce_kernel<float><<<T, 256, 0, stream>>>(static_cast<const float*>(y), static_cast<const float*>(weights), K,
                                                   cum_ep, sel_idx, out_idx, static_cast<float*>(out), cols, accumulate);
  else
    co_reduce_kernel<__nv_bfloat16><<<T, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y),
                                                           static_cast<const __nv_bfloat16*>(weights), K, cum_ep, sel_idx,
                                                           out_idx, static_cast<__nv_bfloat16*>(out), cols, accumulate);
  return launch_ok() ? 0 : -2;
}

extern "C" int olb_co_reduce_bwd(const void* dout, const void* y, const void* weights, int K, const int* cum_ep,
                                 const int* sel_idx, const int* out_idx, void* dy, void* dw, int T, int cols, int fp32,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  const int blocks = (T * 32 + 255) / 256;
  if (fp32)
    co_reduce_bwd_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(dout), static_cast<const float*>(y),
                                                            static_cast<const float*>(weights), K, cum_ep, sel_idx, out_idx,
                                                            static_cast<float*>(dy), static_cast<float*>(dw), T, cols);
  else
    co_reduce_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(y),
        static_cast<const __nv_bfloat16*>(weights), K, cum_ep, sel_idx, out_idx, static_cast<__nv_bfloat16*>(dy),
        static_cast<__nv_bfloat16*>(dw), T, cols);
  return launch_ok() ? 0 : -2;
}

extern "C" int olb_co_index_add(const void* src, void* dst, const int* idx, int rows, int cols, int fp32,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (fp32) {
    co_index_add_f32_kernel<<<rows, 256, 0, stream>>>(static_cast<const float*>(src), static_cast<float*>(dst), idx, cols);
  } else {
    if (cols % 2) return -1;
    co_index_add_bf16_kernel<<<rows, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src),
                                                       static_cast<__nv_bfloat16*>(dst), idx, cols);
  }
  return launch_ok() ? 0 : -2;
}
