// Embedding lookup and its deterministic backward, vocabulary-parallel capable.
//
// forward : out[t, :] = (v_start <= id[t] < v_start + rows) ? W[id[t] - v_start, :] : 0
//           (the reference masks out-of-range ids, looks up and zeroes the rows, then all-reduces over the
//            tensor-parallel group: optimus/models/common/parallel_modules.py:32-45)
// backward: dW[v, :] (+)= sum over the tokens with id == v of dy[t, :], in token order.  The ids arrive sorted
//           (stable) together with the permutation; the block standing on the first position of a run of equal
//           ids sums the run in fp32 and is the only writer of that row - no atomics, the same bits every run.
//           torch's embedding_dense_backward makes a dense gradient that autograd then adds into .grad; this one
//           accumulates straight into the gradient buffer.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                     __nv_bfloat16* __restrict__ out, int tokens, int cols, int v_start, int rows) {
  const int vec = cols / 8;
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    const long long id = ids[t] - v_start;
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(t) * cols);
    if (id >= 0 && id < rows) {
      const uint4* src = reinterpret_cast<const uint4*>(w + id * cols);
      for (int c = threadIdx.x; c < vec; c += blockDim.x) dst[c] = src[c];
    } else {
      for (int c = threadIdx.x; c < vec; c += blockDim.x) dst[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ perm,
                     const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dw, int tokens, int cols,
                     int v_start, int rows, long long padding_idx, int accumulate) {
  const int vec = cols / 8;
  for (int i = blockIdx.x; i < tokens; i += gridDim.x) {
    const long long id = sorted_ids[i];
    if (i > 0 && sorted_ids[i - 1] == id) continue;  // not the first position of its run
    const long long r = id - v_start;
    if (r < 0 || r >= rows || id == padding_idx) continue;
    int end = i + 1;
    while (end < tokens && sorted_ids[end] == id) ++end;
    for (int c = threadIdx.x; c < vec; c += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
      for (int j = i; j < end; ++j) {
        const uint4 v = *(reinterpret_cast<const uint4*>(dy + perm[j] * cols) + c);
        float2 a;
        a = unpack_bf16(v.x); acc[0] += a.x; acc[1] += a.y;
        a = unpack_bf16(v.y); acc[2] += a.x; acc[3] += a.y;
        a = unpack_bf16(v.z); acc[4] += a.x; acc[5] += a.y;
        a = unpack_bf16(v.w); acc[6] += a.x; acc[7] += a.y;
      }
      uint4* dst = reinterpret_cast<uint4*>(dw + r * cols) + c;
      if (accumulate) {
        const uint4 o = *dst;
        float2 a;
        a = unpack_bf16(o.x); acc[0] += a.x; acc[1] += a.y;
        a = unpack_bf16(o.y); acc[2] += a.x; acc[3] += a.y;
        a = unpack_bf16(o.z); acc[4] += a.x; acc[5] += a.y;
        a = unpack_bf16(o.w); acc[6] += a.x; acc[7] += a.y;
      }
      uint4 o;
      o.x = pack_bf16(acc[0], acc[1]);
      o.y = pack_bf16(acc[2], acc[3]);
      o.z = pack_bf16(acc[4], acc[5]);
      o.w = pack_bf16(acc[6], acc[7]);
      *dst = o;
    }
  }
}

}  // namespace olb

extern "C" int olb_embedding_fwd(const long long* ids, const void* w, void* out, int tokens, int cols, int v_start,
                                 int rows, cudaStream_t stream) {
  if (cols % 8) return -1;
  if (tokens <= 0) return 0;
  const int grid = tokens < 148 * 16 ? tokens : 148 * 16;
  olb::embedding_fwd_kernel<<<grid, 256, 0, stream>>>(ids, static_cast<const __nv_bfloat16*>(w),
                                                      static_cast<__nv_bfloat16*>(out), tokens, cols, v_start, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_embedding_bwd(const long long* sorted_ids, const long long* perm, const void* dy, void* dw, int tokens,
                                 int cols, int v_start, int rows, long long padding_idx, int accumulate,
                                 cudaStream_t stream) {
  if (cols % 8) return -1;
  if (tokens <= 0) return 0;
  const int grid = tokens < 148 * 16 ? tokens : 148 * 16;
  olb::embedding_bwd_kernel<<<grid, 256, 0, stream>>>(sorted_ids, perm, static_cast<const __nv_bfloat16*>(dy),
                                                      static_cast<__nv_bfloat16*>(dw), tokens, cols, v_start, rows,
                                                      padding_idx, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
