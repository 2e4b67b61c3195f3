// SwiGLU (forward / backward) and rotary embedding on bf16 data, 16-byte vector accesses.
// Reference ops: silu(gate)*up and its hand-written backward in
// optimus/models/common/moe.py:37-41,75-78,134-147; rotate-half RoPE in
// optimus/models/olmoe/modeling_olmoe.py:107-119 and the interleaved DeepSeek-V3 variant in
// optimus/models/deepseek_v3/rope_utils.py:79-91.
#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  float2 a;
  a = unpack_bf16(v.x); f[0] = a.x; f[1] = a.y;
  a = unpack_bf16(v.y); f[2] = a.x; f[3] = a.y;
  a = unpack_bf16(v.z); f[4] = a.x; f[5] = a.y;
  a = unpack_bf16(v.w); f[6] = a.x; f[7] = a.y;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16(f[0], f[1]);
  v.y = pack_bf16(f[2], f[3]);
  v.z = pack_bf16(f[4], f[5]);
  v.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ g, long long ldg, const __nv_bfloat16* __restrict__ u,
                                  long long ldu, __nv_bfloat16* __restrict__ act, long long ldact, long long rows,
                                  int cols) {
  const int vec_per_row = cols / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    float fg[8], fu[8], o[8];
    ld8(g + r * ldg + c, fg);
    ld8(u + r * ldu + c, fu);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      // silu in fp32, rounded to bf16 before the product like the eager reference
      const float s = fg[k] / (1.f + __expf(-fg[k]));
      o[k] = __bfloat162float(__float2bfloat16_rn(s)) * fu[k];
    }
    st8(act + r * ldact + c, o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dact, long long lddact,
                                  const __nv_bfloat16* __restrict__ g, long long ldg,
                                  const __nv_bfloat16* __restrict__ u, long long ldu, __nv_bfloat16* __restrict__ dg,
                                  long long lddg, __nv_bfloat16* __restrict__ du, long long lddu, long long rows,
                                  int cols) {
  const int vec_per_row = cols / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    float fd[8], fg[8], fu[8], og[8], ou[8];
    ld8(dact + r * lddact + c, fd);
    ld8(g + r * ldg + c, fg);
    ld8(u + r * ldu + c, fu);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sig = 1.f / (1.f + __expf(-fg[k]));
      const float silu = fg[k] * sig;
      ou[k] = fd[k] * silu;
      og[k] = fd[k] * fu[k] * (sig + silu * (1.f - sig));
    }
    st8(dg + r * lddg + c, og);
    st8(du + r * lddu + c, ou);
  }
}

// Half-rotate variant: one thread handles 8 consecutive "first half" elements and their 8
// partners; reads and writes touch the same addresses, so the update is safely in place.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, long long token_stride, int tokens, int heads, int head_dim,
                            int rot_dim, int seq_len, const float* __restrict__ cos_tab,
                            const float* __restrict__ sin_tab, int conj) {
  const int half = rot_dim / 2;
  const int vec_per_head = half / 8;
  const long long total = static_cast<long long>(tokens) * heads * vec_per_head;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vec_per_head);
    const long long th = i / vec_per_head;
    const int h = static_cast<int>(th % heads);
    const long long t = th / heads;
    const int pos = static_cast<int>(t % seq_len);
    __nv_bfloat16* base = x + t * token_stride + static_cast<long long>(h) * head_dim;
    const int j0 = v * 8;
    float a[8], b[8], oa[8], ob[8];
    ld8(base + j0, a);
    ld8(base + half + j0, b);
    const float* cr = cos_tab + static_cast<long long>(pos) * rot_dim;
    const float* sr = sin_tab + static_cast<long long>(pos) * rot_dim;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float c = cr[j0 + k];  // table columns j and j+half hold the same angle
      const float s = conj ? -sr[j0 + k] : sr[j0 + k];
      oa[k] = a[k] * c - b[k] * s;
      ob[k] = b[k] * c + a[k] * s;
    }
    st8(base + j0, oa);
    st8(base + half + j0, ob);
  }
}

// Interleaved variant (rot_dim <= 128): one thread owns a whole head because the
// de-interleave permutes positions.  Forward reads pairs (2j, 2j+1) and leaves the result in
// de-interleaved order; the backward (conj) maps gradients back to the interleaved order.
__global__ void rope_interleaved_kernel(__nv_bfloat16* __restrict__ x, long long token_stride, int tokens, int heads,
                                        int head_dim, int rot_dim, int seq_len, const float* __restrict__ cos_tab,
                                        const float* __restrict__ sin_tab, int conj) {
  const int half = rot_dim / 2;
  const long long total = static_cast<long long>(tokens) * heads;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int h = static_cast<int>(i % heads);
    const long long t = i / heads;
    const int pos = static_cast<int>(t % seq_len);
    __nv_bfloat16* base = x + t * token_stride + static_cast<long long>(h) * head_dim;
    const float* cr = cos_tab + static_cast<long long>(pos) * rot_dim;
    const float* sr = sin_tab + static_cast<long long>(pos) * rot_dim;
    float buf[128];
    for (int c = 0; c < rot_dim; c += 8) {
      float f[8];
      ld8(base + c, f);
#pragma unroll
      for (int k = 0; k < 8; ++k) buf[c + k] = f[k];
    }
    float out[128];
    for (int j = 0; j < half; ++j) {
      const float c = cr[j];
      if (!conj) {
        const float a = buf[2 * j], b = buf[2 * j + 1], s = sr[j];
        out[j] = a * c - b * s;
        out[half + j] = b * c + a * s;
      } else {
        const float a = buf[j], b = buf[half + j], s = -sr[j];
        out[2 * j] = a * c - b * s;
        out[2 * j + 1] = b * c + a * s;
      }
    }
    for (int c = 0; c < rot_dim; c += 8) {
      float f[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = out[c + k];
      st8(base + c, f);
    }
  }
}

// Expert-MLP activation with the routing weight folded in: act[row] = w(row) * silu(g) * u, where
// w(row) = weights[src_of[row], k_of[row]] (0 for padding rows).  Scaling before the down
// projection makes the combine an unweighted sum and removes the need to keep the expert
// outputs for the routing-weight gradient.  One warp per row.
__global__ void __launch_bounds__(256)
swiglu_rowscale_fwd_kernel(const __nv_bfloat16* __restrict__ g, long long ldg, const __nv_bfloat16* __restrict__ u,
                           long long ldu, const int* __restrict__ src_of, const int* __restrict__ k_of,
                           const float* __restrict__ weights, int K, const int* __restrict__ meta,
                           __nv_bfloat16* __restrict__ act, long long ldact, int cap, int cols) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nrows = min(meta[0] * 128, cap);
  for (int row = blockIdx.x * 8 + warp; row < nrows; row += gridDim.x * 8) {
    const int t = src_of[row];
    const float w = t >= 0 ? weights[static_cast<long long>(t) * K + k_of[row]] : 0.f;
    for (int c = lane * 8; c < cols; c += 256) {
      float fg[8], fu[8], o[8];
      if (t >= 0) {
        ld8(g + row * ldg + c, fg);
        ld8(u + row * ldu + c, fu);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = w * (fg[k] / (1.f + __expf(-fg[k]))) * fu[k];
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = 0.f;
      }
      st8(act + row * ldact + c, o);
    }
  }
}

// dg = dact * w * u * silu'(g); du = dact * w * silu(g); dweights[t,k] = <dact, silu(g) * u>.
__global__ void __launch_bounds__(256)
swiglu_rowscale_bwd_kernel(const __nv_bfloat16* __restrict__ dact, long long lddact,
                           const __nv_bfloat16* __restrict__ g, long long ldg, const __nv_bfloat16* __restrict__ u,
                           long long ldu, const int* __restrict__ src_of, const int* __restrict__ k_of,
                           const float* __restrict__ weights, int K, const int* __restrict__ meta,
                           __nv_bfloat16* __restrict__ dg, long long lddg, __nv_bfloat16* __restrict__ du,
                           long long lddu, float* __restrict__ dweights, int cap, int cols) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nrows = min(meta[0] * 128, cap);
  for (int row = blockIdx.x * 8 + warp; row < nrows; row += gridDim.x * 8) {
    const int t = src_of[row];
    const int kk = t >= 0 ? k_of[row] : 0;
    const float w = t >= 0 ? weights[static_cast<long long>(t) * K + kk] : 0.f;
    float dot = 0.f;
    for (int c = lane * 8; c < cols; c += 256) {
      float og[8], ou[8];
      if (t >= 0) {
        float fd[8], fg[8], fu[8];
        ld8(dact + row * lddact + c, fd);
        ld8(g + row * ldg + c, fg);
        ld8(u + row * ldu + c, fu);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float sig = 1.f / (1.f + __expf(-fg[k]));
          const float silu = fg[k] * sig;
          dot += fd[k] * silu * fu[k];
          ou[k] = fd[k] * w * silu;
          og[k] = fd[k] * w * fu[k] * (sig + silu * (1.f - sig));
        }
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) og[k] = ou[k] = 0.f;
      }
      st8(dg + row * lddg + c, og);
      st8(du + row * lddu + c, ou);
    }
    if (dweights && t >= 0) {
      dot = warp_sum(dot);
      if (lane == 0) dweights[static_cast<long long>(t) * K + kk] = dot;
    }
  }
}

}  // namespace olb

using namespace olb;

extern "C" int olb_swiglu_rowscale_fwd(const void* g, long long ldg, const void* u, long long ldu, const int* src_of,
                                       const int* k_of, const float* weights, int K, const int* meta, void* act,
                                       long long ldact, int cap, int cols, cudaStream_t stream) {
  if (cols % 8 || ldg % 8 || ldu % 8 || ldact % 8) return -1;
  int grid = (cap + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid <= 0) return 0;
  swiglu_rowscale_fwd_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(g), ldg,
                                                       static_cast<const __nv_bfloat16*>(u), ldu, src_of, k_of, weights,
                                                       K, meta, static_cast<__nv_bfloat16*>(act), ldact, cap, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_swiglu_rowscale_bwd(const void* dact, long long lddact, const void* g, long long ldg, const void* u,
                                       long long ldu, const int* src_of, const int* k_of, const float* weights, int K,
                                       const int* meta, void* dg, long long lddg, void* du, long long lddu,
                                       float* dweights, int cap, int cols, cudaStream_t stream) {
  if (cols % 8 || ldg % 8 || ldu % 8 || lddact % 8 || lddg % 8 || lddu % 8) return -1;
  int grid = (cap + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid <= 0) return 0;
  swiglu_rowscale_bwd_kernel<<<grid, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dact), lddact, static_cast<const __nv_bfloat16*>(g), ldg,
      static_cast<const __nv_bfloat16*>(u), ldu, src_of, k_of, weights, K, meta, static_cast<__nv_bfloat16*>(dg), lddg,
      static_cast<__nv_bfloat16*>(du), lddu, dweights, cap, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

static inline int grid_for(long long work, int threads) {
  long long b = (work + threads - 1) / threads;
  const long long cap = 148LL * 16;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

extern "C" int olb_swiglu_fwd(const void* g, long long ldg, const void* u, long long ldu, void* act, long long ldact,
                              long long rows, int cols, cudaStream_t stream) {
  if (cols % 8 || ldg % 8 || ldu % 8 || ldact % 8) return -1;
  if (rows <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for(rows * (cols / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(g), ldg, static_cast<const __nv_bfloat16*>(u), ldu,
      static_cast<__nv_bfloat16*>(act), ldact, rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_swiglu_bwd(const void* dact, long long lddact, const void* g, long long ldg, const void* u,
                              long long ldu, void* dg, long long lddg, void* du, long long lddu, long long rows,
                              int cols, cudaStream_t stream) {
  if (cols % 8 || ldg % 8 || ldu % 8 || lddact % 8 || lddg % 8 || lddu % 8) return -1;
  if (rows <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for(rows * (cols / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dact), lddact, static_cast<const __nv_bfloat16*>(g), ldg,
      static_cast<const __nv_bfloat16*>(u), ldu, static_cast<__nv_bfloat16*>(dg), lddg,
      static_cast<__nv_bfloat16*>(du), lddu, rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_rope_inplace(void* x, long long token_stride, int tokens, int heads, int head_dim, int rot_dim,
                                int seq_len, const float* cos_tab, const float* sin_tab, int interleaved, int conj,
                                cudaStream_t stream) {
  if (rot_dim % 16 || token_stride % 8 || head_dim % 8 || rot_dim > head_dim) return -1;
  if (tokens <= 0) return 0;
  if (interleaved) {
    if (rot_dim > 128) return -1;
    const long long work = static_cast<long long>(tokens) * heads;
    rope_interleaved_kernel<<<grid_for(work, 128), 128, 0, stream>>>(static_cast<__nv_bfloat16*>(x), token_stride, tokens,
                                                                     heads, head_dim, rot_dim, seq_len, cos_tab, sin_tab,
                                                                     conj);
  } else {
    const long long work = static_cast<long long>(tokens) * heads * (rot_dim / 16);
    rope_kernel<<<grid_for(work, 256), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(x), token_stride, tokens, heads,
                                                         head_dim, rot_dim, seq_len, cos_tab, sin_tab, conj);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
