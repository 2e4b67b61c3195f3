// RMSNorm / non-parametric LayerNorm, forward and backward, bf16 data with fp32 statistics.
// One warp owns one row; 16-byte vector accesses; the row is read twice (second read is an
// L1/L2 hit).  The weight gradient is reduced deterministically: each warp keeps its own
// fp32 accumulator row in shared memory, blocks write partial rows to a scratch buffer and
// a second kernel sums the partials in a fixed order.
//
// Reference semantics (optimus/models/olmoe/modeling_olmoe.py:93-104): the normalised value
// is rounded to the input dtype before it is multiplied by the weight; OLMo's LayerNorm has
// no affine parameters and eps 1e-5 (optimus/models/olmo/modeling_olmo.py:19-30).
#include <mutex>

#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

constexpr int NORM_WARPS = 4;
constexpr int NORM_THREADS = NORM_WARPS * 32;

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  float2 a;
  a = unpack_bf16(v.x); f[0] = a.x; f[1] = a.y;
  a = unpack_bf16(v.y); f[2] = a.x; f[3] = a.y;
  a = unpack_bf16(v.z); f[4] = a.x; f[5] = a.y;
  a = unpack_bf16(v.w); f[6] = a.x; f[7] = a.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16(f[0], f[1]);
  v.y = pack_bf16(f[2], f[3]);
  v.z = pack_bf16(f[4], f[5]);
  v.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, int cols, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + warp;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * cols;
  __nv_bfloat16* yr = y + row * cols;
  float ss = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    float f[8];
    load8(xr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / cols + eps);
  if (lane == 0 && rstd) rstd[row] = r;
  for (int c = lane * 8; c < cols; c += 256) {
    float f[8], g[8];
    load8(xr + c, f);
    if (w) load8(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float n = round_bf16(f[i] * r);
      f[i] = w ? n * g[i] : n;
    }
    store8(yr + c, f);
  }
}

// h = a + b (rounded to bf16, the residual stream) and y = rmsnorm(h) * w in one pass over the rows.
__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ y,
                       float* __restrict__ rstd, int rows, int cols, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + warp;
  if (row >= rows) return;
  const __nv_bfloat16* ar = a + row * cols;
  const __nv_bfloat16* br = b + row * cols;
  __nv_bfloat16* hr = h + row * cols;
  __nv_bfloat16* yr = y + row * cols;
  float ss = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    float fa[8], fb[8];
    load8(ar + c, fa);
    load8(br + c, fb);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      fa[i] = round_bf16(fa[i] + fb[i]);
      ss += fa[i] * fa[i];
    }
    store8(hr + c, fa);
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / cols + eps);
  if (lane == 0 && rstd) rstd[row] = r;
  __syncwarp();
  for (int c = lane * 8; c < cols; c += 256) {
    float f[8], g[8];
    load8(hr + c, f);  // this lane's own stores
    if (w) load8(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float n = round_bf16(f[i] * r);
      f[i] = w ? n * g[i] : n;
    }
    store8(yr + c, f);
  }
}

// dx = r * (dn - n * mean(dn * n)) (+ dres), dn = dy * w, n = x * r.  dw partial = sum_rows dy * n.
// `dres` (optional) is the gradient that reaches x along the residual path; adding it here saves the separate
// accumulation pass.
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int rows, int cols,
                   const __nv_bfloat16* __restrict__ dres = nullptr) {
  extern __shared__ float s_dw[];  // [NORM_WARPS][cols] when dw_partial != NULL
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* my_dw = s_dw + static_cast<size_t>(warp) * cols;
  if (dw_partial) {
    for (int c = lane; c < cols; c += 32) my_dw[c] = 0.f;
  }
  __syncwarp();
  for (long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + warp; row < rows;
       row += static_cast<long long>(gridDim.x) * NORM_WARPS) {
    const __nv_bfloat16* xr = x + row * cols;
    const __nv_bfloat16* dyr = dy + row * cols;
    const float r = rstd[row];
    float dot = 0.f;
    for (int c = lane * 8; c < cols; c += 256) {
      float fx[8], fd[8], fw[8];
      load8(xr + c, fx);
      load8(dyr + c, fd);
      if (w) load8(w + c, fw);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float n = fx[i] * r;
        const float dn = w ? fd[i] * fw[i] : fd[i];
        dot += dn * n;
        if (dw_partial) my_dw[c + i] += fd[i] * round_bf16(n);
      }
    }
    dot = warp_sum(dot) / cols;
    for (int c = lane * 8; c < cols; c += 256) {
      float fx[8], fd[8], fw[8], o[8];
      load8(xr + c, fx);
      load8(dyr + c, fd);
      if (w) load8(w + c, fw);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float n = fx[i] * r;
        const float dn = w ? fd[i] * fw[i] : fd[i];
        o[i] = r * (dn - n * dot);
      }
      if (dres) {
        float fr[8];
        load8(dres + row * cols + c, fr);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = round_bf16(o[i]) + fr[i];  // the sum of two bf16 gradients, as autograd adds them
      }
      store8(dx + row * cols + c, o);
    }
  }
  if (dw_partial) {
    __syncthreads();
    for (int c = threadIdx.x; c < cols; c += NORM_THREADS) {
      float s = 0.f;
#pragma unroll
      for (int wi = 0; wi < NORM_WARPS; ++wi) s += s_dw[static_cast<size_t>(wi) * cols + c];
      dw_partial[static_cast<size_t>(blockIdx.x) * cols + c] = s;
    }
  }
}

// Same math for cols = NCH * 256 <= 2048 with the row held in registers: x and dy are read from global memory
// once, and each lane keeps the weight-gradient sums of its own columns in registers over all rows of its warp
// (no shared-memory read-modify-write per element); the warps' sums meet in shared memory once at the end.
template <int NCH>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_reg_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                       __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int rows,
                       const __nv_bfloat16* __restrict__ dres = nullptr) {
  constexpr int cols = NCH * 256;
  __shared__ __align__(16) __nv_bfloat16 s_w[cols];
  __shared__ float s_dw[NORM_WARPS][cols + 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (w) {
    for (int c = threadIdx.x * 8; c < cols; c += NORM_THREADS * 8)
      *reinterpret_cast<uint4*>(s_w + c) = *reinterpret_cast<const uint4*>(w + c);
  }
  __syncthreads();
  float dw_acc[NCH][8];
#pragma unroll
  for (int k = 0; k < NCH; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) dw_acc[k][i] = 0.f;
  const float inv_cols = 1.f / cols;
  for (long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + warp; row < rows;
       row += static_cast<long long>(gridDim.x) * NORM_WARPS) {
    uint4 vx[NCH], vd[NCH];
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      vx[k] = *reinterpret_cast<const uint4*>(x + row * cols + k * 256 + lane * 8);
      vd[k] = *reinterpret_cast<const uint4*>(dy + row * cols + k * 256 + lane * 8);
    }
    const float r = rstd[row];
    const float2 r2 = make_float2(r, r);
    // two elements per instruction (packed fp32): the products and sums are the same fused operations as in the
    // scalar form, so the results do not change
    float2 dot2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const uint32_t ux[4] = {vx[k].x, vx[k].y, vx[k].z, vx[k].w}, ud[4] = {vd[k].x, vd[k].y, vd[k].z, vd[k].w};
      uint4 vw = make_uint4(0, 0, 0, 0);
      if (w) vw = *reinterpret_cast<const uint4*>(s_w + k * 256 + lane * 8);
      const uint32_t uw[4] = {vw.x, vw.y, vw.z, vw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fd = unpack_bf16(ud[i]);
        const float2 n2 = mul2(unpack_bf16(ux[i]), r2);
        const float2 d2 = w ? mul2(fd, unpack_bf16(uw[i])) : fd;
        dot2 = fma2(d2, n2, dot2);
        const float2 nr = unpack_bf16(pack_bf16(n2.x, n2.y));  // the normalised value as the forward rounded it
        const float2 acc = fma2(fd, nr, make_float2(dw_acc[k][2 * i], dw_acc[k][2 * i + 1]));
        dw_acc[k][2 * i] = acc.x;
        dw_acc[k][2 * i + 1] = acc.y;
      }
    }
    const float dot = warp_sum(dot2.x + dot2.y) * inv_cols;
    const float2 ndot2 = make_float2(-dot, -dot);
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const uint32_t ux[4] = {vx[k].x, vx[k].y, vx[k].z, vx[k].w}, ud[4] = {vd[k].x, vd[k].y, vd[k].z, vd[k].w};
      uint4 vw = make_uint4(0, 0, 0, 0);
      if (w) vw = *reinterpret_cast<const uint4*>(s_w + k * 256 + lane * 8);
      const uint32_t uw[4] = {vw.x, vw.y, vw.z, vw.w};
      uint4 vr = make_uint4(0, 0, 0, 0);
      if (dres) vr = *reinterpret_cast<const uint4*>(dres + row * cols + k * 256 + lane * 8);
      const uint32_t ur[4] = {vr.x, vr.y, vr.z, vr.w};
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fd = unpack_bf16(ud[i]);
        const float2 n2 = mul2(unpack_bf16(ux[i]), r2);
        const float2 d2 = w ? mul2(fd, unpack_bf16(uw[i])) : fd;
        const float2 g2 = mul2(r2, fma2(n2, ndot2, d2));
        o[i] = pack_bf16(g2.x, g2.y);
        if (dres) {
          const float2 s2 = add2(unpack_bf16(o[i]), unpack_bf16(ur[i]));  // dx rounded first, as two kernels would
          o[i] = pack_bf16(s2.x, s2.y);
        }
      }
      *reinterpret_cast<uint4*>(dx + row * cols + k * 256 + lane * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  if (dw_partial) {
#pragma unroll
    for (int k = 0; k < NCH; ++k)
#pragma unroll
      for (int i = 0; i < 8; ++i) s_dw[warp][k * 256 + lane * 8 + i] = dw_acc[k][i];
    __syncthreads();
    for (int c = threadIdx.x; c < cols; c += NORM_THREADS) {
      float s = 0.f;
#pragma unroll
      for (int wi = 0; wi < NORM_WARPS; ++wi) s += s_dw[wi][c];
      dw_partial[static_cast<size_t>(blockIdx.x) * cols + c] = s;
    }
  }
}

__global__ void colsum_finalize_kernel(const float* __restrict__ partial, int nparts, int cols, void* dw, int dw_fp32,
                                       int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[static_cast<size_t>(p) * cols + c];
  if (dw_fp32) {
    float* o = static_cast<float*>(dw);
    o[c] = accumulate ? o[c] + s : s;
  } else {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(dw);
    o[c] = __float2bfloat16_rn(accumulate ? __bfloat162float(o[c]) + s : s);
  }
}

__global__ void __launch_bounds__(NORM_THREADS)
layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
                     float* __restrict__ rstd, int rows, int cols, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + warp;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * cols;
  float s = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    float f[8];
    load8(xr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += f[i];
  }
  const float mu = warp_sum(s) / cols;
  float ss = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    float f[8];
    load8(xr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += (f[i] - mu) * (f[i] - mu);
  }
  const float r = rsqrtf(warp_sum(ss) / cols + eps);
  if (lane == 0) {
    mean[row] = mu;
    rstd[row] = r;
  }
  for (int c = lane * 8; c < cols; c += 256) {
    float f[8];
    load8(xr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = (f[i] - mu) * r;
    store8(y + row * cols + c, f);
  }
}

// dx = r * (dy - mean(dy) - n * mean(dy * n))
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const float* __restrict__ mean, const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                     int rows, int cols) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + warp;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * cols;
  const __nv_bfloat16* dyr = dy + row * cols;
  const float mu = mean[row], r = rstd[row];
  float s1 = 0.f, s2 = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    float fx[8], fd[8];
    load8(xr + c, fx);
    load8(dyr + c, fd);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s1 += fd[i];
      s2 += fd[i] * (fx[i] - mu) * r;
    }
  }
  s1 = warp_sum(s1) / cols;
  s2 = warp_sum(s2) / cols;
  for (int c = lane * 8; c < cols; c += 256) {
    float fx[8], fd[8], o[8];
    load8(xr + c, fx);
    load8(dyr + c, fd);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = r * (fd[i] - s1 - (fx[i] - mu) * r * s2);
    store8(dx + row * cols + c, o);
  }
}

// The shared-memory opt-in of rmsnorm_bwd_kernel is a per-device attribute: raise it once on each device that
// runs a wide row (the caller's device is current).
static bool raise_bwd_smem_limit() {
  constexpr int MAX_DEVICES = 64;
  static std::mutex mu;
  static bool raised[MAX_DEVICES] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (!raised[dev]) {
    if (cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    raised[dev] = true;
  }
  return true;
}

// Launch the register-resident backward when `cols` is one of its widths.  Returns false when it is not.
static bool launch_bwd_reg(const __nv_bfloat16* pdy, const __nv_bfloat16* px, const __nv_bfloat16* pw, const float* rstd,
                           __nv_bfloat16* pdx, float* dw_partial, int rows, int cols, int nb, cudaStream_t stream,
                           const __nv_bfloat16* dres = nullptr) {
  switch (cols) {
    case 256: rmsnorm_bwd_reg_kernel<1><<<nb, NORM_THREADS, 0, stream>>>(pdy, px, pw, rstd, pdx, dw_partial, rows, dres); return true;
    case 512: rmsnorm_bwd_reg_kernel<2><<<nb, NORM_THREADS, 0, stream>>>(pdy, px, pw, rstd, pdx, dw_partial, rows, dres); return true;
    case 1024: rmsnorm_bwd_reg_kernel<4><<<nb, NORM_THREADS, 0, stream>>>(pdy, px, pw, rstd, pdx, dw_partial, rows, dres); return true;
    case 2048: rmsnorm_bwd_reg_kernel<8><<<nb, NORM_THREADS, 0, stream>>>(pdy, px, pw, rstd, pdx, dw_partial, rows, dres); return true;
    default: return false;
  }
}

}  // namespace olb

using namespace olb;

extern "C" int olb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps,
                               cudaStream_t stream) {
  if (cols % 8) return -1;
  if (rows <= 0) return 0;
  rmsnorm_fwd_kernel<<<(rows + NORM_WARPS - 1) / NORM_WARPS, NORM_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), rstd,
      rows, cols, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_rmsnorm_bwd_blocks(int rows) {
  int nb = (rows + NORM_WARPS - 1) / NORM_WARPS;
  return nb < 296 ? (nb < 1 ? 1 : nb) : 296;
}

extern "C" int olb_add_rmsnorm_fwd(const void* a, const void* b, const void* w, void* h, void* y, float* rstd, int rows,
                                   int cols, float eps, cudaStream_t stream) {
  if (cols % 8) return -1;
  if (rows <= 0) return 0;
  add_rmsnorm_fwd_kernel<<<(rows + NORM_WARPS - 1) / NORM_WARPS, NORM_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), static_cast<const __nv_bfloat16*>(w),
      static_cast<__nv_bfloat16*>(h), static_cast<__nv_bfloat16*>(y), rstd, rows, cols, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                               float* dw_partial, int rows, int cols, cudaStream_t stream) {
  return olb_rmsnorm_bwd_res(dy, x, w, rstd, dx, dw_partial, nullptr, rows, cols, stream);
}

extern "C" int olb_rmsnorm_bwd_res(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                   float* dw_partial, const void* dres, int rows, int cols, cudaStream_t stream) {
  if (cols % 8) return -1;
  if (rows <= 0) return 0;
  const int nb = olb_rmsnorm_bwd_blocks(rows);
  if (launch_bwd_reg(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                     static_cast<const __nv_bfloat16*>(w), rstd, static_cast<__nv_bfloat16*>(dx), dw_partial, rows, cols,
                     nb, stream, static_cast<const __nv_bfloat16*>(dres)))
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  const size_t smem = dw_partial ? sizeof(float) * NORM_WARPS * cols : 0;
  if (smem > 200 * 1024) return -3;
  if (smem > 48 * 1024 && !raise_bwd_smem_limit()) return -4;
  rmsnorm_bwd_kernel<<<nb, NORM_THREADS, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      rstd, static_cast<__nv_bfloat16*>(dx), dw_partial, rows, cols, static_cast<const __nv_bfloat16*>(dres));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_colsum_finalize(const float* partial, int nparts, int cols, void* dw, int dw_fp32, int accumulate,
                                   cudaStream_t stream) {
  colsum_finalize_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(partial, nparts, cols, dw, dw_fp32, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_layernorm_fwd(const void* x, void* y, float* mean, float* rstd, int rows, int cols, float eps,
                                 cudaStream_t stream) {
  if (cols % 8) return -1;
  if (rows <= 0) return 0;
  layernorm_fwd_kernel<<<(rows + NORM_WARPS - 1) / NORM_WARPS, NORM_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), mean, rstd, rows, cols, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_layernorm_bwd(const void* dy, const void* x, const float* mean, const float* rstd, void* dx,
                                 int rows, int cols, cudaStream_t stream) {
  if (cols % 8) return -1;
  if (rows <= 0) return 0;
  layernorm_bwd_kernel<<<(rows + NORM_WARPS - 1) / NORM_WARPS, NORM_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), mean, rstd,
      static_cast<__nv_bfloat16*>(dx), rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the RMSNorm backward (see olb_noalloc.h).  The per-block partial
// sums of the weight gradient go to a device array that is part of the library image.
#include "olb_noalloc.h"

namespace olb {

static __device__ __align__(256) float g_noalloc_dw_partial[OLB_NOALLOC_MAX_PARTS * OLB_NOALLOC_MAX_COLS];

// Device code may name the array directly; only host code needs its address.
__global__ void colsum_finalize_static_kernel(int nparts, int cols, void* dw, int dw_fp32) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += g_noalloc_dw_partial[static_cast<size_t>(p) * cols + c];
  if (dw_fp32)
    static_cast<float*>(dw)[c] = s;
  else
    static_cast<__nv_bfloat16*>(dw)[c] = __float2bfloat16_rn(s);
}

constexpr int NOALLOC_MAX_DEVICES = 64;
struct NoallocDeviceState {
  float* scratch = nullptr;  // device address of g_noalloc_dw_partial on this device
};
static NoallocDeviceState g_noalloc_state[NOALLOC_MAX_DEVICES];
static std::mutex g_noalloc_mutex;

// One-time set-up per device, with that device current.  In host code the array's name is only
// a handle for the runtime, not a device address, so the address is looked up explicitly.
static int noalloc_setup(int dev, bool need_big_smem, float** scratch) {
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  NoallocDeviceState& st = g_noalloc_state[dev];
  if (st.scratch == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_dw_partial) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return OLB_NOALLOC_ERR_SYMBOL;
    }
    st.scratch = ptr;
  }
  if (need_big_smem && !raise_bwd_smem_limit()) return OLB_NOALLOC_ERR_SYMBOL;
  *scratch = st.scratch;
  return OLB_NOALLOC_OK;
}

}  // namespace olb

extern "C" const char* olb_noalloc_strerror(int code) {
  switch (code) {
    case OLB_NOALLOC_OK: return "ok";
    case OLB_NOALLOC_ERR_BAD_COLS: return "cols must be a multiple of 8";
    case OLB_NOALLOC_ERR_LAUNCH: return "kernel launch failed";
    case OLB_NOALLOC_ERR_TOO_LARGE: return "cols exceeds OLB_NOALLOC_MAX_COLS (8192): the built-in scratch array is too small";
    case OLB_NOALLOC_ERR_SYMBOL: return "could not resolve the device address of the built-in scratch array";
    case OLB_NOALLOC_ERR_DEVICE: return "no usable current CUDA device";
    case OLB_NOALLOC_ERR_NULL: return "dy, x, rstd, dx and dw must not be null";
    default: return "unknown error";
  }
}

extern "C" int olb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                       void* dw, int dw_fp32, int rows, int cols, cudaStream_t stream) {
  if (cols % 8) return OLB_NOALLOC_ERR_BAD_COLS;
  if (cols > OLB_NOALLOC_MAX_COLS) return OLB_NOALLOC_ERR_TOO_LARGE;
  if (rows <= 0) return OLB_NOALLOC_OK;
  if (!dy || !x || !rstd || !dx || !dw) return OLB_NOALLOC_ERR_NULL;  // the kernels would store through them
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return OLB_NOALLOC_ERR_DEVICE;
  const int nb = olb_rmsnorm_bwd_blocks(rows);  // <= OLB_NOALLOC_MAX_PARTS
  const bool reg = cols == 256 || cols == 512 || cols == 1024 || cols == 2048;  // widths of the register-resident kernel
  const size_t smem = sizeof(float) * NORM_WARPS * cols;
  float* scratch = nullptr;
  const int rc = noalloc_setup(dev, !reg && smem > 48 * 1024, &scratch);
  if (rc != OLB_NOALLOC_OK) return rc;
  if (!launch_bwd_reg(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<__nv_bfloat16*>(dx), scratch, rows, cols, nb,
                      stream))
    rmsnorm_bwd_kernel<<<nb, NORM_THREADS, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
        rstd, static_cast<__nv_bfloat16*>(dx), scratch, rows, cols);
  if (cudaGetLastError() != cudaSuccess) return OLB_NOALLOC_ERR_LAUNCH;
  colsum_finalize_static_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(nb, cols, dw, dw_fp32);
  return cudaGetLastError() == cudaSuccess ? OLB_NOALLOC_OK : OLB_NOALLOC_ERR_LAUNCH;
}
