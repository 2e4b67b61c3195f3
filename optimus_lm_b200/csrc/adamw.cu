// Fused mixed-precision AdamW on one flat shard, plus the deterministic sum-of-squares used
// for the global gradient norm.
//
// Update rule of the reference optimizers (optimus/optimizers.py:193-205, 455-479):
//   g    = fp32(grad) * grad_scale * clip_coef
//   m    = b1*m + (1-b1)*g ;  v = b2*v + (1-b2)*g*g
//   p32 -= lr * (m/(1-b1^t)) / (sqrt(v/(1-b2^t)) + eps)
//   p32 += p32 * (-lr*wd)            (decay on the already updated weight)
//   p16  = cast(p32)
// The reference runs ~12 elementwise ATen kernels with temporaries per 128Mi-element chunk;
// this is one pass that reads grad, m, v, master and writes m, v, master, param.
#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

constexpr int SUMSQ_THREADS = 256;
constexpr long long SUMSQ_ELEMS_PER_BLOCK = 1 << 16;

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float s[32];
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  if (threadIdx.x < 32) {
    r = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.f;
    r = warp_sum(r);
  }
  __syncthreads();
  return r;
}

// Fixed mapping of elements to blocks and a fixed reduction tree -> bitwise reproducible.
__global__ void __launch_bounds__(SUMSQ_THREADS)
sumsq_partial_kernel(const void* __restrict__ grad, int grad_fp32, long long n, float grad_scale,
                     float* __restrict__ partial) {
  const long long begin = static_cast<long long>(blockIdx.x) * SUMSQ_ELEMS_PER_BLOCK;
  const long long end = min(begin + SUMSQ_ELEMS_PER_BLOCK, n);
  float acc = 0.f;
  if (grad_fp32) {
    const float* g = static_cast<const float*>(grad);
    for (long long i = begin + threadIdx.x; i < end; i += SUMSQ_THREADS) {
      const float x = g[i] * grad_scale;
      acc += x * x;
    }
  } else {
    const __nv_bfloat16* g = static_cast<const __nv_bfloat16*>(grad);
    // 16-byte vectors when the block start is aligned (it is: 2^16 elements per block)
    const bool aligned = (reinterpret_cast<uintptr_t>(g + begin) & 15) == 0;
    long long i = begin;
    if (aligned) {
      const long long nvec = (end - begin) / 8;
      const uint4* gv = reinterpret_cast<const uint4*>(g + begin);
      for (long long j = threadIdx.x; j < nvec; j += SUMSQ_THREADS) {
        const uint4 v = gv[j];
        float2 a;
        a = unpack_bf16(v.x); acc += (a.x * grad_scale) * (a.x * grad_scale) + (a.y * grad_scale) * (a.y * grad_scale);
        a = unpack_bf16(v.y); acc += (a.x * grad_scale) * (a.x * grad_scale) + (a.y * grad_scale) * (a.y * grad_scale);
        a = unpack_bf16(v.z); acc += (a.x * grad_scale) * (a.x * grad_scale) + (a.y * grad_scale) * (a.y * grad_scale);
        a = unpack_bf16(v.w); acc += (a.x * grad_scale) * (a.x * grad_scale) + (a.y * grad_scale) * (a.y * grad_scale);
      }
      i = begin + nvec * 8;
    }
    for (i += threadIdx.x; i < end; i += SUMSQ_THREADS) {
      const float x = __bfloat162float(g[i]) * grad_scale;
      acc += x * x;
    }
  }
  const float r = block_sum(acc);
  if (threadIdx.x == 0) partial[blockIdx.x] = r;
}

__global__ void sum_finalize_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out,
                                    int accumulate) {
  // single block, fixed order
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc += partial[i];
  const float r = block_sum(acc);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + r : r;
}

template <bool GRAD_FP32, bool PARAM_FP32>
__global__ void __launch_bounds__(256)
adamw_kernel(const void* __restrict__ grad_, float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
             void* __restrict__ param_, long long n, olb_adamw_hparams hp, const float* __restrict__ clip_coef_dev,
             float* __restrict__ norm_partial) {
  // norm_partial (optional, one float per block): sum of squares of the scaled, unclipped gradients this block saw -
  // the gradient norm as a by-product of the update's own read of the gradients (fixed grid and strides: the same
  // bits every run), for the steps in which the update does not depend on the norm.
  float sq = 0.f;
  const float clip = clip_coef_dev ? *clip_coef_dev : 1.f;
  const float gs = hp.grad_scale * clip;
  const float inv_bc1 = 1.f / hp.bias_correction1;
  const float inv_bc2 = 1.f / hp.bias_correction2;
  const float decay = -hp.lr * hp.weight_decay;
  const long long nvec = n / 4;
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < nvec;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g[4];
    if (GRAD_FP32) {
      const float4 t = reinterpret_cast<const float4*>(grad_)[j];
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    } else {
      const uint2 t = reinterpret_cast<const uint2*>(grad_)[j];
      float2 a = unpack_bf16(t.x), b = unpack_bf16(t.y);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    }
    float4 mm = reinterpret_cast<float4*>(m)[j];
    float4 vv = reinterpret_cast<float4*>(v)[j];
    float4 pp = reinterpret_cast<float4*>(master)[j];
    float* mp = reinterpret_cast<float*>(&mm);
    float* vp = reinterpret_cast<float*>(&vv);
    float* p = reinterpret_cast<float*>(&pp);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = g[k] * gs;
      sq += (g[k] * hp.grad_scale) * (g[k] * hp.grad_scale);
      mp[k] = hp.beta1 * mp[k] + (1.f - hp.beta1) * gk;
      vp[k] = hp.beta2 * vp[k] + (1.f - hp.beta2) * gk * gk;
      if (!hp.skip_weight_update) {
        const float mhat = mp[k] * inv_bc1;
        const float vhat = vp[k] * inv_bc2;
        float w = p[k] - hp.lr * mhat / (sqrtf(vhat) + hp.eps);
        w += w * decay;
        p[k] = w;
      }
    }
    reinterpret_cast<float4*>(m)[j] = mm;
    reinterpret_cast<float4*>(v)[j] = vv;
    reinterpret_cast<float4*>(master)[j] = pp;
    if (PARAM_FP32) {
      if (param_ != static_cast<void*>(master)) reinterpret_cast<float4*>(param_)[j] = pp;
    } else {
      uint2 o;
      o.x = pack_bf16(p[0], p[1]);
      o.y = pack_bf16(p[2], p[3]);
      reinterpret_cast<uint2*>(param_)[j] = o;
    }
  }
  if (norm_partial != nullptr) {
    const float r = block_sum(sq);
    if (threadIdx.x == 0) norm_partial[blockIdx.x] = r;
  }
}

}  // namespace olb

using namespace olb;

extern "C" int olb_sumsq_blocks(long long n) {
  return static_cast<int>((n + SUMSQ_ELEMS_PER_BLOCK - 1) / SUMSQ_ELEMS_PER_BLOCK);
}

extern "C" int olb_sumsq_partial(const void* grad, int grad_fp32, long long n, float grad_scale, float* partial,
                                 cudaStream_t stream) {
  if (n <= 0) return 0;
  sumsq_partial_kernel<<<olb_sumsq_blocks(n), SUMSQ_THREADS, 0, stream>>>(grad, grad_fp32, n, grad_scale, partial);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_sum_finalize(const float* partial, int nparts, float* out, int accumulate, cudaStream_t stream) {
  sum_finalize_kernel<<<1, 1024, 0, stream>>>(partial, nparts, out, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_adamw_blocks(long long n) {
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}

extern "C" int olb_adamw_step(const void* grad, int grad_fp32, float* master, float* m, float* v, void* param,
                              int param_fp32, long long n, const olb_adamw_hparams* hp, const float* clip_coef_dev,
                              float* norm_partial, cudaStream_t stream) {
  if (n <= 0) return 0;
  // shards are multiples of 512 elements and 16-byte aligned
  if (n % 4 || (reinterpret_cast<uintptr_t>(grad) & 7) || (reinterpret_cast<uintptr_t>(master) & 15) ||
      (reinterpret_cast<uintptr_t>(m) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (reinterpret_cast<uintptr_t>(param) & 7))
    return -1;
  if (grad_fp32 && (reinterpret_cast<uintptr_t>(grad) & 15)) return -1;
  if (param_fp32 && (reinterpret_cast<uintptr_t>(param) & 15)) return -1;
  const int grid = olb_adamw_blocks(n);
  if (grad_fp32 && param_fp32)
    adamw_kernel<true, true><<<grid, 256, 0, stream>>>(grad, master, m, v, param, n, *hp, clip_coef_dev, norm_partial);
  else if (grad_fp32)
    adamw_kernel<true, false><<<grid, 256, 0, stream>>>(grad, master, m, v, param, n, *hp, clip_coef_dev, norm_partial);
  else if (param_fp32)
    adamw_kernel<false, true><<<grid, 256, 0, stream>>>(grad, master, m, v, param, n, *hp, clip_coef_dev, norm_partial);
  else
    adamw_kernel<false, false><<<grid, 256, 0, stream>>>(grad, master, m, v, param, n, *hp, clip_coef_dev, norm_partial);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
