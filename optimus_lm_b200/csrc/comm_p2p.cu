// Kernels that move data between GPUs themselves, over NVLink peer memory (plain P2P loads and
// stores on pointers into other GPUs' symmetric buffers), fused with the computation that
// consumes or produces the data.  No TMA cluster fan-out and no library kernels touch peer
// memory here.
//
//   symm_barrier        : all ranks of a group rendezvous through signal words in each other's
//                         memory (bounded spin; on timeout the status word gets ST_TIMEOUT_PEER).
//   ep_gather_rows      : expert-parallel dispatch fused with the expert permutation - every rank
//                         pulls exactly the token rows routed to its experts straight from the
//                         owners' activation buffers into its expert-grouped GEMM operand.
//   ep_combine          : expert-parallel combine - every rank pulls the K expert outputs of each
//                         of its tokens from the ranks that own the experts and reduces them in
//                         fp32 (the reference reduce-scatters a [EP*T, H] buffer,
//                         optimus/models/olmoe/modeling_olmoe.py:338-341).
//   ep_pull_dweights    : routing-weight gradients back to the tokens' rank.
//   rs_adamw            : (plain peer loads / stores, or multimem.ld_reduce / multimem.st through the NVSwitch when the
//                         buffers have a multicast address)
//                         gradient reduce-scatter fused with the bf16->fp32 cast, the 1/N scaling,
//                         the gradient-norm partial, the sharded AdamW update and the parameter
//                         all-gather (updated bf16 parameters are stored into every peer's flat
//                         parameter buffer).  Replaces reduce_scatter_tensor + ~12 elementwise
//                         kernels + all_gather_into_tensor of optimus/optimizers.py:354-494.
//   pull_reduce_rows    : reduce-scatter epilogue of a row-parallel GEMM: sum the peers' partial
//                         outputs of this rank's row block.
#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

constexpr int MAX_PEERS = 16;
struct PeerPtrs {
  const void* p[MAX_PEERS];
};
struct PeerPtrsMut {
  void* p[MAX_PEERS];
};

__device__ __forceinline__ void st_release_sys_u32(unsigned* addr, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* addr) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// signal layout on every rank: pad[channel * MAX_PEERS + src_rank]
__global__ void symm_barrier_kernel(PeerPtrsMut pads, int my_rank, int n, int channel, unsigned epoch, int* status,
                                    unsigned long long wait_limit_ns) {
  const int peer = threadIdx.x;
  if (peer >= n) return;
  __threadfence_system();
  unsigned* remote = static_cast<unsigned*>(pads.p[peer]) + channel * MAX_PEERS + my_rank;
  st_release_sys_u32(remote, epoch);
  const unsigned* mine = static_cast<const unsigned*>(pads.p[my_rank]) + channel * MAX_PEERS + peer;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  // epochs only grow; a peer may already be one barrier ahead
  const unsigned long long limit = wait_limit_ns ? wait_limit_ns : WAIT_LIMIT_NS;
  while (static_cast<int>(ld_acquire_sys_u32(mine) - epoch) < 0) {
    if ((++spins & 63u) == 0 && globaltimer_ns() - t0 > limit) {
      if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER);
      break;
    }
    __nanosleep(spins < 64u ? 20u : 200u);  // back off: the polls cross NVLink or at least the L2
  }
}

// All-gather of the routing metadata by stores: this rank's [count] indices and weights go to slot `off` of every
// peer's gathered arrays (a few hundred KB per rank and layer; the barrier that follows publishes them together with
// the token rows).
__global__ void ep_publish_meta_kernel(PeerPtrsMut idx_all, PeerPtrsMut w_all, const int* __restrict__ idx,
                                       const float* __restrict__ w, int n, long long off, long long count) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = idx[i];
    const float f = w[i];
    for (int p = 0; p < n; ++p) {
      static_cast<int*>(idx_all.p[p])[off + i] = v;
      static_cast<float*>(w_all.p[p])[off + i] = f;
    }
  }
}

// out[t,:] = sum_k recv[t,k,:] in fp32, fixed k order: the owner's side of the combine after the expert outputs
// were pushed into its receive buffer.
__global__ void __launch_bounds__(256)
sum_slots_kernel(const __nv_bfloat16* __restrict__ recv, int T, int K, int cols, __nv_bfloat16* __restrict__ out) {
  const long long nvec = static_cast<long long>(T) * (cols / 8);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / (cols / 8);
    const int c = static_cast<int>(i - t * (cols / 8)) * 8;
    const __nv_bfloat16* base = recv + (t * K) * cols + c;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += 8) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        v[j] = (k0 + j < K) ? *reinterpret_cast<const uint4*>(base + static_cast<long long>(k0 + j) * cols) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float2 a;
        a = unpack_bf16(v[j].x); acc[0] += a.x; acc[1] += a.y;
        a = unpack_bf16(v[j].y); acc[2] += a.x; acc[3] += a.y;
        a = unpack_bf16(v[j].z); acc[4] += a.x; acc[5] += a.y;
        a = unpack_bf16(v[j].w); acc[6] += a.x; acc[7] += a.y;
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]);
    o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]);
    o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + t * cols + c) = o;
  }
}

// out[row,:] = peer_x[g / T][(g % T), :] with g = src_of[row]; padding rows -> 0.  One warp per row; a lane keeps up
// to eight 16-byte loads in flight, so that few resident warps saturate NVLink and the kernel can run underneath a
// GEMM (the grid is capped well below the SMs' thread capacity).  `blk_range` (optional, device) restricts the rows to
// the 128-row blocks [blk_range[0], blk_range[1]).
__global__ void __launch_bounds__(256)
ep_gather_rows_kernel(PeerPtrs peer_x, int T, const int* __restrict__ src_of, const int* __restrict__ meta,
                      const int* __restrict__ blk_range, __nv_bfloat16* __restrict__ out, int cap, int cols) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int row_begin = 0, row_end = min(meta[0] * 128, cap);
  if (blk_range) {
    row_begin = blk_range[0] * 128;
    row_end = min(row_end, blk_range[1] * 128);
  }
  const int vec = cols / 8;  // 16-byte vectors per row
  for (int row = row_begin + blockIdx.x * 8 + warp; row < row_end; row += gridDim.x * 8) {
    const int g = src_of[row];
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * cols);
    if (g >= 0) {
      const int r = g / T, t = g - r * T;
      const uint4* s = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(peer_x.p[r]) +
                                                      static_cast<long long>(t) * cols);
      for (int c0 = 0; c0 < vec; c0 += 256) {
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = c0 + i * 32 + lane;
          if (c < vec) v[i] = s[c];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = c0 + i * 32 + lane;
          if (c < vec) dst[c] = v[i];
        }
      }
    } else {
      for (int c = lane; c < vec; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

// rows[t,k] = peer_row_of[d][(my_rank*T + t)*K + k], d = idx[t,k] / E_loc: where each of my routed pairs
// landed in the owner's expert-grouped layout (-1 if it was dropped there).
__global__ void ep_resolve_rows_kernel(PeerPtrs peer_row_of, const int* __restrict__ idx, int my_rank, int T, int K,
                                       int E_loc, int* __restrict__ rows) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= static_cast<long long>(T) * K) return;
  const int d = idx[i] / E_loc;
  rows[i] = static_cast<const int*>(peer_row_of.p[d])[static_cast<long long>(my_rank) * T * K + i];
}

// out[t,:] = sum_k peer_y[d][rows[t,k], :],  d = idx[t,k] / E_loc  (fp32 accumulation, fixed k order).
__global__ void __launch_bounds__(256)
ep_combine_kernel(PeerPtrs peer_y, const int* __restrict__ rows, const int* __restrict__ idx, int T, int K, int E_loc,
                  __nv_bfloat16* __restrict__ out, int cols) {
  __shared__ int s_rank[32];
  __shared__ int s_row[32];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < K) {
      s_rank[threadIdx.x] = idx[static_cast<long long>(t) * K + threadIdx.x] / E_loc;
      s_row[threadIdx.x] = rows[static_cast<long long>(t) * K + threadIdx.x];
    }
    __syncthreads();
    for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int k0 = 0; k0 < K; k0 += 8) {  // up to eight peer loads in flight per thread, summed in fixed k order
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int k = k0 + i;
          v[i] = make_uint4(0, 0, 0, 0);
          if (k < K && s_row[k] >= 0)
            v[i] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(peer_y.p[s_rank[k]]) +
                                                   static_cast<long long>(s_row[k]) * cols + c);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float2 a;
          a = unpack_bf16(v[i].x); acc[0] += a.x; acc[1] += a.y;
          a = unpack_bf16(v[i].y); acc[2] += a.x; acc[3] += a.y;
          a = unpack_bf16(v[i].z); acc[4] += a.x; acc[5] += a.y;
          a = unpack_bf16(v[i].w); acc[6] += a.x; acc[7] += a.y;
        }
      }
      uint4 o;
      o.x = pack_bf16(acc[0], acc[1]);
      o.y = pack_bf16(acc[2], acc[3]);
      o.z = pack_bf16(acc[4], acc[5]);
      o.w = pack_bf16(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * cols + c) = o;
    }
  }
}

// dw[t,k] = peer_dw[d][(my_rank*T + t)*K + k]  (0 when the pair was dropped on the destination)
__global__ void ep_pull_dweights_kernel(PeerPtrs peer_dw, const int* __restrict__ idx, int my_rank, int T, int K,
                                        int E_loc, float* __restrict__ dw) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= static_cast<long long>(T) * K) return;
  const int d = idx[i] / E_loc;
  dw[i] = static_cast<const float*>(peer_dw.p[d])[static_cast<long long>(my_rank) * T * K + i];
}

// out[r,:] = sum_p peer_partial[p][(row0 + r), :]   (fp32 accumulation, fixed peer order)
__global__ void __launch_bounds__(256)
pull_reduce_rows_kernel(PeerPtrs peer_partial, int n, long long row0, int rows, int cols, long long ld,
                        __nv_bfloat16* __restrict__ out) {
  const long long nvec = static_cast<long long>(rows) * (cols / 8);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / (cols / 8);
    const int c = static_cast<int>(i - r * (cols / 8)) * 8;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int p = 0; p < n; ++p) {
      const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(peer_partial.p[p]) +
                                                      (row0 + r) * ld + c);
      float2 a;
      a = unpack_bf16(v.x); acc[0] += a.x; acc[1] += a.y;
      a = unpack_bf16(v.y); acc[2] += a.x; acc[3] += a.y;
      a = unpack_bf16(v.z); acc[4] += a.x; acc[5] += a.y;
      a = unpack_bf16(v.w); acc[6] += a.x; acc[7] += a.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]);
    o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]);
    o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + r * cols + c) = o;
  }
}

// Fused gradient reduce-scatter + AdamW + parameter all-gather on this rank's shard
// [shard_off, shard_off + n_elems) of the flat buffers.  peer_grad / peer_param: the flat bf16
// buffers of all ranks of the group.  mode 0: only the norm partial of the reduced, scaled
// gradient; mode 1: update (+ norm partial).
constexpr long long RS_ELEMS_PER_BLOCK = 1 << 15;

// NVLS forms (MC): `mc_grad` / `mc_param` are the buffers' multicast addresses (the same offsets reach every rank's
// copy through the NVSwitch).  One multimem.ld_reduce returns the sum over all ranks of eight bf16 gradients
// (fp32 accumulation in the switch, rounded to bf16 as a bf16 reduce-scatter would), one multimem.st delivers the
// eight updated parameters to every rank: 16 bytes cross this GPU's links once per direction instead of n - 1 times.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st_bf16x8(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

template <bool MC>
__global__ void __launch_bounds__(256)
rs_adamw_kernel(PeerPtrs peer_grad, PeerPtrsMut peer_param, int n, long long shard_off, long long n_elems,
                float* __restrict__ master, float* __restrict__ m, float* __restrict__ v, olb_adamw_hparams hp,
                const float* __restrict__ clip_coef_dev, float* __restrict__ norm_partial, int mode,
                const __nv_bfloat16* mc_grad, __nv_bfloat16* mc_param, const long long* __restrict__ local_only,
                int n_local_only, int my_rank) {
  __shared__ float s_red[8];
  const long long begin = static_cast<long long>(blockIdx.x) * RS_ELEMS_PER_BLOCK;
  const long long end = min(begin + RS_ELEMS_PER_BLOCK, n_elems);
  const float clip = (mode == 1 && clip_coef_dev) ? *clip_coef_dev : 1.f;
  const float inv_bc1 = 1.f / hp.bias_correction1, inv_bc2 = 1.f / hp.bias_correction2;
  const float decay = -hp.lr * hp.weight_decay;
  float sq = 0.f;
  // NVLS: a reduced load makes a round trip through the switch, so four of them are issued ahead of their use
  constexpr int MC_DEPTH = 4;
  uint4 pre[MC_DEPTH];
  if constexpr (MC) {
#pragma unroll
    for (int u = 0; u < MC_DEPTH; ++u) {
      const long long j = begin + threadIdx.x * 8 + static_cast<long long>(u) * 256 * 8;
      if (j < end) pre[u] = multimem_ld_reduce_bf16x8(mc_grad + shard_off + j);
    }
  }
  int turn = 0;
  for (long long i = begin + threadIdx.x * 8; i < end; i += 256 * 8, ++turn) {
    float g[8];
    if constexpr (MC) {
      uint4 t = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < MC_DEPTH; ++u)
        if ((turn % MC_DEPTH) == u) {
          t = pre[u];
          const long long j = i + static_cast<long long>(MC_DEPTH) * 256 * 8;   // refill this slot for a later turn
          if (j < end) pre[u] = multimem_ld_reduce_bf16x8(mc_grad + shard_off + j);
        }
      float2 a;
      a = unpack_bf16(t.x); g[0] = a.x; g[1] = a.y;
      a = unpack_bf16(t.y); g[2] = a.x; g[3] = a.y;
      a = unpack_bf16(t.z); g[4] = a.x; g[5] = a.y;
      a = unpack_bf16(t.w); g[6] = a.x; g[7] = a.y;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = 0.f;
      for (int p = 0; p < n; ++p) {
        const uint4 t = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(peer_grad.p[p]) + shard_off + i);
        float2 a;
        a = unpack_bf16(t.x); g[0] += a.x; g[1] += a.y;
        a = unpack_bf16(t.y); g[2] += a.x; g[3] += a.y;
        a = unpack_bf16(t.z); g[4] += a.x; g[5] += a.y;
        a = unpack_bf16(t.w); g[6] += a.x; g[7] += a.y;
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      g[k] *= hp.grad_scale;
      sq += g[k] * g[k];
    }
    if (mode == 0) continue;
    float4 m0 = *reinterpret_cast<float4*>(m + i), m1 = *reinterpret_cast<float4*>(m + i + 4);
    float4 v0 = *reinterpret_cast<float4*>(v + i), v1 = *reinterpret_cast<float4*>(v + i + 4);
    float4 p0 = *reinterpret_cast<float4*>(master + i), p1 = *reinterpret_cast<float4*>(master + i + 4);
    float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = g[k] * clip;
      mm[k] = hp.beta1 * mm[k] + (1.f - hp.beta1) * gk;
      vv[k] = hp.beta2 * vv[k] + (1.f - hp.beta2) * gk * gk;
      if (!hp.skip_weight_update) {
        float w = pp[k] - hp.lr * (mm[k] * inv_bc1) / (sqrtf(vv[k] * inv_bc2) + hp.eps);
        w += w * decay;
        pp[k] = w;
      }
    }
    *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(m + i + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
    *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(v + i + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
    *reinterpret_cast<float4*>(master + i) = make_float4(pp[0], pp[1], pp[2], pp[3]);
    *reinterpret_cast<float4*>(master + i + 4) = make_float4(pp[4], pp[5], pp[6], pp[7]);
    uint4 o;
    o.x = pack_bf16(pp[0], pp[1]);
    o.y = pack_bf16(pp[2], pp[3]);
    o.z = pack_bf16(pp[4], pp[5]);
    o.w = pack_bf16(pp[6], pp[7]);
    // ranges whose all-gather is left to the first GEMM that consumes the weight: the update stays on this GPU
    bool keep_local = false;
    if (n_local_only > 0) {
      const long long pos = shard_off + i;
      int lo = 0, hi = n_local_only;   // last range with start <= pos
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (local_only[2 * mid] <= pos) lo = mid + 1; else hi = mid;
      }
      keep_local = lo > 0 && pos < local_only[2 * (lo - 1) + 1];
    }
    if (keep_local) {
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(peer_param.p[my_rank]) + shard_off + i) = o;
    } else if constexpr (MC) {
      multimem_st_bf16x8(mc_param + shard_off + i, o);
    } else {
      for (int p = 0; p < n; ++p)
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(peer_param.p[p]) + shard_off + i) = o;
    }
  }
  // deterministic block reduction of the norm partial
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += s_red[w];
    norm_partial[blockIdx.x] = t;
  }
}

}  // namespace olb

using namespace olb;

static inline PeerPtrs to_peers(const void* const* ptrs, int n) {
  PeerPtrs p{};
  for (int i = 0; i < n && i < MAX_PEERS; ++i) p.p[i] = ptrs[i];
  return p;
}
static inline PeerPtrsMut to_peers_mut(void* const* ptrs, int n) {
  PeerPtrsMut p{};
  for (int i = 0; i < n && i < MAX_PEERS; ++i) p.p[i] = ptrs[i];
  return p;
}

// Streaming multiprocessors of the current device (the side-stream kernels size their grids from it).
static int sm_count() {
  constexpr int MAX_DEVICES = 64;
  static int cached[MAX_DEVICES] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

extern "C" int olb_symm_barrier(void* const* pads, int my_rank, int n, int channel, unsigned epoch, int* status,
                                unsigned long long wait_limit_ns, cudaStream_t stream) {
  if (n > MAX_PEERS || n < 1) return -1;
  symm_barrier_kernel<<<1, 32, 0, stream>>>(to_peers_mut(pads, n), my_rank, n, channel, epoch, status, wait_limit_ns);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_ep_publish_meta(void* const* idx_all, void* const* w_all, int n, const int* idx, const float* w,
                                   long long off, long long count, cudaStream_t stream) {
  if (n > MAX_PEERS || n < 1) return -1;
  if (count <= 0) return 0;
  long long blocks = (count + 255) / 256;
  if (blocks > sm_count() * 4) blocks = sm_count() * 4;
  ep_publish_meta_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(to_peers_mut(idx_all, n), to_peers_mut(w_all, n), idx,
                                                                       w, n, off, count);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_sum_slots(const void* recv, int T, int K, int cols, void* out, cudaStream_t stream) {
  if (cols % 8 || K < 1) return -1;
  if (T <= 0) return 0;
  long long blocks = (static_cast<long long>(T) * (cols / 8) + 255) / 256;
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  sum_slots_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(recv), T, K, cols,
                                                                 static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_ep_gather_rows(const void* const* peer_x, int n, int T, const int* src_of, const int* meta,
                                  const int* blk_range, void* out, int cap, int cols, cudaStream_t stream) {
  if (n > MAX_PEERS || cols % 8) return -1;
  int grid = (cap + 7) / 8;
  if (grid > sm_count() * 3) grid = sm_count() * 3;  // leaves room for a GEMM CTA on every SM
  if (grid <= 0) return 0;
  ep_gather_rows_kernel<<<grid, 256, 0, stream>>>(to_peers(peer_x, n), T, src_of, meta, blk_range,
                                                  static_cast<__nv_bfloat16*>(out), cap, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_ep_resolve_rows(const void* const* peer_row_of, int n, const int* idx, int my_rank, int T, int K,
                                   int E_loc, int* rows, cudaStream_t stream) {
  if (n > MAX_PEERS) return -1;
  const long long total = static_cast<long long>(T) * K;
  if (total <= 0) return 0;
  ep_resolve_rows_kernel<<<static_cast<int>((total + 255) / 256), 256, 0, stream>>>(to_peers(peer_row_of, n), idx,
                                                                                     my_rank, T, K, E_loc, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_ep_combine(const void* const* peer_y, int n, const int* rows, const int* idx, int T, int K,
                              int E_loc, void* out, int cols, cudaStream_t stream) {
  if (n > MAX_PEERS || cols % 8 || K > 32) return -1;
  if (T <= 0) return 0;
  // at most three 256-thread blocks per SM: leaves room for a GEMM CTA running on the main stream meanwhile
  const int grid = T < sm_count() * 3 ? T : sm_count() * 3;
  ep_combine_kernel<<<grid, 256, 0, stream>>>(to_peers(peer_y, n), rows, idx, T, K, E_loc,
                                              static_cast<__nv_bfloat16*>(out), cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_ep_pull_dweights(const void* const* peer_dw, int n, const int* idx, int my_rank, int T, int K,
                                    int E_loc, float* dw, cudaStream_t stream) {
  if (n > MAX_PEERS) return -1;
  const long long total = static_cast<long long>(T) * K;
  if (total <= 0) return 0;
  ep_pull_dweights_kernel<<<static_cast<int>((total + 255) / 256), 256, 0, stream>>>(to_peers(peer_dw, n), idx, my_rank,
                                                                                      T, K, E_loc, dw);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_pull_reduce_rows(const void* const* peer_partial, int n, long long row0, int rows, int cols,
                                    long long ld, void* out, cudaStream_t stream) {
  if (n > MAX_PEERS || cols % 8 || ld % 8) return -1;
  if (rows <= 0) return 0;
  long long blocks = (static_cast<long long>(rows) * (cols / 8) + 255) / 256;
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  pull_reduce_rows_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(to_peers(peer_partial, n), n, row0, rows, cols,
                                                                        ld, static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_rs_adamw_blocks(long long n_elems) {
  return static_cast<int>((n_elems + RS_ELEMS_PER_BLOCK - 1) / RS_ELEMS_PER_BLOCK);
}

extern "C" int olb_rs_adamw(const void* const* peer_grad, void* const* peer_param, int n, long long shard_off,
                            long long n_elems, float* master, float* m, float* v, const olb_adamw_hparams* hp,
                            const float* clip_coef_dev, float* norm_partial, int mode, cudaStream_t stream) {
  return olb_rs_adamw_ex(peer_grad, peer_param, n, shard_off, n_elems, master, m, v, hp, clip_coef_dev, norm_partial, mode,
                         nullptr, nullptr, nullptr, 0, 0, stream);
}

extern "C" int olb_rs_adamw_mc(const void* const* peer_grad, void* const* peer_param, int n, long long shard_off,
                               long long n_elems, float* master, float* m, float* v, const olb_adamw_hparams* hp,
                               const float* clip_coef_dev, float* norm_partial, int mode, const void* mc_grad,
                               void* mc_param, cudaStream_t stream) {
  return olb_rs_adamw_ex(peer_grad, peer_param, n, shard_off, n_elems, master, m, v, hp, clip_coef_dev, norm_partial, mode,
                         mc_grad, mc_param, nullptr, 0, 0, stream);
}

// dst[i] = src[i] for `bytes` bytes (multiple of 16, both 16-byte aligned); src may be another GPU's memory.
__global__ void __launch_bounds__(256) peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long vecs) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

extern "C" int olb_peer_copy(const void* src, void* dst, long long bytes, cudaStream_t stream) {
  if ((bytes % 16) || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)) return -1;
  if (bytes <= 0) return 0;
  long long blocks = (bytes / 16 + 255) / 256;
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  peer_copy_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst),
                                                                 bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_rs_adamw_ex(const void* const* peer_grad, void* const* peer_param, int n, long long shard_off,
                               long long n_elems, float* master, float* m, float* v, const olb_adamw_hparams* hp,
                               const float* clip_coef_dev, float* norm_partial, int mode, const void* mc_grad,
                               void* mc_param, const long long* local_only, int n_local_only, int my_rank,
                               cudaStream_t stream) {
  if (n > MAX_PEERS || (n_elems % 8) || (shard_off % 8)) return -1;
  if (n_local_only > 0 && (local_only == nullptr || my_rank < 0 || my_rank >= n)) return -1;
  if ((mc_grad == nullptr) != (mc_param == nullptr)) return -1;
  if ((reinterpret_cast<uintptr_t>(mc_grad) | reinterpret_cast<uintptr_t>(mc_param)) & 15) return -1;
  if (n_elems <= 0) return 0;
  if (mc_grad)
    rs_adamw_kernel<true><<<olb_rs_adamw_blocks(n_elems), 256, 0, stream>>>(
        to_peers(peer_grad, n), to_peers_mut(peer_param, n), n, shard_off, n_elems, master, m, v, *hp, clip_coef_dev,
        norm_partial, mode, static_cast<const __nv_bfloat16*>(mc_grad), static_cast<__nv_bfloat16*>(mc_param), local_only,
        n_local_only, my_rank);
  else
    rs_adamw_kernel<false><<<olb_rs_adamw_blocks(n_elems), 256, 0, stream>>>(
        to_peers(peer_grad, n), to_peers_mut(peer_param, n), n, shard_off, n_elems, master, m, v, *hp, clip_coef_dev,
        norm_partial, mode, nullptr, nullptr, local_only, n_local_only, my_rank);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
