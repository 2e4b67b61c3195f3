// MoE token permutation: index build, row gather, weighted combine and their backward.
//
// Replaces the reference's bucketed permutation chain K1-K6
// (pytorch_xpu_extensions/pcl.xpu.customops/csrc/ops/sparse_moe_block.sycl:56-532 and
// optimus/kernels/moe_nongemm.py:6-176), which needs two host synchronisations per layer
// (optimus/models/common/moe.py:397,514-520).  Here the whole index lives on the device:
//
//   build_index  : three launches (count -> scan -> place).  Placement is deterministic:
//                  rows of one expert are ordered by token id.  Every expert's row range is
//                  padded to a multiple of 128 so that a GEMM tile never spans two experts,
//                  and the scan kernel also emits the GEMM tile table and padded offsets.
//   gather_rows  : x_perm[row] = x[src_of[row]]          (padding rows are zero-filled)
//   combine      : out[t]      = sum_k w[t,k] * y[row_of[t,k]]   (fp32 accumulation)
//   combine_bwd  : dy[row]     = w[t,k] * dout[t],  dw[t,k] = <y[row], dout[t]>
#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

constexpr int IDX_THREADS = 256;  // one token per thread
constexpr int IDX_WARPS = IDX_THREADS / 32;
constexpr int MAX_E_LOC = 256;

// Per-thread bit set of the local experts its token selected (E_loc <= 256).
struct ExpertSet {
  unsigned w[8];
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = 0;
  }
  __device__ __forceinline__ void set(int e) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i == (e >> 5)) w[i] |= 1u << (e & 31);
  }
  __device__ __forceinline__ bool test(int e) const {
    unsigned v = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i == (e >> 5)) v = w[i];
    return (v >> (e & 31)) & 1u;
  }
};

__device__ __forceinline__ void load_set(const int* indices, int t, int T, int K, int e_start, int E_loc, ExpertSet& s) {
  s.clear();
  if (t < T) {
    for (int k = 0; k < K; ++k) {
      const int e = indices[static_cast<long long>(t) * K + k] - e_start;
      if (e >= 0 && e < E_loc) s.set(e);
    }
  }
}

// ws layout: block_counts[nblocks][E_loc] | block_offsets[nblocks][E_loc]
__global__ void __launch_bounds__(IDX_THREADS)
moe_count_kernel(const int* __restrict__ indices, int T, int K, int e_start, int E_loc, int* __restrict__ ws) {
  __shared__ int s_cnt[IDX_WARPS][MAX_E_LOC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * IDX_THREADS + threadIdx.x;
  ExpertSet set;
  load_set(indices, t, T, K, e_start, E_loc, set);
  for (int e = 0; e < E_loc; ++e) {
    const unsigned b = __ballot_sync(0xffffffffu, set.test(e));
    if (lane == 0) s_cnt[warp][e] = __popc(b);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E_loc; e += IDX_THREADS) {
    int c = 0;
#pragma unroll
    for (int w = 0; w < IDX_WARPS; ++w) c += s_cnt[w][e];
    ws[static_cast<long long>(blockIdx.x) * E_loc + e] = c;
  }
}

// One block; thread e scans expert e over the token blocks, then thread 0 lays out the experts.
__global__ void moe_scan_kernel(int* __restrict__ ws, int nblocks, int E_loc, int cap, int row_pad, int* __restrict__ meta,
                                int* __restrict__ offsets, int* __restrict__ counts, int* __restrict__ status) {
  __shared__ int s_total[MAX_E_LOC];
  __shared__ int s_off[MAX_E_LOC + 1];
  int* block_counts = ws;
  int* block_offsets = ws + static_cast<long long>(nblocks) * E_loc;
  for (int e = threadIdx.x; e < E_loc; e += blockDim.x) {
    int run = 0;
    for (int b = 0; b < nblocks; ++b) {
      block_offsets[static_cast<long long>(b) * E_loc + e] = run;
      run += block_counts[static_cast<long long>(b) * E_loc + e];
    }
    s_total[e] = run;
    counts[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    bool overflow = false;
    for (int e = 0; e < E_loc; ++e) {
      s_off[e] = off;
      int padded = (s_total[e] + row_pad - 1) / row_pad * row_pad;
      if (off + padded > cap) {
        overflow = true;
        padded = (cap - off) / row_pad * row_pad;  // clamp: the excess pairs of this expert are dropped
      }
      off += padded;
    }
    s_off[E_loc] = off;
    if (overflow && status) atomicCAS(status, 0, ST_OVERFLOW);
    meta[0] = off / 128;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E_loc; e += blockDim.x) offsets[e] = s_off[e];
  // tile table: block i belongs to the expert whose padded range contains row 128*i
  const int nrow_blocks = s_off[E_loc] / 128;
  for (int i = threadIdx.x; i < nrow_blocks; i += blockDim.x) {
    const int row = i * 128;
    int lo = 0, hi = E_loc - 1;
    while (lo < hi) {  // last e with s_off[e] <= row
      const int mid = (lo + hi + 1) >> 1;
      if (s_off[mid] <= row) lo = mid; else hi = mid - 1;
    }
    // skip experts with an empty range that share the same offset
    while (lo + 1 < E_loc && s_off[lo + 1] <= row) ++lo;
    meta[1 + i] = lo;
  }
}

__global__ void __launch_bounds__(IDX_THREADS)
moe_place_kernel(const int* __restrict__ indices, int T, int K, int e_start, int E_loc, const int* __restrict__ ws,
                 int nblocks, const int* __restrict__ offsets, int* __restrict__ row_of, int* __restrict__ src_of,
                 int* __restrict__ k_of) {
  __shared__ int s_cnt[IDX_WARPS][MAX_E_LOC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * IDX_THREADS + threadIdx.x;
  const int* block_offsets = ws + static_cast<long long>(nblocks) * E_loc + static_cast<long long>(blockIdx.x) * E_loc;
  ExpertSet set;
  load_set(indices, t, T, K, e_start, E_loc, set);
  for (int e = 0; e < E_loc; ++e) {
    const unsigned b = __ballot_sync(0xffffffffu, set.test(e));
    if (lane == 0) s_cnt[warp][e] = __popc(b);
  }
  __syncthreads();
  // Whole warps past the end may leave; a partially filled warp keeps all lanes for the
  // shuffles below and guards its writes instead.
  if (blockIdx.x * IDX_THREADS + warp * 32 >= T) return;
  const bool live = t < T;
  const unsigned lt_mask = (1u << lane) - 1u;
  for (int k = 0; k < K; ++k) {
    const int e = live ? indices[static_cast<long long>(t) * K + k] - e_start : -1;
    int row = -1;
    if (e >= 0 && e < E_loc) {
      // rank inside the expert: tokens of earlier blocks, earlier warps, earlier lanes
      int r = block_offsets[e];
      for (int w = 0; w < warp; ++w) r += s_cnt[w][e];
      // ballot over the lanes of this warp that selected e (any k); all lanes must take part,
      // so the ballot is recomputed without divergence below
      row = r;
    }
    // convergent ballot: every lane proposes its expert, peers test membership
    unsigned peers = 0;
    for (int src = 0; src < 32; ++src) {
      const int ee = __shfl_sync(0xffffffffu, e, src);
      const bool has = (ee >= 0 && ee < E_loc) ? set.test(ee) : false;
      const unsigned b = __ballot_sync(0xffffffffu, has);
      if (src == lane) peers = b;
    }
    if (!live) continue;
    if (row >= 0) {
      row += __popc(peers & lt_mask);
      const int limit = offsets[e + 1];
      row += offsets[e];
      if (row < limit) {
        row_of[static_cast<long long>(t) * K + k] = row;
        src_of[row] = t;
        k_of[row] = k;
      } else {
        row_of[static_cast<long long>(t) * K + k] = -1;
      }
    } else {
      row_of[static_cast<long long>(t) * K + k] = -1;
    }
  }
}

__global__ void fill_int_kernel(int* p, long long n, int v) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    p[i] = v;
}

// One warp per row, 16-byte vectors.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src_of,
                       const int* __restrict__ meta, __nv_bfloat16* __restrict__ out, int cap, int cols) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nrows = min(meta[0] * 128, cap);
  for (int row = blockIdx.x * 8 + warp; row < nrows; row += gridDim.x * 8) {
    const int src = src_of[row];
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * cols);
    if (src >= 0) {
      const uint4* s = reinterpret_cast<const uint4*>(x + static_cast<long long>(src) * cols);
      for (int c = lane; c < cols / 8; c += 32) dst[c] = s[c];
    } else {
      for (int c = lane; c < cols / 8; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

// One block per token; thread owns 8 columns at a time.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ row_of, const float* __restrict__ w,
                   __nv_bfloat16* __restrict__ out, int T, int K, int cols) {
  __shared__ int s_row[32];
  __shared__ float s_w[32];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < K) {
      s_row[threadIdx.x] = row_of[static_cast<long long>(t) * K + threadIdx.x];
      s_w[threadIdx.x] = w ? w[static_cast<long long>(t) * K + threadIdx.x] : 1.f;
    }
    __syncthreads();
    for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int k = 0; k < K; ++k) {
        const int row = s_row[k];
        if (row < 0) continue;
        const uint4 v = *reinterpret_cast<const uint4*>(y + static_cast<long long>(row) * cols + c);
        const float wk = s_w[k];
        float2 a;
        a = unpack_bf16(v.x); acc[0] += wk * a.x; acc[1] += wk * a.y;
        a = unpack_bf16(v.y); acc[2] += wk * a.x; acc[3] += wk * a.y;
        a = unpack_bf16(v.z); acc[4] += wk * a.x; acc[5] += wk * a.y;
        a = unpack_bf16(v.w); acc[6] += wk * a.x; acc[7] += wk * a.y;
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

// One warp per row.
__global__ void __launch_bounds__(256)
moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                       const int* __restrict__ src_of, const int* __restrict__ k_of, const int* __restrict__ meta,
                       const float* __restrict__ w, __nv_bfloat16* __restrict__ dy, float* __restrict__ dw, int cap,
                       int K, int cols) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nrows = min(meta[0] * 128, cap);
  for (int row = blockIdx.x * 8 + warp; row < nrows; row += gridDim.x * 8) {
    const int t = src_of[row];
    uint4* dst = reinterpret_cast<uint4*>(dy + static_cast<long long>(row) * cols);
    if (t < 0) {
      for (int c = lane; c < cols / 8; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int k = k_of[row];
    const float wk = w ? w[static_cast<long long>(t) * K + k] : 1.f;
    const uint4* g = reinterpret_cast<const uint4*>(dout + static_cast<long long>(t) * cols);
    const uint4* yy = y ? reinterpret_cast<const uint4*>(y + static_cast<long long>(row) * cols) : nullptr;
    float dot = 0.f;
    for (int c = lane; c < cols / 8; c += 32) {
      const uint4 gv = g[c];
      float2 g0 = unpack_bf16(gv.x), g1 = unpack_bf16(gv.y), g2 = unpack_bf16(gv.z), g3 = unpack_bf16(gv.w);
      if (yy) {
        const uint4 yv = yy[c];
        float2 y0 = unpack_bf16(yv.x), y1 = unpack_bf16(yv.y), y2 = unpack_bf16(yv.z), y3 = unpack_bf16(yv.w);
        dot += g0.x * y0.x + g0.y * y0.y + g1.x * y1.x + g1.y * y1.y + g2.x * y2.x + g2.y * y2.y + g3.x * y3.x +
               g3.y * y3.y;
      }
      uint4 o;
      o.x = pack_bf16(wk * g0.x, wk * g0.y);
      o.y = pack_bf16(wk * g1.x, wk * g1.y);
      o.z = pack_bf16(wk * g2.x, wk * g2.y);
      o.w = pack_bf16(wk * g3.x, wk * g3.y);
      dst[c] = o;
    }
    if (dw) {
      dot = warp_sum(dot);
      if (lane == 0) dw[static_cast<long long>(t) * K + k] = dot;
    }
  }
}

// dweights[src_of[row], k_of[row]] = sum_j partial[row, j] in a fixed order: the routing-weight gradients from the
// per-column-tile partials that the down projection's input-gradient launch left behind.
__global__ void moe_scatter_dweights_kernel(const float* __restrict__ partial, int nblk, const int* __restrict__ src_of,
                                            const int* __restrict__ k_of, const int* __restrict__ meta, int K,
                                            float* __restrict__ out, int cap) {
  const int nrows = min(meta[0] * 128, cap);
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < nrows; row += gridDim.x * blockDim.x) {
    const int t = src_of[row];
    if (t < 0) continue;
    float s = 0.f;
    for (int j = 0; j < nblk; ++j) s += partial[static_cast<long long>(row) * nblk + j];
    out[static_cast<long long>(t) * K + k_of[row]] = s;
  }
}

}  // namespace olb

using namespace olb;

extern "C" int olb_moe_scatter_dweights(const float* partial, int nblk, const int* src_of, const int* k_of, const int* meta,
                                        int K, float* out, int cap, cudaStream_t stream) {
  if (cap <= 0 || nblk <= 0) return 0;
  int grid = (cap + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  moe_scatter_dweights_kernel<<<grid, 256, 0, stream>>>(partial, nblk, src_of, k_of, meta, K, out, cap);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" long long olb_moe_ws_ints(int T, int E_loc) {
  const long long nblocks = (T + IDX_THREADS - 1) / IDX_THREADS;
  return 2 * nblocks * E_loc;
}

extern "C" int olb_moe_build_index(const int* indices, int T, int K, int e_start, int E_loc, int cap, int row_pad, int* ws,
                                   int* row_of, int* src_of, int* k_of, int* meta, int* offsets, int* counts,
                                   int* status, cudaStream_t stream) {
  if (E_loc > MAX_E_LOC || E_loc <= 0 || K > 32 || (row_pad != 128 && row_pad != 256) || cap % row_pad) return -1;
  if (T <= 0) return 0;
  const int nblocks = (T + IDX_THREADS - 1) / IDX_THREADS;
  fill_int_kernel<<<148, 256, 0, stream>>>(src_of, cap, -1);
  moe_count_kernel<<<nblocks, IDX_THREADS, 0, stream>>>(indices, T, K, e_start, E_loc, ws);
  moe_scan_kernel<<<1, 256, 0, stream>>>(ws, nblocks, E_loc, cap, row_pad, meta, offsets, counts, status);
  moe_place_kernel<<<nblocks, IDX_THREADS, 0, stream>>>(indices, T, K, e_start, E_loc, ws, nblocks, offsets, row_of,
                                                        src_of, k_of);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_moe_gather_rows(const void* x, const int* src_of, const int* meta, void* out, int cap, int cols,
                                   cudaStream_t stream) {
  if (cols % 8) return -1;
  int grid = (cap + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid <= 0) return 0;
  moe_gather_rows_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), src_of, meta,
                                                   static_cast<__nv_bfloat16*>(out), cap, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_moe_combine(const void* y, const int* row_of, const float* w, void* out, int T, int K, int cols,
                               cudaStream_t stream) {
  if (cols % 8 || K > 32) return -1;
  if (T <= 0) return 0;
  int grid = T < 148 * 16 ? T : 148 * 16;
  int threads = cols / 8 < 256 ? ((cols / 8 + 31) / 32) * 32 : 256;
  if (threads < 32) threads = 32;
  moe_combine_kernel<<<grid, threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), row_of, w,
                                                   static_cast<__nv_bfloat16*>(out), T, K, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int olb_moe_combine_bwd(const void* dout, const void* y, const int* src_of, const int* k_of,
                                   const int* meta, const float* w, void* dy, float* dw, int cap, int K, int cols,
                                   cudaStream_t stream) {
  if (cols % 8) return -1;
  int grid = (cap + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid <= 0) return 0;
  moe_combine_bwd_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(dout),
                                                   static_cast<const __nv_bfloat16*>(y), src_of, k_of, meta, w,
                                                   static_cast<__nv_bfloat16*>(dy), dw, cap, K, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
