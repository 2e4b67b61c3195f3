// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   C[M,N] (+)= A * B     fp32 accumulation in TMEM, bf16 (or fp32) output
//
// One persistent, warp-specialised kernel covers the dense projections (q/k/v/o, router,
// lm_head, dense MLP), their input/weight gradients, and the three grouped expert GEMMs of
// the MoE block:
//   * warp 0   : TMA producer - tiled bulk tensor loads into a 128B-swizzled smem ring
//   * warp 1   : one elected thread issues tcgen05.mma (UMMA 128 x BLOCK_N x 16) into one of
//                two TMEM accumulators and commits to mbarriers
//   * warps 2-5: epilogue - tcgen05.ld the accumulator (each warp owns 32 TMEM lanes), convert, stage the warp's
//                32 rows in 128B-swizzled shared memory and write them with cp.async.bulk.tensor stores (full
//                128-byte lines) while the next tile's main loop runs; accumulating epilogues (C += A*B) use
//                plain loads and stores.  With EPI_SWIGLU the tile holds 128 gate and 128 up columns of the same
//                expert and the epilogue writes gate | up (for the backward) and w(row) * silu(gate) * up.
//   * warps 6-9: only in the variants with a fused transfer (PeerArg<true>): all-gather of A's rows from the other
//                GPUs, gather of the routed token rows into the expert-grouped operand (expert-parallel dispatch, or
//                the local permutation on one GPU), or push of finished rows of C to their owners
// Each operand may be K-major (rows of K contiguous) or MN-major (rows of M/N contiguous),
// which gives NT / NN / TN / TT products without a transpose pass:
//   forward   Y  = X  W^T    A K-major,  B K-major
//   dgrad     dX = dY W      A K-major,  B MN-major
//   wgrad     dW = dY^T X    A MN-major, B MN-major
// Grouping modes (the per-expert row ranges live on the device, no host sync):
//   MODE_RAGGED_M : A/C rows are grouped by expert, each group padded to a multiple of 128
//                   rows; meta[0] = number of 128-row blocks in use, meta[1+i] = expert of
//                   block i.  B is the merged weight [E, rows_per_expert, ld].
//   MODE_RAGGED_K : per-expert wgrad, K runs over the expert's (padded) row range
//                   meta[e] .. meta[e+1]; C is [E, M, N].
// The reference computes these with torch.matmul per expert or with XPU Triton kernels
// (optimus/models/common/moe.py:43-215, optimus/kernels/merged_mlp_triton_kernels.py:8-269,
// optimus/kernels/grouped_linear_*.py).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;  // 64 bf16 = 128 bytes = one swizzle atom
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int A_STAGE_BYTES = BLOCK_M * BLOCK_K * 2;
constexpr int MN_BOX_BYTES = 64 * BLOCK_K * 2;  // one [64 k-rows][64 mn] box

struct GemmParams {
  void* C;
  long long ldc;
  int M, N, K;
  int a_mn_major, b_mn_major;
  int mode;
  const int* meta;
  int num_experts;
  int b_expert_rows;           // rows of B's 2D view that belong to one expert
  long long c_expert_stride;   // elements between consecutive experts' C (ragged-K)
  int accumulate;              // C += A*B instead of C = A*B
  int out_fp32;
  int kb_split;                // > 0: k-blocks from this one on read B from the second tensor map (K-concatenated B)
  int m_rotate_blocks;         // row-block rotation of the tile order (start on the rows this GPU owns)
  const int* blk_range;        // ragged-M only, optional (device): restrict to row blocks [blk_range[0], blk_range[1])
  int* status;
  int pair_rows;               // ragged-M: expert groups are padded to 256 rows (a CTA pair's tile never spans two)
  int c_tma;                   // epilogue writes C through tensor-map stores (tma_c); 0 = plain stores
  // EPI_SWIGLU: N is the width of act (= I); the tile's B rows come from tma_b (gate) and tma_b2 (up), tma_c covers
  // h [rows, 2 * N] (gate | up) and tma_c2 act [rows, N].  Row weights: weights[src_of[row] * topk + k_of[row]],
  // 0 for padding rows (src_of < 0); all three null = weight 1.
  const int* row_src_of;
  const int* row_k_of;
  const float* row_weights;
  int row_topk;
  // EPI_SWIGLU_BWD: the accumulator is d(act) [rows, N]; aux_in = saved gate | up [rows, 2 N] (row stride aux_ld);
  // tma_c covers d(gate) | d(up) [rows, 2 N]; aux_out [rows, ceil(N / 256)] receives, per row and column tile, the
  // partial dot product <d(act), silu(gate) * up> (the routing-weight gradient, summed over its tiles afterwards).
  const void* aux_in;
  long long aux_ld;
  float* aux_out;
};

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_SWIGLU_BWD = 2 };

// All-gather fused into the GEMM: the outer rows of A live in the memories of up to 8 GPUs.  Four extra warps per
// CTA ("stagers") copy the other GPUs' rows into this GPU's gathered copy of A with plain loads over NVLink and
// count the rows that have landed per 128-row block; the TMA producer waits (bounded) for a block's count before it
// loads tiles of that block from the local copy.  A remote row crosses NVLink once, however many column tiles read it.
template <bool PEER>
struct PeerArg {
  char unused;
};
template <>
struct PeerArg<true> {
  const void* src[8];  // peer r's slice [rows, K], row stride ld
  void* dst;           // this GPU's gathered copy [n * rows, K] (what tma_a covers), row stride ld
  int* flags;          // rows landed per 128-row block of dst; zero at launch
  long long ld;        // elements between rows
  int rows;            // rows per peer, a multiple of BLOCK_M
  int row_vecs;        // 16-byte vectors per row (K / 8; N / 8 when pushing)
  int n, me;
  // Reduce-scatter transport instead (push != 0): `flags` counts the epilogue warps that have stored their part of a
  // 128-row block of C; the stagers copy finished rows of peer r's block from C to push_dst[r] (its receive slot).
  int push;
  int flags_full;      // count at which a row block of C is complete (4 epilogue warps x column tiles)
  void* push_dst[8];
  const void* c_base;  // C and its row stride, as the stagers read it
  long long ldc;
  // Expert-parallel combine transport (push == 2, ragged-M mode): row u of C is the expert output of the routed pair
  // (token src_of[u] of the group's T-token-per-rank numbering, choice k_of[u]); it goes to the token owner's
  // receive buffer [T, topk, N] at push_dst[owner] + (t * topk + k) * ld.  Padding rows (src_of < 0) are not sent.
  // Expert-parallel dispatch (push == 3, ragged-M mode): row u of A is token src_of[u] (rank src_of[u] / T, local
  // index src_of[u] % T) of src[rank] (row stride src_ld); the stagers copy it into dst + u * ld (zeros for padding
  // rows) and count the rows per 128-row block in `flags`; the producer waits for 128 before it loads a block.
  const int* src_of;
  const int* k_of;
  int T, topk;
  long long src_ld;
  // Parameter all-gather inside the consuming GEMM (push == 4, dense mode, B K-major and contiguous [N, K]): elements
  // [seg_lo[r], seg_hi[r]) of B (counted from B's first element, multiples of 8) are current only in peer r's copy
  // src[r]; the stagers copy them into this GPU's B (`dst`) row piece by row piece and count the 16-byte vectors that
  // have landed per 128-row block of B in `flags`; the producer of a CTA waits until its 128 rows of B are complete.
  long long seg_lo[8], seg_hi[8];
};

// 16-byte vectors of rows [blk * 128, blk * 128 + 128) of B [N, K] that the stagers have to bring in (push == 4).
__device__ __forceinline__ int stale_vectors_in_block(const PeerArg<true>& peers, int blk, int N, int K) {
  const long long b_lo = static_cast<long long>(blk) * 128 * K;
  const long long b_hi = static_cast<long long>(min((blk + 1) * 128, N)) * K;
  long long total = 0;
  for (int r = 0; r < peers.n; ++r) {
    const long long lo = max(b_lo, peers.seg_lo[r]), hi = min(b_hi, peers.seg_hi[r]);
    if (hi > lo) total += (hi - lo) / 8;
  }
  return static_cast<int>(total);
}
constexpr int STAGER_WARPS = 4;
constexpr int NUM_THREADS_STAGED = NUM_THREADS + 32 * STAGER_WARPS;

// Epilogue staging: each of the four epilogue warps owns two buffers of 32 rows x 128 bytes (what one tensor-map
// store of its rows takes), laid out with the 128-byte swizzle the store expects.
constexpr int EPI_BUF_BYTES = 32 * 128;
constexpr int EPI_STAGING_BYTES = 4 * 2 * EPI_BUF_BYTES;

template <int BLOCK_N>
struct SmemLayout {
  static constexpr int B_STAGE_BYTES = BLOCK_N * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = (BLOCK_N == 256) ? 4 : (BLOCK_N == 128 ? 6 : 8);
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_STAGING_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + slack for 1024B alignment
};

struct TileInfo {
  int m0, n0;        // element offsets of the tile in C
  int kb_begin, kb_end;  // K range in units of BLOCK_K
  int expert;
};

// Map a linear tile id to its coordinates.  Returns false when `t` is past the last tile.
template <int BLOCK_N, int EPI = EPI_PLAIN>
__device__ __forceinline__ bool get_tile(const GemmParams& p, int t, int num_m_blocks, int blk0, TileInfo& ti) {
  constexpr int TILE_N = EPI == EPI_SWIGLU ? BLOCK_N / 2 : BLOCK_N;  // output columns per tile
  const int num_n_blocks = (p.N + TILE_N - 1) / TILE_N;
  if (p.mode == OLB_GEMM_RAGGED_K) {
    const int per_expert = num_m_blocks * num_n_blocks;
    if (t >= per_expert * p.num_experts) return false;
    const int e = t / per_expert;
    const int r = t - e * per_expert;
    ti.expert = e;
    ti.m0 = (r / num_n_blocks) * BLOCK_M;
    ti.n0 = (r % num_n_blocks) * TILE_N;
    ti.kb_begin = p.meta[e] / BLOCK_K;
    ti.kb_end = p.meta[e + 1] / BLOCK_K;
    return true;
  }
  if (t >= num_m_blocks * num_n_blocks) return false;
  // Walk N fastest inside bands of 8 row blocks so that concurrently resident CTAs share
  // operand tiles through L2.
  constexpr int BAND = 8;
  const int band_tiles = BAND * num_n_blocks;
  const int band = t / band_tiles;
  const int first_m = band * BAND;
  const int rows_in_band = min(BAND, num_m_blocks - first_m);
  const int r = t - band * band_tiles;
  int m_blk = first_m + r % rows_in_band;
  if (p.m_rotate_blocks) m_blk = (m_blk + p.m_rotate_blocks) % num_m_blocks;
  const int n_blk = r / rows_in_band;
  m_blk += blk0;  // first row block of the requested range
  ti.m0 = m_blk * BLOCK_M;
  ti.n0 = n_blk * TILE_N;
  ti.kb_begin = 0;
  ti.kb_end = (p.K + BLOCK_K - 1) / BLOCK_K;
  ti.expert = (p.mode == OLB_GEMM_RAGGED_M) ? p.meta[1 + m_blk] : 0;
  return true;
}

// Bounded wait until `*count >= need` (a counter that warps of this GPU raise).  False, with the status word set,
// when the limit runs out or another role of the CTA has given up.
__device__ __forceinline__ bool wait_count(const int* count, int need, int* status, volatile int* abort_flag) {
  unsigned long long t0 = 0;
  for (uint32_t it = 0; ld_acquire_gpu_s32(count) < need; ++it) {
    if ((it & 15u) == 15u) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (*abort_flag || now - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER);
        return false;
      }
    }
    __nanosleep(100);
  }
  return true;
}

// One warp copies a row of `vecs` 16-byte vectors, up to eight loads in flight per lane; the loads bypass L1
// (the row was written by other SMs during this kernel).
__device__ __forceinline__ void copy_row_ldcg(const uint4* s, uint4* d, int vecs, int lane) {
  for (int c0 = 0; c0 < vecs; c0 += 256) {
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = c0 + i * 32 + lane;
      if (c < vecs) v[i] = __ldcg(s + c);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = c0 + i * 32 + lane;
      if (c < vecs) d[c] = v[i];
    }
  }
}

// One warp stores its 32 rows x 128 bytes through a tensor-map store: the lane's row (`v`, 32 words) goes to the
// staging buffer in the swizzled layout, then lane 0 issues the store.  Buffers alternate; before a buffer is
// rewritten the store that used it two turns ago must have finished reading it.
struct EpiStage {
  uint32_t base;   // shared-memory address of this warp's two buffers
  int turn;
};
__device__ __forceinline__ void epi_store_chunk(EpiStage& es, const CUtensorMap* map, const uint32_t (&v)[32], int lane,
                                                int x, int y) {
  const uint32_t buf = es.base + (es.turn & 1) * EPI_BUF_BYTES;
  es.turn++;
  if (lane == 0) tma_store_wait_read_n<1>();
  __syncwarp();
  const uint32_t row = buf + lane * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    st_shared_v4(row + ((j ^ (lane & 7)) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(map, buf, x, y);
    tma_store_commit();
  }
}

// Epilogue of one 128-row accumulator tile without a fused activation: through staged tensor-map stores when the
// output allows it, else with plain loads / stores (accumulating epilogues, layouts a tensor map cannot describe).
// `taddr` is the accumulator's TMEM address for this warp's 32 lanes; `ti.m0` the first of the CTA's 128 rows.
template <int BLOCK_N>
__device__ __forceinline__ void epilogue_plain(const GemmParams& p, const CUtensorMap* tma_c, EpiStage& es, uint32_t taddr,
                                               const TileInfo& ti, bool has_k, int lane_group, int lane) {
  const int row = ti.m0 + lane_group * 32 + lane;
  const bool row_ok = row < p.M;
  if (p.c_tma) {
    // ---- staged tensor-map stores: 128 bytes of every row per turn (64 bf16 or 32 fp32 columns)
    long long y = ti.m0 + lane_group * 32;
    const bool rows_ok = y < p.M;
    if (p.mode == OLB_GEMM_RAGGED_K) y += static_cast<long long>(ti.expert) * p.M;
    if (p.out_fp32) {
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t r[32];
        if (has_k) {
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        const int x = ti.n0 + c * 32;
        if (rows_ok && x < p.N) epi_store_chunk(es, tma_c, r, lane, x, static_cast<int>(y));
      }
    } else {
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 64; ++c) {
        uint32_t v[32];
        if (has_k) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(taddr + c * 64, r0);
          tmem_ld_32x32b_x32(taddr + c * 64 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            v[i] = pack_bf16(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
            v[16 + i] = pack_bf16(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        const int x = ti.n0 + c * 64;
        if (rows_ok && x < p.N) epi_store_chunk(es, tma_c, v, lane, x, static_cast<int>(y));
      }
    }
  } else {
    // ---- plain loads / stores (accumulating epilogues, layouts a tensor map cannot describe)
    char* c_row;
    {
      long long off = static_cast<long long>(row) * p.ldc + ti.n0;
      if (p.mode == OLB_GEMM_RAGGED_K) off += static_cast<long long>(ti.expert) * p.c_expert_stride;
      c_row = static_cast<char*>(p.C) + off * (p.out_fp32 ? 4 : 2);
    }
#pragma unroll 1
    for (int c = 0; c < BLOCK_N / 32; ++c) {
      uint32_t r[32];
      if (has_k) {
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      if (row_ok) {
        const int col0 = ti.n0 + c * 32;
        if (p.out_fp32) {
          float4* dst = reinterpret_cast<float4*>(c_row + c * 32 * 4);
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if (col0 + g * 4 < p.N) {
              float4 v = make_float4(__uint_as_float(r[4 * g]), __uint_as_float(r[4 * g + 1]),
                                     __uint_as_float(r[4 * g + 2]), __uint_as_float(r[4 * g + 3]));
              if (p.accumulate) {
                float4 o = dst[g];
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
              }
              dst[g] = v;
            }
          }
        } else {
          uint4* dst = reinterpret_cast<uint4*>(c_row + c * 32 * 2);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (col0 + g * 8 < p.N) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[8 * g + i]);
              if (p.accumulate) {
                uint4 o = dst[g];
                float2 a;
                a = unpack_bf16(o.x); f[0] += a.x; f[1] += a.y;
                a = unpack_bf16(o.y); f[2] += a.x; f[3] += a.y;
                a = unpack_bf16(o.z); f[4] += a.x; f[5] += a.y;
                a = unpack_bf16(o.w); f[6] += a.x; f[7] += a.y;
              }
              uint4 v;
              v.x = pack_bf16(f[0], f[1]);
              v.y = pack_bf16(f[2], f[3]);
              v.z = pack_bf16(f[4], f[5]);
              v.w = pack_bf16(f[6], f[7]);
              dst[g] = v;
            }
          }
        }
      }
    }
  }
}

// Epilogue of one 128-row tile of the fused gate|up projection: accumulator columns [0,128) are gate, [128,256) up,
// both for act columns [ti.n0, ti.n0 + 128).  Writes gate | up (bf16) to tma_c and w(row) * silu(gate) * up to tma_c2.
__device__ __forceinline__ void epilogue_swiglu(const GemmParams& p, const CUtensorMap* tma_c, const CUtensorMap* tma_c2,
                                                EpiStage& es, uint32_t taddr, const TileInfo& ti, int lane_group, int lane) {
  const int row = ti.m0 + lane_group * 32 + lane;
  const bool row_ok = row < p.M;
  // columns [0,128) of the accumulator are gate, [128,256) up, both for act columns [n0, n0 + 128)
  float w = 1.f;
  if (p.row_src_of) {
    const int src = row_ok ? p.row_src_of[row] : -1;
    w = src >= 0 ? p.row_weights[static_cast<long long>(src) * p.row_topk + p.row_k_of[row]] : 0.f;
  }
  const int y = ti.m0 + lane_group * 32;
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {  // 64 act columns per turn
    uint32_t hg[32], hu[32];
    {
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(taddr + c * 64, r0);
      tmem_ld_32x32b_x32(taddr + c * 64 + 32, r1);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        hg[i] = pack_bf16(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
        hg[16 + i] = pack_bf16(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
      }
    }
    const int x = ti.n0 + c * 64;
    if (y < p.M && x < p.N) epi_store_chunk(es, tma_c, hg, lane, x, y);
    {
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(taddr + 128 + c * 64, r0);
      tmem_ld_32x32b_x32(taddr + 128 + c * 64 + 32, r1);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        hu[i] = pack_bf16(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
        hu[16 + i] = pack_bf16(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
      }
    }
    if (y < p.M && x < p.N) epi_store_chunk(es, tma_c, hu, lane, p.N + x, y);
    // the activation from the rounded values, as the backward recomputes it from the saved gate | up
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float2 g = unpack_bf16(hg[i]), u = unpack_bf16(hu[i]);
      hg[i] = pack_bf16(w * (g.x / (1.f + __expf(-g.x))) * u.x, w * (g.y / (1.f + __expf(-g.y))) * u.y);
    }
    if (y < p.M && x < p.N) epi_store_chunk(es, tma_c2, hg, lane, x, y);
  }
}

// Epilogue of one 128-row tile of the down projection's input gradient with the SwiGLU backward folded in: the
// accumulator holds d(act) for columns [ti.n0, ti.n0 + 256); gate and up of the same rows and columns are read from
// the saved forward buffer; d(gate) = d(act) w up silu'(gate) and d(up) = d(act) w silu(gate) go out through staged
// tensor-map stores, the row's partial <d(act), silu(gate) up> to aux_out.  d(act) is rounded to bf16 first, as if it
// had been stored and read back by a separate kernel.
__device__ __forceinline__ void epilogue_swiglu_bwd(const GemmParams& p, const CUtensorMap* tma_c, EpiStage& es,
                                                    uint32_t taddr, const TileInfo& ti, int lane_group, int lane) {
  const int row = ti.m0 + lane_group * 32 + lane;
  const bool row_ok = row < p.M;
  const int src = (row_ok && p.row_src_of) ? p.row_src_of[row] : (row_ok ? 0 : -1);
  float w = 0.f;
  if (src >= 0) w = p.row_weights ? p.row_weights[static_cast<long long>(src) * p.row_topk + p.row_k_of[row]] : 1.f;
  const __nv_bfloat16* hrow = static_cast<const __nv_bfloat16*>(p.aux_in) + static_cast<long long>(row) * p.aux_ld;
  const int y = ti.m0 + lane_group * 32;
  float dot = 0.f;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {  // 64 columns per turn
    uint32_t vg[32], vu[32];
    const int x = ti.n0 + c * 64;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(taddr + c * 64 + half * 32, r);
      uint4 g4[4], u4[4];
      if (src >= 0 && x + half * 32 < p.N) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          g4[j] = *reinterpret_cast<const uint4*>(hrow + x + half * 32 + j * 8);
          u4[j] = *reinterpret_cast<const uint4*>(hrow + p.N + x + half * 32 + j * 8);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) g4[j] = u4[j] = make_uint4(0, 0, 0, 0);
      }
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t gw[4] = {g4[j].x, g4[j].y, g4[j].z, g4[j].w}, uw[4] = {u4[j].x, u4[j].y, u4[j].z, u4[j].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i = j * 4 + q;  // pair index inside the 32-column half
          const float2 fg = unpack_bf16(gw[q]), fu = unpack_bf16(uw[q]);
          const float2 fd = unpack_bf16(pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])));
          const float sig0 = 1.f / (1.f + __expf(-fg.x)), sig1 = 1.f / (1.f + __expf(-fg.y));
          const float silu0 = fg.x * sig0, silu1 = fg.y * sig1;
          dot += fd.x * silu0 * fu.x + fd.y * silu1 * fu.y;
          vu[half * 16 + i] = pack_bf16(fd.x * w * silu0, fd.y * w * silu1);
          vg[half * 16 + i] = pack_bf16(fd.x * w * fu.x * (sig0 + silu0 * (1.f - sig0)),
                                        fd.y * w * fu.y * (sig1 + silu1 * (1.f - sig1)));
        }
      }
    }
    if (y < p.M && x < p.N) {
      epi_store_chunk(es, tma_c, vg, lane, x, y);
      epi_store_chunk(es, tma_c, vu, lane, p.N + x, y);
    }
  }
  if (row_ok && p.aux_out) p.aux_out[static_cast<long long>(row) * ((p.N + 255) / 256) + ti.n0 / 256] = dot;
}

// The extra warps of the variants with a fused transfer (PeerArg<true>): `swarp` is the warp's index among the CTA's
// STAGER_WARPS stagers, `num_m_blocks` the number of 128-row blocks of the launch.
__device__ __forceinline__ void stager_loop(const PeerArg<true>& peers, const GemmParams& p, int num_m_blocks, int swarp,
                                            int lane, volatile int* abort_flag) {
  // ---------------------------------------------------------- stagers (warps 6..9)
  // Remote rows in the order the tiles need them.  Every CTA's stagers take rows of the same block at the same
  // time, so blocks complete one after the other.  The gathers wait for nothing; the pushes wait (bounded) for
  // this GPU's own epilogues.
  const long long total = (peers.push == 2 || peers.push == 3)
                              ? min(static_cast<long long>(num_m_blocks) * BLOCK_M, static_cast<long long>(p.M))
                              : static_cast<long long>(peers.n - 1) * peers.rows;
  if (peers.push == 4) {
    // -------- parameter all-gather: the parts of B that other GPUs updated, row piece by row piece in row order
    const long long K = p.K;
    const long long gw = static_cast<long long>(blockIdx.x) * STAGER_WARPS + swarp;
    const long long nw = static_cast<long long>(gridDim.x) * STAGER_WARPS;
    for (int s = 0; s < peers.n; ++s) {
      if (peers.seg_hi[s] <= peers.seg_lo[s]) continue;
      const long long r0 = peers.seg_lo[s] / K, r1 = (peers.seg_hi[s] - 1) / K;
      for (long long r = r0 + gw; r <= r1; r += nw) {
        const long long lo = max(peers.seg_lo[s], r * K), hi = min(peers.seg_hi[s], (r + 1) * K);
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(peers.src[s]) + lo * 2);
        uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(peers.dst) + lo * 2);
        const int vecs = static_cast<int>((hi - lo) / 8);
        for (int c0 = 0; c0 < vecs; c0 += 256) {
          uint4 v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int c = c0 + i * 32 + lane;
            if (c < vecs) v[i] = src[c];
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int c = c0 + i * 32 + lane;
            if (c < vecs) dst[c] = v[i];
          }
        }
        fence_proxy_async_all();
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(peers.flags + r / BLOCK_M, vecs);
      }
    }
    return;
  }
  if (peers.push == 3) {
    // -------- expert-parallel dispatch: the routed token rows come from their owners into the grouped operand.
    // A warp takes two consecutive rows per turn (same 128-row block): 16 loads of 16 bytes in flight per lane, and
    // one fence + one count update for both.
    for (long long c = blockIdx.x * STAGER_WARPS + swarp; 2 * c < total; c += static_cast<long long>(gridDim.x) * STAGER_WARPS) {
      const long long u0 = 2 * c;
      const uint4* s[2];
      uint4* d[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        int g = peers.src_of[u0 + r];
        if (g >= 0 && !OLB_INDEX_OK(g, static_cast<long long>(peers.n) * peers.T, p.status)) g = -1;
        const int owner = g >= 0 ? g / peers.T : 0;
        s[r] = g >= 0 ? reinterpret_cast<const uint4*>(static_cast<const char*>(peers.src[owner]) +
                                                       static_cast<long long>(g - owner * peers.T) * peers.src_ld * 2)
                      : nullptr;
        d[r] = reinterpret_cast<uint4*>(static_cast<char*>(peers.dst) + (u0 + r) * peers.ld * 2);
      }
      for (int c0 = 0; c0 < peers.row_vecs; c0 += 256) {
        uint4 v[2][8];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int cc = c0 + i * 32 + lane;
            v[r][i] = (s[r] != nullptr && cc < peers.row_vecs) ? s[r][cc] : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int cc = c0 + i * 32 + lane;
            if (cc < peers.row_vecs) d[r][cc] = v[r][i];
          }
      }
      fence_proxy_async_all();
      __threadfence();
      __syncwarp();
      if (lane == 0) atomicAdd(peers.flags + u0 / BLOCK_M, 2);
    }
    return;
  }
  int ready_blk = -1;
  bool ok = true;
  for (long long u = blockIdx.x * STAGER_WARPS + swarp; ok && u < total;
       u += static_cast<long long>(gridDim.x) * STAGER_WARPS) {
    if (peers.push == 2) {
      // -------- expert-parallel combine transport: a finished row goes to the owner of its token
      const int blk = static_cast<int>(u / BLOCK_M);
      if (blk != ready_blk) {
        if (!wait_count(peers.flags + blk, peers.flags_full, p.status, abort_flag)) {
          ok = false;
          break;
        }
        ready_blk = blk;
      }
      const int g = peers.src_of[u];
      if (g < 0) continue;
      if (!OLB_INDEX_OK(g, static_cast<long long>(peers.n) * peers.T, p.status) ||
          !OLB_INDEX_OK(peers.k_of[u], peers.topk, p.status))
        continue;
      const int owner = g / peers.T;
      const long long slot = static_cast<long long>(g - owner * peers.T) * peers.topk + peers.k_of[u];
      const uint4* s = reinterpret_cast<const uint4*>(static_cast<const char*>(peers.c_base) + u * peers.ldc * 2);
      uint4* d = reinterpret_cast<uint4*>(static_cast<char*>(peers.push_dst[owner]) + slot * peers.ld * 2);
      copy_row_ldcg(s, d, peers.row_vecs, lane);
      continue;
    }
    const int j = static_cast<int>(u / peers.rows);
    const int r = static_cast<int>(u - static_cast<long long>(j) * peers.rows);
    const int peer = (peers.me + 1 + j) % peers.n;
    const long long drow = static_cast<long long>(peer) * peers.rows + r;
    if (peers.push) {
      // -------- reduce-scatter transport: row `drow` of C goes to its owner once every tile of its block is stored
      const int blk = static_cast<int>(drow / BLOCK_M);
      if (blk != ready_blk) {
        if (!wait_count(peers.flags + blk, peers.flags_full, p.status, abort_flag)) {
          ok = false;
          break;
        }
        ready_blk = blk;
      }
      const uint4* s = reinterpret_cast<const uint4*>(static_cast<const char*>(peers.c_base) + drow * peers.ldc * 2);
      uint4* d = reinterpret_cast<uint4*>(static_cast<char*>(peers.push_dst[peer]) + r * peers.ldc * 2);
      copy_row_ldcg(s, d, peers.row_vecs, lane);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(static_cast<const char*>(peers.src[peer]) + r * peers.ld * 2);
    uint4* d = reinterpret_cast<uint4*>(static_cast<char*>(peers.dst) + drow * peers.ld * 2);
    for (int c0 = 0; c0 < peers.row_vecs; c0 += 256) {
      uint4 v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = c0 + i * 32 + lane;
        if (c < peers.row_vecs) v[i] = s[c];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = c0 + i * 32 + lane;
        if (c < peers.row_vecs) d[c] = v[i];
      }
    }
    fence_proxy_async_all();
    __threadfence();
    __syncwarp();
    if (lane == 0) atomicAdd(peers.flags + drow / BLOCK_M, 1);
  }
}

template <int BLOCK_N, bool PEER, int EPI>
__global__ void __launch_bounds__(PEER ? NUM_THREADS_STAGED : NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_b2, const __grid_constant__ CUtensorMap tma_c,
                 const __grid_constant__ CUtensorMap tma_c2, const __grid_constant__ PeerArg<PEER> peers,
                 const GemmParams p) {
  using L = SmemLayout<BLOCK_N>;
  constexpr int STAGES = L::STAGES;
  constexpr uint32_t TMEM_COLS = (2 * BLOCK_N < 32) ? 32 : 2 * BLOCK_N;
  static_assert(EPI == EPI_PLAIN || BLOCK_N == 256, "the SwiGLU epilogue pairs 128 gate with 128 up columns");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  // barrier map: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::BAR_OFFSET + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::BAR_OFFSET + 8 * (2 * STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (p.c_tma) tma_prefetch_desc(&tma_c);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int num_m_blocks, blk0 = 0;
  if (p.mode == OLB_GEMM_RAGGED_M) {
    num_m_blocks = min(p.meta[0], (p.M + BLOCK_M - 1) / BLOCK_M);
    if (p.blk_range) {
      blk0 = p.blk_range[0];
      num_m_blocks = max(0, min(num_m_blocks, p.blk_range[1]) - blk0);
    }
  } else {
    num_m_blocks = (p.M + BLOCK_M - 1) / BLOCK_M;
  }

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TileInfo ti;
      for (int t = blockIdx.x; ok && get_tile<BLOCK_N, EPI>(p, t, num_m_blocks, blk0, ti); t += gridDim.x) {
        if constexpr (PEER) {
          // rows that the stagers bring in: wait until the whole row block is in the local operand
          bool wait_rows = false;
          int need = 0;
          if (peers.push == 0 && ti.m0 / peers.rows != peers.me) {
            wait_rows = true;
            need = min(BLOCK_M, p.M - ti.m0);
          } else if (peers.push == 3) {
            wait_rows = true;
            need = BLOCK_M;
          }
          if (wait_rows) {
            if (!wait_count(peers.flags + ti.m0 / BLOCK_M, need, p.status, abort_flag)) {
              ok = false;
              break;
            }
            fence_proxy_async_all();  // the rows were written by ordinary stores; the loads below are TMA
          }
        }
        for (int kb = ti.kb_begin; kb < ti.kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
          const uint32_t fb = full_bar(stage);
          mbar_expect_tx(fb, L::STAGE_BYTES);
          const int k0 = kb * BLOCK_K;
          if (!p.a_mn_major) {
            tma_load_2d(sa, &tma_a, fb, k0, ti.m0);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_M / 64; ++j) tma_load_2d(sa + j * MN_BOX_BYTES, &tma_a, fb, ti.m0 + j * 64, k0);
          }
          if constexpr (EPI == EPI_SWIGLU) {
            // 128 rows of the gate weight and the same 128 rows of the up weight: accumulator columns 0-127 | 128-255
            const int brow = ti.expert * p.b_expert_rows + ti.n0;
            tma_load_2d(sb, &tma_b, fb, k0, brow);
            tma_load_2d(sb + (BLOCK_N / 2) * BLOCK_K * 2, &tma_b2, fb, k0, brow);
          } else {
            // K-concatenated B: the second half of the K range comes from a second tensor of the same layout
            const bool second = p.kb_split > 0 && kb >= p.kb_split;
            const CUtensorMap* tmb = second ? &tma_b2 : &tma_b;
            const int kB = second ? k0 - p.kb_split * BLOCK_K : k0;
            if (!p.b_mn_major) {
              tma_load_2d(sb, tmb, fb, kB, ti.expert * p.b_expert_rows + ti.n0);
            } else {
              const int krow = (p.mode == OLB_GEMM_RAGGED_M ? ti.expert * p.b_expert_rows : 0) + kB;
#pragma unroll
              for (int j = 0; j < BLOCK_N / 64; ++j) tma_load_2d(sb + j * MN_BOX_BYTES, tmb, fb, ti.n0 + j * 64, krow);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // Drain: every issued load must have landed before the CTA's shared memory goes away.
      // The MMA warp consumes all stages in the normal case; after an abort wait (bounded)
      // for the loads of the current ring pass.
      if (!ok || *abort_flag) {
        for (int s = 0; s < STAGES; ++s) {
          unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(full_bar(s), (s < stage) ? phase : (phase ^ 1u))) {
            if (globaltimer_ns() - t0 > 200000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(BLOCK_M, BLOCK_N, p.a_mn_major, p.b_mn_major);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      TileInfo ti;
      for (int t = blockIdx.x; ok && get_tile<BLOCK_N, EPI>(p, t, num_m_blocks, blk0, ti); t += gridDim.x) {
        if (ti.kb_end <= ti.kb_begin) continue;  // empty expert: the epilogue writes zeros
        if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, p.status, ST_TIMEOUT_ACC_EMPTY, abort_flag)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = ti.kb_begin; kb < ti.kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.status, ST_TIMEOUT_FULL, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            const uint64_t da = p.a_mn_major ? make_smem_desc(sa + k * (UMMA_K * 128), MN_BOX_BYTES, 1024)
                                             : make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = p.b_mn_major ? make_smem_desc(sb + k * (UMMA_K * 128), MN_BOX_BYTES, 1024)
                                             : make_smem_desc(sb + k * (UMMA_K * 2), 16, 1024);
            umma_ss(tmem_d, da, db, idesc, (kb > ti.kb_begin || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // the stage is free once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(acc_full_bar(acc));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int lane_group = warp & 3;  // TMEM lanes [32*lane_group, +32) belong to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    TileInfo ti;
    EpiStage es{smem_base + L::EPI_OFFSET + lane_group * 2 * EPI_BUF_BYTES, 0};
    for (int t = blockIdx.x; get_tile<BLOCK_N, EPI>(p, t, num_m_blocks, blk0, ti); t += gridDim.x) {
      const bool has_k = ti.kb_end > ti.kb_begin;
      if (has_k) {
        if (!mbar_wait(acc_full_bar(acc), acc_phase, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) break;
        tc_fence_after();
      } else if (p.accumulate) {
        continue;  // nothing to add
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + acc * BLOCK_N;
      if constexpr (EPI == EPI_SWIGLU) {
        epilogue_swiglu(p, &tma_c, &tma_c2, es, taddr, ti, lane_group, lane);
      } else {
        epilogue_plain<BLOCK_N>(p, &tma_c, es, taddr, ti, has_k, lane_group, lane);
      }
      if constexpr (PEER) {
        if (peers.push == 1 || peers.push == 2) {  // this warp's 32 rows of the tile are stored: let the stagers know
          if (p.c_tma || EPI == EPI_SWIGLU) {
            if (lane == 0) tma_store_wait_all();   // the stores issued by this lane are complete, not only read
            fence_proxy_async_all();
          }
          __threadfence();
          __syncwarp();
          if (lane == 0) atomicAdd(peers.flags + ti.m0 / BLOCK_M, 1);
        }
      }
      if (has_k) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(acc));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
    if (lane == 0) tma_store_wait_read();  // the staging buffers must outlive the stores that read them
  }

  if constexpr (PEER) {
    if (warp >= 6) {
      stager_loop(peers, p, num_m_blocks, warp - 6, lane, abort_flag);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): one 256 x 256 output tile per cluster of two CTAs.  CTA r of the pair stages rows
// [m0 + 128 r, +128) of A and rows [n0 + 128 r, +128) of B; the MMAs (UMMA 256 x 256 x 16), issued by one thread of
// CTA 0, read both CTAs' shared memory and write rows [128 r, +128) x 256 columns of D into CTA r's TMEM.  Per flop
// each SM reads half as many B bytes from shared memory as the single-CTA kernel, which is what that kernel runs out
// of at 128 x 256.  Barriers: the "full" barrier of a stage lives in CTA 0 and counts the bytes of both CTAs' loads;
// "empty" and "accumulator full" exist in both CTAs and are signalled by the MMA thread's commits to both; "accumulator
// empty" lives in CTA 0 and collects the eight epilogue warps of the pair.
struct SmemLayoutPair {
  static constexpr int B_STAGE_BYTES = 128 * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_STAGING_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};

template <int EPI>
__device__ __forceinline__ bool get_tile_pair(const GemmParams& p, int t, int num_m, TileInfo& ti) {
  // 256-row tiles (two 128-row blocks, one per CTA); same walk as the single-CTA kernel (N fastest inside bands)
  constexpr int TILE_N = EPI == EPI_SWIGLU ? 128 : 256;
  const int num_n = (p.N + TILE_N - 1) / TILE_N;
  if (p.mode == OLB_GEMM_RAGGED_K) {
    const int per_expert = num_m * num_n;
    if (t >= per_expert * p.num_experts) return false;
    const int e = t / per_expert;
    const int r = t - e * per_expert;
    ti.expert = e;
    ti.m0 = (r / num_n) * 256;
    ti.n0 = (r % num_n) * TILE_N;
    ti.kb_begin = p.meta[e] / BLOCK_K;
    ti.kb_end = p.meta[e + 1] / BLOCK_K;
    return true;
  }
  if (t >= num_m * num_n) return false;
  constexpr int BAND = 8;
  const int band_tiles = BAND * num_n;
  const int band = t / band_tiles;
  const int first_m = band * BAND;
  const int rows_in_band = min(BAND, num_m - first_m);
  const int r = t - band * band_tiles;
  const int m_pair = first_m + r % rows_in_band;
  ti.m0 = m_pair * 256;
  ti.n0 = (r / rows_in_band) * TILE_N;
  ti.kb_begin = 0;
  ti.kb_end = (p.K + BLOCK_K - 1) / BLOCK_K;
  // expert groups are padded to 256 rows (p.pair_rows), so both blocks of a pair belong to one expert
  ti.expert = (p.mode == OLB_GEMM_RAGGED_M) ? p.meta[1 + 2 * m_pair] : 0;
  return true;
}

template <bool PEER, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PEER ? NUM_THREADS_STAGED : NUM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const __grid_constant__ CUtensorMap tma_b2, const __grid_constant__ CUtensorMap tma_c,
                      const __grid_constant__ CUtensorMap tma_c2, const __grid_constant__ PeerArg<PEER> peers,
                      const GemmParams p) {
  using L = SmemLayoutPair;
  constexpr int STAGES = L::STAGES;
  constexpr int BLOCK_N = 256;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::BAR_OFFSET + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::BAR_OFFSET + 8 * (2 * STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0 = the CTA that issues the MMAs
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);     // CTA 0's: its producer's arrive.expect_tx for the bytes of both CTAs
      mbar_init(empty_bar(s), 1);    // one commit of the MMA thread
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 8);  // CTA 0's: four epilogue warps of each CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (p.c_tma) tma_prefetch_desc(&tma_c);
  }
  if (warp == 2) {
    // every CTA allocates all 512 columns of its own TMEM (one CTA per SM): both get the same base
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  // the peer's barriers must be initialised before anything of this CTA can reach them
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int num_m_blocks;   // 128-row blocks of the launch (the stagers' unit); tiles take two of them
  if (p.mode == OLB_GEMM_RAGGED_M)
    num_m_blocks = min(p.meta[0], (p.M + BLOCK_M - 1) / BLOCK_M);
  else
    num_m_blocks = (p.M + BLOCK_M - 1) / BLOCK_M;
  const int num_m = (num_m_blocks + 1) / 2;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs, each for its own halves)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TileInfo ti;
      for (int t = pair_id; ok && get_tile_pair<EPI>(p, t, num_m, ti); t += num_pairs) {
        const int m0 = ti.m0 + static_cast<int>(rank) * 128;
        if constexpr (PEER) {
          if (peers.push == 4) {
            // this CTA's 128 rows of B: wait for the parts that other GPUs own (nothing to wait for once they are in)
            const int nb = (ti.n0 + static_cast<int>(rank) * 128) / BLOCK_M;
            if (nb * BLOCK_M < p.N) {
              const int need = stale_vectors_in_block(peers, nb, p.N, p.K);
              if (need > 0) {
                if (!wait_count(peers.flags + nb, need, p.status, abort_flag)) {
                  ok = false;
                  break;
                }
                fence_proxy_async_all();
              }
            }
          }
          if (peers.push == 3) {
            // the stagers bring this CTA's 128 rows into the local operand (the other CTA waits for its own)
            if (!wait_count(peers.flags + m0 / BLOCK_M, BLOCK_M, p.status, abort_flag)) {
              ok = false;
              break;
            }
            fence_proxy_async_all();
          }
        }
        for (int kb = ti.kb_begin; kb < ti.kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
          const uint32_t fb = mapa_shared(full_bar(stage), 0);
          const int k0 = kb * BLOCK_K;
          if (!p.a_mn_major) {
            tma_load_2d_pair(sa, &tma_a, fb, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * MN_BOX_BYTES, &tma_a, fb, m0 + j * 64, k0);
          }
          if constexpr (EPI == EPI_SWIGLU) {
            // CTA 0 stages 128 rows of the gate weight, CTA 1 the same rows of the up weight:
            // accumulator columns 0-127 | 128-255 in both CTAs
            tma_load_2d_pair(sb, rank == 0 ? &tma_b : &tma_b2, fb, k0, ti.expert * p.b_expert_rows + ti.n0);
          } else {
            const int n0 = ti.n0 + static_cast<int>(rank) * 128;
            const bool second = p.kb_split > 0 && kb >= p.kb_split;
            const CUtensorMap* tmb = second ? &tma_b2 : &tma_b;
            const int kB = second ? k0 - p.kb_split * BLOCK_K : k0;
            if (!p.b_mn_major) {
              tma_load_2d_pair(sb, tmb, fb, kB, ti.expert * p.b_expert_rows + n0);
            } else {
              const int krow = (p.mode == OLB_GEMM_RAGGED_M ? ti.expert * p.b_expert_rows : 0) + kB;
#pragma unroll
              for (int j = 0; j < 2; ++j) tma_load_2d_pair(sb + j * MN_BOX_BYTES, tmb, fb, n0 + j * 64, krow);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag) {
        // after a timeout: give this CTA's loads in flight time to land before its shared memory goes away
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (one thread of CTA 0 for the pair)
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = make_idesc_bf16(256, BLOCK_N, p.a_mn_major, p.b_mn_major);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      TileInfo ti;
      for (int t = pair_id; ok && get_tile_pair<EPI>(p, t, num_m, ti); t += num_pairs) {
        if (ti.kb_end <= ti.kb_begin) continue;
        if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, p.status, ST_TIMEOUT_ACC_EMPTY, abort_flag)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = ti.kb_begin; kb < ti.kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.status, ST_TIMEOUT_FULL, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            const uint64_t da = p.a_mn_major ? make_smem_desc(sa + k * (UMMA_K * 128), MN_BOX_BYTES, 1024)
                                             : make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = p.b_mn_major ? make_smem_desc(sb + k * (UMMA_K * 128), MN_BOX_BYTES, 1024)
                                             : make_smem_desc(sb + k * (UMMA_K * 2), 16, 1024);
            umma_ss_pair(tmem_d, da, db, idesc, (kb > ti.kb_begin || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage), 3);  // both CTAs' stages are free once these MMAs have read them
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(acc_full_bar(acc), 3);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs, own 128 rows)
    const int lane_group = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    TileInfo ti;
    EpiStage es{smem_base + L::EPI_OFFSET + lane_group * 2 * EPI_BUF_BYTES, 0};
    const uint32_t acc_empty_remote0 = mapa_shared(acc_empty_bar(0), 0);
    const uint32_t acc_empty_remote1 = mapa_shared(acc_empty_bar(1), 0);
    for (int t = pair_id; get_tile_pair<EPI>(p, t, num_m, ti); t += num_pairs) {
      const bool has_k = ti.kb_end > ti.kb_begin;
      if (has_k) {
        if (!mbar_wait(acc_full_bar(acc), acc_phase, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) break;
        tc_fence_after();
      } else if (p.accumulate) {
        continue;
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + acc * BLOCK_N;
      TileInfo mine = ti;
      mine.m0 = ti.m0 + static_cast<int>(rank) * 128;
      if constexpr (EPI == EPI_SWIGLU) {
        epilogue_swiglu(p, &tma_c, &tma_c2, es, taddr, mine, lane_group, lane);
      } else if constexpr (EPI == EPI_SWIGLU_BWD) {
        epilogue_swiglu_bwd(p, &tma_c, es, taddr, mine, lane_group, lane);
      } else {
        epilogue_plain<BLOCK_N>(p, &tma_c, es, taddr, mine, has_k, lane_group, lane);
      }
      if constexpr (PEER) {
        if (peers.push == 1 || peers.push == 2) {  // this warp's 32 rows of the tile are stored: let the stagers know
          if (p.c_tma || EPI == EPI_SWIGLU) {
            if (lane == 0) tma_store_wait_all();
            fence_proxy_async_all();
          }
          __threadfence();
          __syncwarp();
          if (lane == 0 && mine.m0 < p.M) atomicAdd(peers.flags + mine.m0 / BLOCK_M, 1);
        }
      }
      if (has_k) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc ? acc_empty_remote1 : acc_empty_remote0);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
    if (lane == 0) tma_store_wait_read();
  }
  if constexpr (PEER) {
    if (warp >= 6) stager_loop(peers, p, num_m_blocks, warp - 6, lane, abort_flag);
  }

  // neither CTA may leave while its partner can still signal its barriers or read its shared memory
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// Host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

// 2D tensor maps with 128B swizzle are pure functions of (base, extents, stride, box, element type).  A training
// step asks for the same few hundred of them every iteration (weights, flat gradient buffer, activations that the
// caching allocator hands back at the same addresses), so they are kept in a small per-thread table instead of being
// encoded two to five times per launch.
struct TmapKey {
  const void* base;
  uint64_t inner, outer, stride;
  uint32_t box_inner, box_outer, fp32;
  bool operator==(const TmapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && stride == o.stride && box_inner == o.box_inner &&
           box_outer == o.box_outer && fp32 == o.fp32;
  }
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int TMAP_CACHE_SLOTS = 2048;

static int make_tmap_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                        uint32_t box_inner, uint32_t box_outer, bool fp32) {
  static thread_local TmapSlot* table = nullptr;
  if (!table) table = new TmapSlot[TMAP_CACHE_SLOTS]();
  const TmapKey key{base, inner, outer, row_stride_bytes, box_inner, box_outer, fp32 ? 1u : 0u};
  uint64_t h = reinterpret_cast<uintptr_t>(base) * 0x9E3779B97F4A7C15ull;
  h ^= (inner * 0xC2B2AE3D27D4EB4Full) ^ (outer * 0x165667B19E3779F9ull) ^ (row_stride_bytes << 17) ^
       (static_cast<uint64_t>(box_inner) << 40) ^ (static_cast<uint64_t>(box_outer) << 52) ^ (fp32 ? 0x8000u : 0u);
  TmapSlot& slot = table[(h >> 20) % TMAP_CACHE_SLOTS];
  if (slot.used && slot.key == key) {
    *map = slot.map;
    return 0;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -2;
  slot.key = key;
  slot.map = *map;
  slot.used = true;
  return 0;
}

// 2D bf16 tensor map with 128B swizzle.  dims/box are {inner, outer}.
int make_tmap_2d_bf16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                      uint32_t box_inner, uint32_t box_outer) {
  return make_tmap_2d(map, base, inner, outer, row_stride_bytes, box_inner, box_outer, false);
}

// 4D bf16 tensor map with 128B swizzle (attention: dims {D, H, S, B} over a strided [B, S, H, D] view).
int make_tmap_4d_bf16(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides_bytes[3],
                      const uint32_t box[4]) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t s[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t b[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), d, s, b, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

struct TensorMaps {
  CUtensorMap a, b, b2, c, c2;
};

template <int BLOCK_N, bool PEER, int EPI>
static int launch(const TensorMaps& tm, const PeerArg<PEER>& peers, const GemmParams& p, int num_sms, cudaStream_t stream) {
  using L = SmemLayout<BLOCK_N>;
  // the shared-memory opt-in is an attribute of the function on one device
  constexpr int MAX_DEVICES = 64;
  static bool configured[MAX_DEVICES] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -3;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BLOCK_N, PEER, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return -3;
    configured[dev] = true;
  }
  constexpr int TILE_N = EPI == EPI_SWIGLU ? BLOCK_N / 2 : BLOCK_N;
  const long long nm = (p.M + BLOCK_M - 1) / BLOCK_M, nn = (p.N + TILE_N - 1) / TILE_N;
  const long long tiles = nm * nn * (p.mode == OLB_GEMM_RAGGED_K ? p.num_experts : 1);
  int grid = static_cast<int>(tiles < num_sms ? tiles : num_sms);
  if (grid <= 0) return 0;
  gemm_bf16_kernel<BLOCK_N, PEER, EPI><<<grid, PEER ? NUM_THREADS_STAGED : NUM_THREADS, L::TOTAL, stream>>>(
      tm.a, tm.b, tm.b2, tm.c, tm.c2, peers, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <bool PEER, int EPI>
static int launch_pair(const TensorMaps& tm, const PeerArg<PEER>& peers, const GemmParams& p, int num_sms,
                       cudaStream_t stream) {
  using L = SmemLayoutPair;
  constexpr int MAX_DEVICES = 64;
  static bool configured[MAX_DEVICES] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -3;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(gemm_bf16_pair_kernel<PEER, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) !=
        cudaSuccess)
      return -3;
    configured[dev] = true;
  }
  constexpr int TILE_N = EPI == EPI_SWIGLU ? 128 : 256;
  const long long nm = (p.M + 255) / 256, nn = (p.N + TILE_N - 1) / TILE_N;
  const long long tiles = nm * nn * (p.mode == OLB_GEMM_RAGGED_K ? p.num_experts : 1);
  const int max_pairs = num_sms / 2;
  const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
  if (pairs <= 0) return 0;
  gemm_bf16_pair_kernel<PEER, EPI><<<2 * pairs, PEER ? NUM_THREADS_STAGED : NUM_THREADS, L::TOTAL, stream>>>(
      tm.a, tm.b, tm.b2, tm.c, tm.c2, peers, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// OLB_GEMM_PAIR=0 keeps every GEMM on the single-CTA kernel (A/B comparisons, debugging).
static bool pair_kernel_enabled() {
  static const bool on = [] {
    const char* v = getenv("OLB_GEMM_PAIR");
    return !(v && v[0] == '0');
  }();
  return on;
}

template <bool PEER>
static int dispatch(int block_n, int epi, const TensorMaps& tm, const PeerArg<PEER>& peers, const GemmParams& p, int sms,
                    cudaStream_t stream) {
  if (epi == EPI_SWIGLU) return block_n == 256 ? launch<256, PEER, EPI_SWIGLU>(tm, peers, p, sms, stream) : -12;
  switch (block_n) {
    case 256: return launch<256, PEER, EPI_PLAIN>(tm, peers, p, sms, stream);
    case 128: return launch<128, PEER, EPI_PLAIN>(tm, peers, p, sms, stream);
    case 64: return launch<64, PEER, EPI_PLAIN>(tm, peers, p, sms, stream);
    default: return -12;
  }
}

static int device_sm_count() {
  constexpr int MAX_DEVICES = 64;
  static int cached[MAX_DEVICES] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 0;
  if (cached[dev] == 0) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
  return cached[dev];
}

}  // namespace olb

extern "C" int olb_gemm_bf16(const olb_gemm_desc* d, cudaStream_t stream) {
  using namespace olb;
  if (d->M <= 0 || d->N <= 0) return 0;
  if ((d->lda % 8) || (d->ldb % 8) || (d->ldc % 8) || (d->N % 8) || (reinterpret_cast<uintptr_t>(d->A) & 15) ||
      (reinterpret_cast<uintptr_t>(d->B) & 15) || (reinterpret_cast<uintptr_t>(d->C) & 15))
    return -10;
  const int epi = d->epilogue;
  int block_n = d->block_n;
  if (epi == OLB_EPI_SWIGLU) {
    // N = width of act; B / B2 = gate / up weights (K-major, same layout); C = gate | up [rows, 2 N]; C2 = act [rows, N]
    if (d->N % 128 || d->B2 == nullptr || d->C2 == nullptr || d->b_mn_major || d->a_mn_major || d->accumulate ||
        d->out_fp32 || d->mode == OLB_GEMM_RAGGED_K || d->k_split || (d->ldc2 % 8) ||
        (reinterpret_cast<uintptr_t>(d->B2) & 15) || (reinterpret_cast<uintptr_t>(d->C2) & 15) ||
        ((d->row_src_of != nullptr) != (d->row_weights != nullptr)) || ((d->row_src_of != nullptr) != (d->row_k_of != nullptr)))
      return -15;
    block_n = 256;
  } else if (epi == OLB_EPI_SWIGLU_BWD) {
    // C = d(gate) | d(up) [rows, 2 N]; the accumulator d(act) [rows, N] is not stored.  CTA-pair kernel only.
    if (d->N % 256 || d->aux_in == nullptr || d->accumulate || d->out_fp32 || d->mode != OLB_GEMM_RAGGED_M ||
        !d->pair_rows || d->M % 256 || d->a_mn_major || (d->aux_ld % 8) || d->blk_range != nullptr ||
        (reinterpret_cast<uintptr_t>(d->aux_in) & 15) || !pair_kernel_enabled() ||
        ((d->row_src_of != nullptr) != (d->row_weights != nullptr)) || ((d->row_src_of != nullptr) != (d->row_k_of != nullptr)))
      return -16;
    block_n = 256;
  } else if (block_n == 0) {
    if (d->mode != OLB_GEMM_DENSE) {
      block_n = (d->N % 256 == 0) ? 256 : (d->N % 128 == 0 ? 128 : 64);
      if (d->N % 64) return -11;
    } else {
      block_n = d->N > 128 ? 256 : (d->N > 64 ? 128 : 64);
    }
  }
  const int num_sms = device_sm_count();
  if (num_sms <= 0) return -3;
  // CTA pairs (256 x 256 tiles) for the plain dense and per-expert weight-gradient products that fill such tiles
  // (ragged-M: only when the caller padded the expert groups to 256 rows; the dense all-gather / reduce-scatter
  // variants, whose peers own multiples of 128 rows, stay on the single-CTA kernel)
  const bool pair_shape = d->block_n == 0 && block_n == 256 && d->blk_range == nullptr && d->M >= 256 && num_sms >= 2 &&
                          (epi != OLB_EPI_PLAIN || d->N % 256 == 0 || d->N >= 2048);
  const bool use_pair = pair_kernel_enabled() && pair_shape &&
                        (d->mode == OLB_GEMM_RAGGED_M ? (d->pair_rows != 0 && d->M % 256 == 0)
                                                      : ((d->n_peers == 0 || d->B_peers != nullptr) && epi == OLB_EPI_PLAIN));

  // cuTensorMapEncodeTiled is a driver call and needs a current context in the calling thread.
  // A thread that has only been handed tensors (an autograd worker whose first CUDA work is this
  // GEMM) has none yet; one runtime call binds the primary context.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  TensorMaps tm;
  int rc;
  // A: K-major -> global [a_rows, K] (inner K); MN-major -> global [K rows, M] (inner M).
  if (!d->a_mn_major)
    rc = make_tmap_2d_bf16(&tm.a, d->A, d->K, d->a_rows, d->lda * 2, BLOCK_K, BLOCK_M);
  else
    rc = make_tmap_2d_bf16(&tm.a, d->A, d->M, d->a_rows, d->lda * 2, 64, BLOCK_K);
  if (rc) return rc;
  int kb_split = 0;
  const int b_box_rows = use_pair ? 128 : block_n;   // a CTA of a pair stages half of the tile's B rows
  if (epi == OLB_EPI_SWIGLU) {
    rc = make_tmap_2d_bf16(&tm.b, d->B, d->K, d->b_rows, d->ldb * 2, BLOCK_K, 128);
    if (!rc) rc = make_tmap_2d_bf16(&tm.b2, d->B2, d->K, d->b_rows, d->ldb * 2, BLOCK_K, 128);
    if (rc) return rc;
  } else {
    if (!d->b_mn_major)
      rc = make_tmap_2d_bf16(&tm.b, d->B, d->K, d->b_rows, d->ldb * 2, BLOCK_K, b_box_rows);
    else
      rc = make_tmap_2d_bf16(&tm.b, d->B, d->N, d->b_rows, d->ldb * 2, 64, BLOCK_K);
    if (rc) return rc;
    // optional second B (same layout) for the K range [k_split, K)
    tm.b2 = tm.b;
    if (d->B2 != nullptr && d->k_split > 0) {
      if (d->k_split % BLOCK_K || d->k_split >= d->K || d->mode == OLB_GEMM_RAGGED_K || (reinterpret_cast<uintptr_t>(d->B2) & 15))
        return -13;
      const int k1 = d->k_split, k2 = d->K - d->k_split;
      // each map covers only its own K extent, so that reads past it are zero-filled as usual
      if (!d->b_mn_major) {
        rc = make_tmap_2d_bf16(&tm.b, d->B, k1, d->b_rows, d->ldb * 2, BLOCK_K, b_box_rows);
        if (!rc) rc = make_tmap_2d_bf16(&tm.b2, d->B2, k2, d->b_rows, d->ldb * 2, BLOCK_K, b_box_rows);
      } else {
        rc = make_tmap_2d_bf16(&tm.b2, d->B2, d->N, d->b_rows, d->ldb * 2, 64, BLOCK_K);
      }
      if (rc) return rc;
      kb_split = d->k_split / BLOCK_K;
    }
  }

  GemmParams p{};
  p.C = d->C;
  p.ldc = d->ldc;
  p.M = d->M;
  p.N = d->N;
  p.K = d->K;
  p.a_mn_major = d->a_mn_major;
  p.b_mn_major = d->b_mn_major;
  p.mode = d->mode;
  p.meta = d->meta;
  p.num_experts = d->num_experts;
  p.b_expert_rows = d->b_expert_rows;
  p.c_expert_stride = d->c_expert_stride;
  p.accumulate = d->accumulate;
  p.out_fp32 = d->out_fp32;
  p.kb_split = kb_split;
  p.m_rotate_blocks = 0;
  p.blk_range = d->mode == OLB_GEMM_RAGGED_M ? d->blk_range : nullptr;
  p.status = d->status;
  p.row_src_of = d->row_src_of;
  p.row_k_of = d->row_k_of;
  p.row_weights = d->row_weights;
  p.row_topk = d->row_topk;
  p.pair_rows = d->pair_rows;
  p.aux_in = d->aux_in;
  p.aux_ld = d->aux_ld;
  p.aux_out = d->aux_out;

  // Output through tensor-map stores whenever a 2D map describes it: no read-modify-write, and for the per-expert
  // weight gradients experts that tile exactly (a box must not run into the next expert's rows).
  tm.c = tm.a;
  tm.c2 = tm.a;
  p.c_tma = 0;
  if (epi == OLB_EPI_SWIGLU) {
    rc = make_tmap_2d(&tm.c, d->C, 2ull * d->N, d->M, d->ldc * 2, 64, 32, false);
    if (!rc) rc = make_tmap_2d(&tm.c2, d->C2, d->N, d->M, d->ldc2 * 2, 64, 32, false);
    if (rc) return rc;
    p.c_tma = 1;
  } else if (epi == OLB_EPI_SWIGLU_BWD) {
    rc = make_tmap_2d(&tm.c, d->C, 2ull * d->N, d->M, d->ldc * 2, 64, 32, false);
    if (rc) return rc;
    p.c_tma = 1;
  } else if (!d->accumulate) {
    const uint64_t esz = d->out_fp32 ? 4 : 2;
    uint64_t rows = d->M;
    bool ok = (d->ldc * esz) % 16 == 0;
    if (d->mode == OLB_GEMM_RAGGED_K) {
      ok = ok && d->M % BLOCK_M == 0 && d->c_expert_stride == static_cast<long long>(d->M) * d->ldc;
      rows = static_cast<uint64_t>(d->M) * d->num_experts;
    }
    if (ok) {
      rc = make_tmap_2d(&tm.c, d->C, d->N, rows, d->ldc * esz, d->out_fp32 ? 32 : 64, 32, d->out_fp32 != 0);
      if (rc) return rc;
      p.c_tma = 1;
    }
  }

  const int sms = d->max_ctas > 0 && d->max_ctas < num_sms ? d->max_ctas : num_sms;
  if (d->n_peers > 0) {
    const bool push = d->C_peers != nullptr;
    if (d->mode == OLB_GEMM_RAGGED_M) {
      PeerArg<true> peers{};
      peers.flags = d->stage_flags;
      peers.n = d->n_peers;
      peers.me = d->my_peer;
      peers.src_of = d->ep_src_of;
      peers.k_of = d->ep_k_of;
      peers.T = d->ep_tokens;
      peers.topk = d->ep_topk;
      if (d->n_peers > 8 || d->stage_flags == nullptr || d->ep_src_of == nullptr || d->ep_tokens <= 0 ||
          d->blk_range != nullptr)
        return -14;
      if (push) {
        // Expert-parallel combine transport: finished rows of C go to the owners of their tokens.
        if (epi != OLB_EPI_PLAIN || d->ep_k_of == nullptr || d->ep_topk <= 0 || d->out_fp32 || d->accumulate || d->N % 8)
          return -14;
        for (int r = 0; r < 8; ++r) {
          peers.push_dst[r] = d->C_peers[r < d->n_peers ? r : 0];
          if (reinterpret_cast<uintptr_t>(peers.push_dst[r]) & 15) return -14;
        }
        peers.push = 2;
        peers.flags_full = 4 * ((d->N + block_n - 1) / block_n);
        peers.c_base = d->C;
        peers.ldc = d->ldc;
        peers.ld = d->N;
        peers.row_vecs = d->N / 8;
      } else {
        // Expert-parallel dispatch: the routed token rows are gathered into A from their owners' buffers.
        if (d->A_peers == nullptr || d->a_mn_major || d->K % 8 || d->a_src_ld % 8 || d->a_src_ld < d->K) return -14;
        for (int r = 0; r < 8; ++r) {
          peers.src[r] = d->A_peers[r < d->n_peers ? r : 0];
          if (reinterpret_cast<uintptr_t>(peers.src[r]) & 15) return -14;
        }
        peers.push = 3;
        peers.dst = const_cast<void*>(d->A);
        peers.ld = d->lda;
        peers.src_ld = d->a_src_ld;
        peers.row_vecs = d->K / 8;
      }
      if (use_pair) {
        if (epi == OLB_EPI_SWIGLU) return launch_pair<true, EPI_SWIGLU>(tm, peers, p, sms, stream);
        if (epi == OLB_EPI_SWIGLU_BWD) return launch_pair<true, EPI_SWIGLU_BWD>(tm, peers, p, sms, stream);
        return launch_pair<true, EPI_PLAIN>(tm, peers, p, sms, stream);
      }
      if (epi == OLB_EPI_SWIGLU_BWD) return -16;
      return dispatch<true>(block_n, epi, tm, peers, p, sms, stream);
    }
    if (epi != OLB_EPI_PLAIN) return -14;
    if (d->B_peers != nullptr) {
      // Parameter all-gather inside the GEMM: parts of B are fetched from the peers that updated them.
      if (!use_pair || d->n_peers > 8 || d->mode != OLB_GEMM_DENSE || d->stage_flags == nullptr || d->b_seg == nullptr ||
          d->b_mn_major || d->ldb != d->K || d->K % 8 || d->A_peers != nullptr || d->C_peers != nullptr)
        return -17;
      PeerArg<true> peers{};
      peers.flags = d->stage_flags;
      peers.n = d->n_peers;
      peers.me = d->my_peer;
      peers.push = 4;
      peers.dst = const_cast<void*>(d->B);
      for (int r = 0; r < 8; ++r) {
        peers.src[r] = d->B_peers[r < d->n_peers ? r : 0];
        peers.seg_lo[r] = r < d->n_peers ? d->b_seg[2 * r] : 0;
        peers.seg_hi[r] = r < d->n_peers ? d->b_seg[2 * r + 1] : 0;
        if ((reinterpret_cast<uintptr_t>(peers.src[r]) & 15) || (peers.seg_lo[r] % 8) || (peers.seg_hi[r] % 8) ||
            peers.seg_hi[r] > static_cast<long long>(d->N) * d->K || peers.seg_lo[r] < 0)
          return -17;
      }
      return launch_pair<true, EPI_PLAIN>(tm, peers, p, sms, stream);
    }
    if (d->n_peers > 8 || d->mode != OLB_GEMM_DENSE || d->stage_flags == nullptr || d->a_peer_rows <= 0 ||
        d->a_peer_rows % BLOCK_M || d->my_peer < 0 || d->my_peer >= d->n_peers || d->M != d->n_peers * d->a_peer_rows)
      return -14;
    if (push ? (d->A_peers != nullptr || d->out_fp32 || d->accumulate)
             : (d->A_peers == nullptr || d->a_mn_major || d->a_rows < d->M || d->K % 8))
      return -14;
    PeerArg<true> peers{};
    peers.flags = d->stage_flags;
    peers.rows = d->a_peer_rows;
    peers.n = d->n_peers;
    peers.me = d->my_peer;
    if (push) {
      for (int r = 0; r < 8; ++r) {
        peers.push_dst[r] = d->C_peers[r < d->n_peers ? r : 0];
        if (reinterpret_cast<uintptr_t>(peers.push_dst[r]) & 15) return -14;
      }
      peers.push = 1;
      peers.flags_full = 4 * ((d->N + block_n - 1) / block_n);
      peers.c_base = d->C;
      peers.ldc = d->ldc;
      peers.row_vecs = d->N / 8;
      p.m_rotate_blocks = (((d->my_peer + 1) % d->n_peers) * d->a_peer_rows) / BLOCK_M;  // own rows last
    } else {
      for (int r = 0; r < 8; ++r) {
        peers.src[r] = d->A_peers[r < d->n_peers ? r : 0];
        if (reinterpret_cast<uintptr_t>(peers.src[r]) & 15) return -14;
      }
      peers.dst = const_cast<void*>(d->A);
      peers.ld = d->lda;
      peers.row_vecs = d->K / 8;
      p.m_rotate_blocks = (d->my_peer * d->a_peer_rows) / BLOCK_M;  // own rows first
    }
    return dispatch<true>(block_n, epi, tm, peers, p, sms, stream);
  }
  PeerArg<false> nopeers{};
  if (use_pair) {
    if (epi == OLB_EPI_SWIGLU) return launch_pair<false, EPI_SWIGLU>(tm, nopeers, p, sms, stream);
    if (epi == OLB_EPI_SWIGLU_BWD) return launch_pair<false, EPI_SWIGLU_BWD>(tm, nopeers, p, sms, stream);
    return launch_pair<false, EPI_PLAIN>(tm, nopeers, p, sms, stream);
  }
  if (epi == OLB_EPI_SWIGLU_BWD) return -16;
  return dispatch<false>(block_n, epi, tm, nopeers, p, sms, stream);
}
