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
//   * warps 2-5: epilogue - tcgen05.ld the accumulator (each warp owns 32 TMEM lanes),
//                convert and store / accumulate into C while the next tile's main loop runs
//   * warps 6-9: only in the variants with a fused collective (PeerArg<true>): copy the other GPUs' rows of A into the local
//                gathered copy over NVLink while the tiles of the local rows are computed
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
};

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
  const int* src_of;
  const int* k_of;
  int T, topk;
};
constexpr int STAGER_WARPS = 4;
constexpr int NUM_THREADS_STAGED = NUM_THREADS + 32 * STAGER_WARPS;

template <int BLOCK_N>
struct SmemLayout {
  static constexpr int B_STAGE_BYTES = BLOCK_N * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = (BLOCK_N == 256) ? 4 : (BLOCK_N == 128 ? 6 : 8);
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + slack for 1024B alignment
};

struct TileInfo {
  int m0, n0;        // element offsets of the tile in C
  int kb_begin, kb_end;  // K range in units of BLOCK_K
  int expert;
};

// Map a linear tile id to its coordinates.  Returns false when `t` is past the last tile.
template <int BLOCK_N>
__device__ __forceinline__ bool get_tile(const GemmParams& p, int t, int num_m_blocks, int blk0, TileInfo& ti) {
  const int num_n_blocks = (p.N + BLOCK_N - 1) / BLOCK_N;
  if (p.mode == OLB_GEMM_RAGGED_K) {
    const int per_expert = num_m_blocks * num_n_blocks;
    if (t >= per_expert * p.num_experts) return false;
    const int e = t / per_expert;
    const int r = t - e * per_expert;
    ti.expert = e;
    ti.m0 = (r / num_n_blocks) * BLOCK_M;
    ti.n0 = (r % num_n_blocks) * BLOCK_N;
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
  ti.n0 = n_blk * BLOCK_N;
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

template <int BLOCK_N, bool PEER>
__global__ void __launch_bounds__(PEER ? NUM_THREADS_STAGED : NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_b2, const __grid_constant__ PeerArg<PEER> peers,
                 const GemmParams p) {
  using L = SmemLayout<BLOCK_N>;
  constexpr int STAGES = L::STAGES;
  constexpr uint32_t TMEM_COLS = (2 * BLOCK_N < 32) ? 32 : 2 * BLOCK_N;

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
      for (int t = blockIdx.x; ok && get_tile<BLOCK_N>(p, t, num_m_blocks, blk0, ti); t += gridDim.x) {
        if constexpr (PEER) {
          // rows of another GPU: wait until the stagers have brought the whole row block into the local copy
          if (!peers.push && ti.m0 / peers.rows != peers.me) {
            if (!wait_count(peers.flags + ti.m0 / BLOCK_M, min(BLOCK_M, p.M - ti.m0), p.status, abort_flag)) {
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
      for (int t = blockIdx.x; ok && get_tile<BLOCK_N>(p, t, num_m_blocks, blk0, ti); t += gridDim.x) {
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
    for (int t = blockIdx.x; get_tile<BLOCK_N>(p, t, num_m_blocks, blk0, ti); t += gridDim.x) {
      const int row = ti.m0 + lane_group * 32 + lane;
      const bool row_ok = row < p.M;
      const bool has_k = ti.kb_end > ti.kb_begin;
      char* c_row;
      {
        long long off = static_cast<long long>(row) * p.ldc + ti.n0;
        if (p.mode == OLB_GEMM_RAGGED_K) off += static_cast<long long>(ti.expert) * p.c_expert_stride;
        c_row = static_cast<char*>(p.C) + off * (p.out_fp32 ? 4 : 2);
      }
      if (has_k) {
        if (!mbar_wait(acc_full_bar(acc), acc_phase, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) break;
        tc_fence_after();
      } else if (p.accumulate) {
        continue;  // nothing to add
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + acc * BLOCK_N;
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
      if constexpr (PEER) {
        if (peers.push) {  // this warp's 32 rows of the tile are stored: let the stagers know
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
  }

  if constexpr (PEER) {
    if (warp >= 6) {
      // ---------------------------------------------------------- stagers (warps 6..9): the all-gather
      // Remote rows in the order the tiles need them: the peer after this one first.  Every CTA's stagers take rows
      // of the same block at the same time, so blocks complete one after the other.  The gather waits for nothing;
      // the push waits (bounded) for this GPU's own epilogues.
      const long long total = peers.push == 2 ? min(static_cast<long long>(num_m_blocks) * BLOCK_M, static_cast<long long>(p.M))
                                              : static_cast<long long>(peers.n - 1) * peers.rows;
      int ready_blk = -1;
      bool ok = true;
      for (long long u = blockIdx.x * STAGER_WARPS + (warp - 6); ok && u < total;
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
  }

  tc_fence_before();
  __syncthreads();
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

// 2D bf16 tensor map with 128B swizzle.  dims/box are {inner, outer}.
int make_tmap_2d_bf16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                      uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
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

template <int BLOCK_N, bool PEER>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const PeerArg<PEER>& peers,
                  const GemmParams& p, int num_sms, cudaStream_t stream) {
  using L = SmemLayout<BLOCK_N>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BLOCK_N, PEER>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return -3;
    configured = true;
  }
  long long tiles;
  const long long nm = (p.M + BLOCK_M - 1) / BLOCK_M, nn = (p.N + BLOCK_N - 1) / BLOCK_N;
  tiles = nm * nn * (p.mode == OLB_GEMM_RAGGED_K ? p.num_experts : 1);
  int grid = static_cast<int>(tiles < num_sms ? tiles : num_sms);
  if (grid <= 0) return 0;
  gemm_bf16_kernel<BLOCK_N, PEER><<<grid, PEER ? NUM_THREADS_STAGED : NUM_THREADS, L::TOTAL, stream>>>(ta, tb, tb2, peers, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace olb

extern "C" int olb_gemm_bf16(const olb_gemm_desc* d, cudaStream_t stream) {
  using namespace olb;
  static const bool debug = getenv("OLB_DEBUG_GEMM") != nullptr;
  if (debug) {
    fprintf(stderr, "[olb_gemm] M=%d N=%d K=%d a_mn=%d b_mn=%d mode=%d lda=%lld ldb=%lld ldc=%lld a_rows=%lld b_rows=%lld "
            "acc=%d fp32=%d A=%p B=%p C=%p meta=%p\n", d->M, d->N, d->K, d->a_mn_major, d->b_mn_major, d->mode, d->lda,
            d->ldb, d->ldc, d->a_rows, d->b_rows, d->accumulate, d->out_fp32, d->A, d->B, d->C, (const void*)d->meta);
    fflush(stderr);
  }
  if (d->M <= 0 || d->N <= 0) return 0;
  if ((d->lda % 8) || (d->ldb % 8) || (d->ldc % 8) || (d->N % 8) || (reinterpret_cast<uintptr_t>(d->A) & 15) ||
      (reinterpret_cast<uintptr_t>(d->B) & 15) || (reinterpret_cast<uintptr_t>(d->C) & 15))
    return -10;
  int block_n = d->block_n;
  if (block_n == 0) {
    if (d->mode != OLB_GEMM_DENSE) {
      block_n = (d->N % 256 == 0) ? 256 : (d->N % 128 == 0 ? 128 : 64);
      if (d->N % 64) return -11;
    } else {
      block_n = d->N > 128 ? 256 : (d->N > 64 ? 128 : 64);
    }
  }
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }

  // cuTensorMapEncodeTiled is a driver call and needs a current context in the calling thread.
  // A thread that has only been handed tensors (an autograd worker whose first CUDA work is this
  // GEMM) has none yet; one runtime call binds the primary context.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  CUtensorMap ta, tb;
  int rc;
  // A: K-major -> global [a_rows, K] (inner K); MN-major -> global [K rows, M] (inner M).
  if (!d->a_mn_major)
    rc = make_tmap_2d_bf16(&ta, d->A, d->K, d->a_rows, d->lda * 2, BLOCK_K, BLOCK_M);
  else
    rc = make_tmap_2d_bf16(&ta, d->A, d->M, d->a_rows, d->lda * 2, 64, BLOCK_K);
  if (rc) return rc;
  if (!d->b_mn_major)
    rc = make_tmap_2d_bf16(&tb, d->B, d->K, d->b_rows, d->ldb * 2, BLOCK_K, block_n);
  else
    rc = make_tmap_2d_bf16(&tb, d->B, d->N, d->b_rows, d->ldb * 2, 64, BLOCK_K);
  if (rc) return rc;
  // optional second B (same layout) for the K range [k_split, K)
  CUtensorMap tb2 = tb;
  int kb_split = 0;
  if (d->B2 != nullptr && d->k_split > 0) {
    if (d->k_split % BLOCK_K || d->k_split >= d->K || d->mode == OLB_GEMM_RAGGED_K || (reinterpret_cast<uintptr_t>(d->B2) & 15))
      return -13;
    const int k1 = d->k_split, k2 = d->K - d->k_split;
    // each map covers only its own K extent, so that reads past it are zero-filled as usual
    if (!d->b_mn_major) {
      rc = make_tmap_2d_bf16(&tb, d->B, k1, d->b_rows, d->ldb * 2, BLOCK_K, block_n);
      if (!rc) rc = make_tmap_2d_bf16(&tb2, d->B2, k2, d->b_rows, d->ldb * 2, BLOCK_K, block_n);
    } else {
      rc = make_tmap_2d_bf16(&tb2, d->B2, d->N, d->b_rows, d->ldb * 2, 64, BLOCK_K);
    }
    if (rc) return rc;
    kb_split = d->k_split / BLOCK_K;
  }

  if (debug) {
    fprintf(stderr, "[olb_gemm] tensor maps ok, block_n=%d\n", block_n);
    fflush(stderr);
  }
  GemmParams p;
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
  const int sms = d->max_ctas > 0 && d->max_ctas < num_sms ? d->max_ctas : num_sms;
  if (d->n_peers > 0) {
    // All-gather of A's rows fused into the GEMM (see PeerArg<true>).
    const bool push = d->C_peers != nullptr;
    if (d->mode == OLB_GEMM_RAGGED_M) {
      // Expert-parallel combine transport: finished rows of C go to the owners of their tokens.
      if (!push || d->n_peers > 8 || d->stage_flags == nullptr || d->ep_src_of == nullptr || d->ep_k_of == nullptr ||
          d->ep_tokens <= 0 || d->ep_topk <= 0 || d->out_fp32 || d->accumulate || d->blk_range != nullptr || d->N % 8)
        return -14;
      PeerArg<true> peers{};
      for (int r = 0; r < 8; ++r) {
        peers.push_dst[r] = d->C_peers[r < d->n_peers ? r : 0];
        if (reinterpret_cast<uintptr_t>(peers.push_dst[r]) & 15) return -14;
      }
      peers.flags = d->stage_flags;
      peers.n = d->n_peers;
      peers.me = d->my_peer;
      peers.push = 2;
      peers.flags_full = 4 * ((d->N + block_n - 1) / block_n);
      peers.c_base = d->C;
      peers.ldc = d->ldc;
      peers.ld = d->N;
      peers.row_vecs = d->N / 8;
      peers.src_of = d->ep_src_of;
      peers.k_of = d->ep_k_of;
      peers.T = d->ep_tokens;
      peers.topk = d->ep_topk;
      switch (block_n) {
        case 256: return launch<256, true>(ta, tb, tb2, peers, p, sms, stream);
        case 128: return launch<128, true>(ta, tb, tb2, peers, p, sms, stream);
        case 64: return launch<64, true>(ta, tb, tb2, peers, p, sms, stream);
        default: return -12;
      }
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
    switch (block_n) {
      case 256: return launch<256, true>(ta, tb, tb2, peers, p, sms, stream);
      case 128: return launch<128, true>(ta, tb, tb2, peers, p, sms, stream);
      case 64: return launch<64, true>(ta, tb, tb2, peers, p, sms, stream);
      default: return -12;
    }
  }
  PeerArg<false> nopeers{};
  switch (block_n) {
    case 256: return launch<256, false>(ta, tb, tb2, nopeers, p, sms, stream);
    case 128: return launch<128, false>(ta, tb, tb2, nopeers, p, sms, stream);
    case 64: return launch<64, false>(ta, tb, tb2, nopeers, p, sms, stream);
    default: return -12;
  }
}
