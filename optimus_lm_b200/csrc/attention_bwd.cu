// Causal flash-attention backward for sm_100a (tcgen05 + TMEM), deterministic: every gradient element has
// exactly one writer, no atomics.
//
//   delta kernel : delta[b,h,s] = sum_d dO*O  and  lse2 = lse * log2(e), both stored negated   (one warp per row)
//   dK/dV kernel : one CTA per (batch, kv head, 128-row key tile); K and V tiles stay in shared memory,
//                  64-row Q / dO tiles of every query head of the group stream through a TMA ring:
//                    S^T = K Q^T, dP^T = V dO^T            (UMMA 128x64x16 into TMEM)
//                    P^T = exp2(S^T*c - lse2[q]),  dS^T = P^T o (dP^T - delta[q])   (8 warps, two threads per key row)
//                    dV += P^T dO,  dK += dS^T Q          (A = packed bf16 written back over the start of each
//                                                          thread's own score columns in TMEM, B = the streamed
//                                                          tile read MN-major)
//   dQ kernel    : one CTA per (batch, head, 128-row query tile); Q and dO stay, 64-row K / V tiles stream:
//                    S = Q K^T, dP = dO V^T, dS = P o (dP - delta[q]), dQ += dS K
// Both are one template: a resident pair R1/R2 (128 rows), a streamed pair T1/T2 (64 rows), X = R1 T1^T,
// Y = R2 T2^T, acc2 += dS T1 and (key mode only) acc1 += P T2.  Head dims as in the forward kernel:
// D in {64, 128, 192}, Dv in {64, 128}.  The reference relies on autograd through
// F.scaled_dot_product_attention (optimus/models/olmoe/modeling_olmoe.py:219-227) or through the eager
// softmax(QK^T)V of DeepSeek-V3 (optimus/models/deepseek_v3/modeling_deepseek_v3.py:359-369).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>

#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

int attn_tmap(CUtensorMap* map, const void* ptr, int Dh, int H, int S, int B, long long bs, long long ss, long long hs,
              int box_rows);

constexpr int BW_R = 128;  // resident rows per CTA
constexpr int BW_T = 64;   // streamed rows per step

template <int D1, int D2, bool KV_MODE>
struct BwdCfg {
  static constexpr int NB = (KV_MODE && D1 > 128) ? 1 : 2;  // score / dS buffers (TMEM)
  // Recompute warps: NG warps share each group of 32 rows (TMEM lanes) and split the 64 columns of a tile.  The
  // per-tile chain (wait, TMEM read, exp, TMEM write, signal) is latency-bound, so more warps with less
  // work each hide it better: four per lane group where the epilogue's 32-column pieces allow it.
  static constexpr int NG = (D1 == 128 && D2 == 128) ? 4 : 2;
  static constexpr int THREADS = 64 + 128 * NG;                // TMA warp, MMA warp, 4 * NG recompute warps
  static constexpr int R1_BYTES = BW_R * D1 * 2, R2_BYTES = BW_R * D2 * 2;
  static constexpr int T1_BYTES = BW_T * D1 * 2, T2_BYTES = BW_T * D2 * 2;
  // P and dS live in TMEM, so all of shared memory beyond the resident pair is the ring of streamed tiles: a tile
  // is requested one ring length ahead, and the load latency under load is more than one iteration
  static constexpr int TS_FIT = (232448 - 256 - 1024 - R1_BYTES - R2_BYTES) / (T1_BYTES + T2_BYTES);
  static constexpr int TS = TS_FIT > 6 ? 6 : TS_FIT;           // stages of the streamed-tile ring
  static constexpr int OFF_R1 = 0;
  static constexpr int OFF_R2 = OFF_R1 + R1_BYTES;
  static constexpr int OFF_T1 = OFF_R2 + R2_BYTES;
  static constexpr int OFF_T2 = OFF_T1 + TS * T1_BYTES;
  static constexpr int OFF_BAR = OFF_T2 + TS * T2_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
  static_assert(TS >= 2, "ring depth");
  static constexpr uint32_t TM_X = 0, TM_Y = BW_T * NB, TM_ACC1 = 2 * BW_T * NB;
  static constexpr uint32_t TM_ACC2 = KV_MODE ? TM_ACC1 + 128 : TM_ACC1;
  static_assert(TM_ACC2 + D1 <= 512 && D2 <= 128, "TMEM columns");
  static_assert(TOTAL <= 232448, "shared memory size");
};

struct AttnBwdParams {
  const float* lse2;   // [B, Hq, S] minus the log-sum-exp in base 2
  const float* delta;  // [B, Hq, S] minus delta
  __nv_bfloat16 *out1, *out2;  // key mode: dV, dK; query mode: unused, dQ
  long long o1_bs, o1_ss, o1_hs, o2_bs, o2_ss, o2_hs;
  int B, S, Hq, Hkv;
  float scale, scale_log2;
  int* status;
};

enum { BB_R = 0, BB_T_FULL0 = 1, BB_T_EMPTY0 = 7, BB_XY_FULL0 = 13, BB_DS_FULL0 = 15, BB_ACC = 17, BB_COUNT = 18 };

template <int D1, int D2, bool KV_MODE>
__global__ void __launch_bounds__((BwdCfg<D1, D2, KV_MODE>::THREADS), 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_r1, const __grid_constant__ CUtensorMap tm_r2,
                const __grid_constant__ CUtensorMap tm_t1, const __grid_constant__ CUtensorMap tm_t2,
                const AttnBwdParams p) {
  using L = BwdCfg<D1, D2, KV_MODE>;
  constexpr int NB = L::NB, TS = L::TS;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  auto bar = [&](int i) { return base + L::OFF_BAR + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::OFF_BAR + 8 * 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::OFF_BAR + 8 * 20 + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int b = blockIdx.z;
  // key mode: blockIdx.y = kv head, tile = key tile (low tiles have the most work and come first);
  // query mode: blockIdx.y = query head, heavy (late) query tiles first
  const int n_r_tiles = p.S / BW_R;
  const int rt = KV_MODE ? blockIdx.x : n_r_tiles - 1 - blockIdx.x;
  const int r0 = rt * BW_R;
  const int head_r = blockIdx.y;
  const int t_first = KV_MODE ? r0 / BW_T : 0;
  const int t_count = KV_MODE ? p.S / BW_T - t_first : (r0 + BW_R) / BW_T;
  const int n_iter = KV_MODE ? G * t_count : t_count;

  if (threadIdx.x == 0) {
    mbar_init(bar(BB_R), 1);
    for (int s = 0; s < 6; ++s) {
      mbar_init(bar(BB_T_FULL0 + s), 1);
      mbar_init(bar(BB_T_EMPTY0 + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(BB_XY_FULL0 + s), 1);
      mbar_init(bar(BB_DS_FULL0 + s), 4 * L::NG);
    }
    mbar_init(bar(BB_ACC), 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_r1);
    tma_prefetch_desc(&tm_r2);
    tma_prefetch_desc(&tm_t1);
    tma_prefetch_desc(&tm_t2);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // streamed head / row origin of iteration it
  auto t_head = [&](int it) { return KV_MODE ? head_r * G + it / t_count : head_r / G; };
  auto t_row0 = [&](int it) { return (t_first + (KV_MODE ? it % t_count : it)) * BW_T; };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      mbar_expect_tx(bar(BB_R), L::R1_BYTES + L::R2_BYTES);
#pragma unroll
      for (int a = 0; a < D1 / 64; ++a) tma_load_4d(base + L::OFF_R1 + a * (BW_R * 128), &tm_r1, bar(BB_R), a * 64, head_r, r0, b);
#pragma unroll
      for (int a = 0; a < D2 / 64; ++a) tma_load_4d(base + L::OFF_R2 + a * (BW_R * 128), &tm_r2, bar(BB_R), a * 64, head_r, r0, b);
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % TS;
        if (it >= TS && !mbar_wait(bar(BB_T_EMPTY0 + st), ((it / TS) - 1) & 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) break;
        const int th = t_head(it), tr = t_row0(it);
        mbar_expect_tx(bar(BB_T_FULL0 + st), L::T1_BYTES + L::T2_BYTES);
#pragma unroll
        for (int a = 0; a < D1 / 64; ++a)
          tma_load_4d(base + L::OFF_T1 + st * L::T1_BYTES + a * (BW_T * 128), &tm_t1, bar(BB_T_FULL0 + st), a * 64, th, tr, b);
#pragma unroll
        for (int a = 0; a < D2 / 64; ++a)
          tma_load_4d(base + L::OFF_T2 + st * L::T2_BYTES + a * (BW_T * 128), &tm_t2, bar(BB_T_FULL0 + st), a * 64, th, tr, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t idesc_xy = make_idesc_bf16(BW_R, BW_T, 0, 0);
      const uint32_t idesc_a1 = make_idesc_bf16(BW_R, D2, 0, 1);
      const uint32_t idesc_a2 = make_idesc_bf16(BW_R, D1, 0, 1);
      bool ok = mbar_wait(bar(BB_R), 0, p.status, ST_TIMEOUT_FULL, abort_flag);
      tc_fence_after();
      // Descriptors: the fields other than the start address are constant, and shared memory ends below 256 KB, so
      // moving a descriptor by a byte offset is one add on its low word.
      auto desc_at = [](uint64_t d, uint32_t byte_off) { return d + (byte_off >> 4); };
      const uint64_t dr1 = make_smem_desc(base + L::OFF_R1, 16, 1024), dr2 = make_smem_desc(base + L::OFF_R2, 16, 1024);
      constexpr int CPT = BW_T / L::NG;  // columns per recompute thread
      // column, inside a score buffer, of the packed bf16 of K step k (16 elements): the start of the owning
      // thread's own columns
      auto a_col = [](int k) { return static_cast<uint32_t>(((16 * k) / CPT) * CPT + ((16 * k) % CPT) / 2); };
      // acc += (P | dS)(u) x streamed tile of iteration u (A read from TMEM), then release that tile
      auto issue_acc = [&](int u) -> bool {
        const int s = u % NB, st = u % TS;
        if (!mbar_wait(bar(BB_DS_FULL0 + s), (u / NB) & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) return false;
        tc_fence_after();
        const uint64_t dt1 = make_smem_desc(base + L::OFF_T1 + st * L::T1_BYTES, BW_T * 128, 1024);
        const uint64_t dt2 = make_smem_desc(base + L::OFF_T2 + st * L::T2_BYTES, BW_T * 128, 1024);
#pragma unroll
        for (int k = 0; k < BW_T / 16; ++k) {
          if (KV_MODE)
            umma_ts(tmem + L::TM_ACC1, tmem + L::TM_X + s * BW_T + a_col(k), desc_at(dt2, k * 2048), idesc_a1,
                    (u > 0 || k > 0) ? 1u : 0u);
          umma_ts(tmem + L::TM_ACC2, tmem + L::TM_Y + s * BW_T + a_col(k), desc_at(dt1, k * 2048), idesc_a2,
                  (u > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(bar(BB_T_EMPTY0 + st));
        return true;
      };
      for (int it = 0; ok && it < n_iter; ++it) {
        const int s = it % NB, st = it % TS;
        // One score buffer: the products of the previous tile read P and dS from it, so they go first.  Two: the
        // buffer of tile it held P and dS of tile it-2, whose products were issued in the previous turn, and the
        // tcgen05.mma of one thread execute in issue order.
        if (NB == 1 && it >= 1 && !issue_acc(it - 1)) { ok = false; break; }
        if (!mbar_wait(bar(BB_T_FULL0 + st), (it / TS) & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint64_t dt1 = make_smem_desc(base + L::OFF_T1 + st * L::T1_BYTES, 16, 1024);
        const uint64_t dt2 = make_smem_desc(base + L::OFF_T2 + st * L::T2_BYTES, 16, 1024);
#pragma unroll
        for (int k = 0; k < D1 / 16; ++k)
          umma_ss(tmem + L::TM_X + s * BW_T, desc_at(dr1, (k / 4) * (BW_R * 128) + (k % 4) * 32),
                  desc_at(dt1, (k / 4) * (BW_T * 128) + (k % 4) * 32), idesc_xy, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < D2 / 16; ++k)
          umma_ss(tmem + L::TM_Y + s * BW_T, desc_at(dr2, (k / 4) * (BW_R * 128) + (k % 4) * 32),
                  desc_at(dt2, (k / 4) * (BW_T * 128) + (k % 4) * 32), idesc_xy, k > 0 ? 1u : 0u);
        umma_commit(bar(BB_XY_FULL0 + s));
        if (NB == 2 && it >= 1 && !issue_acc(it - 1)) { ok = false; break; }
      }
      if (ok && n_iter > 0 && issue_acc(n_iter - 1)) umma_commit(bar(BB_ACC));
    }
  } else {
    // ---------------------------------------------------------------- softmax recompute, dS, epilogue
    // Warps w, w+4, ... share the 32 rows (TMEM lanes) of lane group w % 4 and split the 64 columns of every tile.
    // (Giving the groups alternate tiles instead was measured slower: 1.67 ms against 1.36 ms for the
    // B4 S4096 H16 D128 backward.)
    constexpr int NG = L::NG;
    constexpr int CPT = BW_T / NG;   // columns per thread: 32 or 16
    const int lg = warp & 3;
    const int grp = (warp - 2) >> 2;
    const int c0 = grp * CPT;        // first column of this thread
    const int row = lg * 32 + lane;  // resident row == TMEM lane
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(lg * 32) << 16);
    bool ok = true;
    float my_nlse2 = 0.f, my_ndelta = 0.f;
    if (!KV_MODE) {
      const long long o = (static_cast<long long>(b) * p.Hq + head_r) * p.S + r0 + row;
      my_nlse2 = p.lse2[o];
      my_ndelta = p.delta[o];
    }
    int tq = 0, hq = 0;  // key mode: tile inside the query head, query head inside the group (no division per tile)
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it % NB;
      const int tr = (t_first + (KV_MODE ? tq : it)) * BW_T;
      const int th = KV_MODE ? head_r * G + hq : 0;
      if (KV_MODE && ++tq == t_count) {
        tq = 0;
        ++hq;
      }
      // rows are keys and columns queries in key mode, the other way round in query mode
      const bool diag = KV_MODE ? (tr < r0 + BW_R) : (tr + BW_T > r0);
      // key mode: the statistics of this tile's queries (negated log-sum-exp and delta), the same CPT values for every
      // thread of the warp, fetched before the wait for the scores so that their latency falls into it
      float4 nl4[CPT / 4], nd4[CPT / 4];
      if (KV_MODE) {
        const long long o = (static_cast<long long>(b) * p.Hq + th) * p.S + tr + c0;
#pragma unroll
        for (int i = 0; i < CPT / 4; ++i) {
          nl4[i] = __ldg(reinterpret_cast<const float4*>(p.lse2 + o) + i);
          nd4[i] = __ldg(reinterpret_cast<const float4*>(p.delta + o) + i);
        }
      }
      if (!mbar_wait(bar(BB_XY_FULL0 + s), (it / NB) & 1u, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t x[CPT], y[CPT];
      if constexpr (CPT == 32) {
        tmem_ld_32x32b_x32(lane_addr + L::TM_X + s * BW_T + c0, x);
        tmem_ld_32x32b_x32(lane_addr + L::TM_Y + s * BW_T + c0, y);
      } else {
        tmem_ld_32x32b_x16(lane_addr + L::TM_X + s * BW_T + c0, x);
        tmem_ld_32x32b_x16(lane_addr + L::TM_Y + s * BW_T + c0, y);
      }
      tmem_ld_wait();
      uint32_t pp[CPT / 2], ds[CPT / 2];
      // P = 2^(x c - lse2) and dS = P (y - delta), two elements per instruction (packed fp32); the statistics are stored
      // negated so that both are one fused operation.  Tiles off the diagonal take the path without comparisons;
      // on the diagonal a masked score is replaced by -FLT_MAX, which makes P and with it dS exactly zero.
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 my_nl2 = make_float2(my_nlse2, my_nlse2), my_nd2 = make_float2(my_ndelta, my_ndelta);
#pragma unroll
      for (int i8 = 0; i8 < CPT / 8; ++i8) {
        float2 nl2[4], nd2[4];
        if (KV_MODE) {
          const float4 a0 = nl4[2 * i8], a1 = nl4[2 * i8 + 1], b0 = nd4[2 * i8], b1 = nd4[2 * i8 + 1];
          nl2[0] = make_float2(a0.x, a0.y); nl2[1] = make_float2(a0.z, a0.w);
          nl2[2] = make_float2(a1.x, a1.y); nl2[3] = make_float2(a1.z, a1.w);
          nd2[0] = make_float2(b0.x, b0.y); nd2[1] = make_float2(b0.z, b0.w);
          nd2[2] = make_float2(b1.x, b1.y); nd2[3] = make_float2(b1.z, b1.w);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x0 = __uint_as_float(x[i8 * 8 + 2 * e]), x1 = __uint_as_float(x[i8 * 8 + 2 * e + 1]);
          if (diag) {
            const int col = c0 + i8 * 8 + 2 * e;
            const int kv = KV_MODE ? r0 + row : tr + col;       // of the first element of the pair
            const int qi = KV_MODE ? tr + col : r0 + row;
            if (kv > qi) x0 = -FLT_MAX;
            if ((KV_MODE ? kv : kv + 1) > (KV_MODE ? qi + 1 : qi)) x1 = -FLT_MAX;
          }
          const float2 t2 = fma2(make_float2(x0, x1), sc2, KV_MODE ? nl2[e] : my_nl2);
          float2 pr;
          pr.x = ex2_approx(t2.x);
          pr.y = ex2_approx(t2.y);
          const float2 dd = add2(make_float2(__uint_as_float(y[i8 * 8 + 2 * e]), __uint_as_float(y[i8 * 8 + 2 * e + 1])),
                                 KV_MODE ? nd2[e] : my_nd2);
          const float2 dv = mul2(pr, dd);
          pp[i8 * 4 + e] = pack_bf16(pr.x, pr.y);
          ds[i8 * 4 + e] = pack_bf16(dv.x, dv.y);
        }
      }
      // dS (and in key mode P) as packed bf16 over the first half of this thread's own score columns: nobody else
      // reads or writes those, and the products that consume them are issued only after every warp has signalled
      if constexpr (CPT == 32) {
        tmem_st_32x32b_x16(lane_addr + L::TM_Y + s * BW_T + c0, ds);
        if (KV_MODE) tmem_st_32x32b_x16(lane_addr + L::TM_X + s * BW_T + c0, pp);
      } else {
        tmem_st_32x32b_x8(lane_addr + L::TM_Y + s * BW_T + c0, ds);
        if (KV_MODE) tmem_st_32x32b_x8(lane_addr + L::TM_X + s * BW_T + c0, pp);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BB_DS_FULL0 + s));
    }
    if (ok && n_iter > 0 && mbar_wait(bar(BB_ACC), 0, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) {
      tc_fence_after();
      // the warps sharing a lane group store equal pieces of the columns
      auto store_rows = [&](uint32_t tm_col, int width, __nv_bfloat16* out, long long bs, long long ss, long long hs, float mul) {
        const int half = width / NG;
        const int c = grp;
        __nv_bfloat16* orow = out + static_cast<long long>(b) * bs + static_cast<long long>(r0 + row) * ss +
                              static_cast<long long>(head_r) * hs + c * half;
#pragma unroll 1
        for (int cc = 0; cc < half / 32; ++cc) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(lane_addr + tm_col + c * half + cc * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[8 * g]) * mul, __uint_as_float(r[8 * g + 1]) * mul);
            v.y = pack_bf16(__uint_as_float(r[8 * g + 2]) * mul, __uint_as_float(r[8 * g + 3]) * mul);
            v.z = pack_bf16(__uint_as_float(r[8 * g + 4]) * mul, __uint_as_float(r[8 * g + 5]) * mul);
            v.w = pack_bf16(__uint_as_float(r[8 * g + 6]) * mul, __uint_as_float(r[8 * g + 7]) * mul);
            *reinterpret_cast<uint4*>(orow + cc * 32 + g * 8) = v;
          }
        }
      };
      if (KV_MODE) store_rows(L::TM_ACC1, D2, p.out1, p.o1_bs, p.o1_ss, p.o1_hs, 1.f);
      store_rows(L::TM_ACC2, D1, p.out2, p.o2_bs, p.o2_ss, p.o2_hs, p.scale);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// delta[b,h,s] = -sum_d dO[b,s,h,d] * O[b,s,h,d];  lse2 = -lse * log2(e): both stored negated, which is how the
// recompute warps add them.  Eight lanes per (b, s, h) row, four rows per warp: every lane has up to four 16-byte
// loads in flight.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  const float* __restrict__ lse, float* __restrict__ delta, float* __restrict__ lse2,
                                  long long o_bs, long long o_ss, long long o_hs, long long do_bs, long long do_ss,
                                  long long do_hs, int B, int S, int H, int Dv) {
  const long long n_rows = static_cast<long long>(B) * S * H;
  const int lane = threadIdx.x & 31, sub = lane & 7;
  long long w = ((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * 4 + (lane >> 3);
  const bool live = w < n_rows;
  if (!live) w = n_rows - 1;  // keep the lane in the shuffles
  const int h = static_cast<int>(w % H);
  const int s = static_cast<int>((w / H) % S);
  const int b = static_cast<int>(w / (static_cast<long long>(H) * S));
  const __nv_bfloat16* orow = o + b * o_bs + s * o_ss + h * o_hs;
  const __nv_bfloat16* drow = dout + b * do_bs + s * do_ss + h * do_hs;
  float acc = 0.f;
  for (int c = sub * 8; c < Dv; c += 64) {
    const uint4 a = *reinterpret_cast<const uint4*>(orow + c);
    const uint4 g = *reinterpret_cast<const uint4*>(drow + c);
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack_bf16(av[i]), y = unpack_bf16(gv[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int m = 4; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
  if (live && sub == 0) {
    const long long idx = (static_cast<long long>(b) * H + h) * S + s;
    delta[idx] = -acc;
    lse2[idx] = -lse[idx] * 1.4426950408889634f;
  }
}

template <int D, int DV>
static int launch_bwd(const olb_attn_bwd_desc* d, cudaStream_t stream) {
  using LK = BwdCfg<D, DV, true>;
  using LQ = BwdCfg<D, DV, false>;
  // the attribute belongs to the function on one device: once per device, not once per process
  static bool configured_on[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  bool& configured = configured_on[dev];
  if (!configured) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<D, DV, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, LK::TOTAL) != cudaSuccess ||
        cudaFuncSetAttribute(attn_bwd_kernel<D, DV, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, LQ::TOTAL) != cudaSuccess)
      return -3;
    configured = true;
  }
  const long long n_rows = static_cast<long long>(d->B) * d->S * d->Hq;
  float* delta = d->delta;
  float* lse2 = d->delta + n_rows;
  attn_delta_kernel<<<static_cast<unsigned>((n_rows * 8 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(d->o), static_cast<const __nv_bfloat16*>(d->dout), d->lse, delta, lse2, d->o_bs,
      d->o_ss, d->o_hs, d->do_bs, d->do_ss, d->do_hs, d->B, d->S, d->Hq, d->Dv);

  CUtensorMap q128, do128, k128, v128, q64, do64, k64, v64;
  if (attn_tmap(&k128, d->k, D, d->Hkv, d->S, d->B, d->k_bs, d->k_ss, d->k_hs, BW_R)) return -4;
  if (attn_tmap(&v128, d->v, DV, d->Hkv, d->S, d->B, d->v_bs, d->v_ss, d->v_hs, BW_R)) return -4;
  if (attn_tmap(&q64, d->q, D, d->Hq, d->S, d->B, d->q_bs, d->q_ss, d->q_hs, BW_T)) return -4;
  if (attn_tmap(&do64, d->dout, DV, d->Hq, d->S, d->B, d->do_bs, d->do_ss, d->do_hs, BW_T)) return -4;
  if (attn_tmap(&q128, d->q, D, d->Hq, d->S, d->B, d->q_bs, d->q_ss, d->q_hs, BW_R)) return -4;
  if (attn_tmap(&do128, d->dout, DV, d->Hq, d->S, d->B, d->do_bs, d->do_ss, d->do_hs, BW_R)) return -4;
  if (attn_tmap(&k64, d->k, D, d->Hkv, d->S, d->B, d->k_bs, d->k_ss, d->k_hs, BW_T)) return -4;
  if (attn_tmap(&v64, d->v, DV, d->Hkv, d->S, d->B, d->v_bs, d->v_ss, d->v_hs, BW_T)) return -4;

  AttnBwdParams p;
  p.lse2 = lse2;
  p.delta = delta;
  p.B = d->B;
  p.S = d->S;
  p.Hq = d->Hq;
  p.Hkv = d->Hkv;
  p.scale = d->scale;
  p.scale_log2 = d->scale * 1.4426950408889634f;
  p.status = d->status;
  // dK / dV
  p.out1 = static_cast<__nv_bfloat16*>(d->dv);
  p.o1_bs = d->dv_bs; p.o1_ss = d->dv_ss; p.o1_hs = d->dv_hs;
  p.out2 = static_cast<__nv_bfloat16*>(d->dk);
  p.o2_bs = d->dk_bs; p.o2_ss = d->dk_ss; p.o2_hs = d->dk_hs;
  attn_bwd_kernel<D, DV, true><<<dim3(d->S / BW_R, d->Hkv, d->B), LK::THREADS, LK::TOTAL, stream>>>(k128, v128, q64, do64, p);
  // dQ
  p.out1 = nullptr;
  p.out2 = static_cast<__nv_bfloat16*>(d->dq);
  p.o2_bs = d->dq_bs; p.o2_ss = d->dq_ss; p.o2_hs = d->dq_hs;
  attn_bwd_kernel<D, DV, false><<<dim3(d->S / BW_R, d->Hq, d->B), LQ::THREADS, LQ::TOTAL, stream>>>(q128, do128, k64, v64, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace olb

extern "C" int olb_attn_bwd(const olb_attn_bwd_desc* d, cudaStream_t stream) {
  using namespace olb;
  if (d->S % BW_R || d->Hq % d->Hkv || d->delta == nullptr) return -1;
  const long long strides[] = {d->q_bs, d->q_ss, d->q_hs, d->k_bs, d->k_ss, d->k_hs, d->v_bs, d->v_ss, d->v_hs,
                               d->o_bs, d->o_ss, d->o_hs, d->do_bs, d->do_ss, d->do_hs, d->dq_bs, d->dq_ss, d->dq_hs,
                               d->dk_bs, d->dk_ss, d->dk_hs, d->dv_bs, d->dv_ss, d->dv_hs};
  for (long long s : strides)
    if (s % 8) return -2;
  const void* ptrs[] = {d->q, d->k, d->v, d->o, d->dout, d->dq, d->dk, d->dv};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return -2;
  if (d->D == 128 && d->Dv == 128) return launch_bwd<128, 128>(d, stream);
  if (d->D == 64 && d->Dv == 64) return launch_bwd<64, 64>(d, stream);
  if (d->D == 192 && d->Dv == 128) return launch_bwd<192, 128>(d, stream);
  return -6;
}
