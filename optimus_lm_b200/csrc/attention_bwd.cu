// Causal flash-attention backward for sm_100a (tcgen05 + TMEM), deterministic: every gradient element has
// exactly one writer, no atomics.
//
//   delta kernel : delta[b,h,s] = sum_d dO*O  and  lse2 = lse * log2(e)            (one warp per row)
//   dK/dV kernel : one CTA per (batch, kv head, 128-row key tile); K and V tiles stay in shared memory,
//                  64-row Q / dO tiles of every query head of the group stream through a TMA ring:
//                    S^T = K Q^T, dP^T = V dO^T            (UMMA 128x64x16 into TMEM)
//                    P^T = exp2(S^T*c - lse2[q]),  dS^T = P^T o (dP^T - delta[q])   (8 warps, two threads per key row)
//                    dV += P^T dO,  dK += dS^T Q          (A = bf16 tiles written to swizzled shared memory,
//                                                          B = the streamed tile read MN-major)
//   dQ kernel    : one CTA per (batch, head, 128-row query tile); Q and dO stay, 64-row K / V tiles stream:
//                    S = Q K^T, dP = dO V^T, dS = P o (dP - delta[q]), dQ += dS K
// Both are one template: a resident pair R1/R2 (128 rows), a streamed pair T1/T2 (64 rows), X = R1 T1^T,
// Y = R2 T2^T, acc2 += dS T1 and (key mode only) acc1 += P T2.  Head dims as in the forward kernel:
// D in {64, 128, 192}, Dv in {64, 128}.  The reference relies on autograd through
// F.scaled_dot_product_attention (optimus/models/olmoe/modeling_olmoe.py:219-227) or through the eager
// softmax(QK^T)V of DeepSeek-V3 (optimus/models/deepseek_v3/modeling_deepseek_v3.py:359-369).
#include <cuda.h>
#include <cuda_runtime.h>

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
  static constexpr int NB = (KV_MODE && D1 > 128) ? 1 : 2;  // score / dS buffers
  static constexpr int TS = (D1 > 128) ? 2 : 3;               // stages of the streamed-tile ring
  // Recompute warps: NG warps share each group of 32 rows (TMEM lanes) and split the 64 columns of a tile.  The
  // per-tile chain (wait, TMEM read, exp, shared-memory write, signal) is latency-bound, so more warps with less
  // work each hide it better: four per lane group where the epilogue's 32-column pieces allow it.
  static constexpr int NG = (D1 == 128 && D2 == 128) ? 4 : 2;
  static constexpr int THREADS = 64 + 128 * NG;                // TMA warp, MMA warp, 4 * NG recompute warps
  static constexpr int R1_BYTES = BW_R * D1 * 2, R2_BYTES = BW_R * D2 * 2;
  static constexpr int T1_BYTES = BW_T * D1 * 2, T2_BYTES = BW_T * D2 * 2;
  static constexpr int DS_BYTES = BW_R * BW_T * 2;
  static constexpr int OFF_R1 = 0;
  static constexpr int OFF_R2 = OFF_R1 + R1_BYTES;
  static constexpr int OFF_T1 = OFF_R2 + R2_BYTES;
  static constexpr int OFF_T2 = OFF_T1 + TS * T1_BYTES;
  static constexpr int OFF_DS = OFF_T2 + TS * T2_BYTES;
  static constexpr int OFF_P = OFF_DS + NB * DS_BYTES;
  static constexpr int OFF_BAR = OFF_P + (KV_MODE ? NB * DS_BYTES : 0);
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
  static constexpr uint32_t TM_X = 0, TM_Y = BW_T * NB, TM_ACC1 = 2 * BW_T * NB;
  static constexpr uint32_t TM_ACC2 = KV_MODE ? TM_ACC1 + 128 : TM_ACC1;
  static_assert(TM_ACC2 + D1 <= 512 && D2 <= 128, "TMEM columns");
  static_assert(TOTAL <= 232448, "shared memory size");
};

struct AttnBwdParams {
  const float* lse2;   // [B, Hq, S] log-sum-exp in base 2
  const float* delta;  // [B, Hq, S]
  __nv_bfloat16 *out1, *out2;  // key mode: dV, dK; query mode: unused, dQ
  long long o1_bs, o1_ss, o1_hs, o2_bs, o2_ss, o2_hs;
  int B, S, Hq, Hkv;
  float scale, scale_log2;
  int* status;
};

enum { BB_R = 0, BB_T_FULL0 = 1, BB_T_EMPTY0 = 4, BB_XY_FULL0 = 7, BB_XY_EMPTY0 = 9, BB_DS_FULL0 = 11, BB_DS_EMPTY0 = 13,
       BB_ACC = 15, BB_COUNT = 16 };

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
    for (int s = 0; s < 3; ++s) {
      mbar_init(bar(BB_T_FULL0 + s), 1);
      mbar_init(bar(BB_T_EMPTY0 + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(BB_XY_FULL0 + s), 1);
      mbar_init(bar(BB_XY_EMPTY0 + s), 4 * L::NG);
      mbar_init(bar(BB_DS_FULL0 + s), 4 * L::NG);
      mbar_init(bar(BB_DS_EMPTY0 + s), 1);
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
      // acc += (P | dS)(u) x streamed tile of iteration u, then release that tile and the dS buffer
      auto issue_acc = [&](int u) -> bool {
        const int s = u % NB, st = u % TS;
        if (!mbar_wait(bar(BB_DS_FULL0 + s), (u / NB) & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) return false;
        tc_fence_after();
        const uint32_t t1 = base + L::OFF_T1 + st * L::T1_BYTES, t2 = base + L::OFF_T2 + st * L::T2_BYTES;
#pragma unroll
        for (int k = 0; k < BW_T / 16; ++k) {
          if (KV_MODE) {
            const uint64_t da = make_smem_desc(base + L::OFF_P + s * L::DS_BYTES + k * 32, 16, 1024);
            const uint64_t db = make_smem_desc(t2 + k * 2048, BW_T * 128, 1024);
            umma_ss(tmem + L::TM_ACC1, da, db, idesc_a1, (u > 0 || k > 0) ? 1u : 0u);
          }
          const uint64_t da = make_smem_desc(base + L::OFF_DS + s * L::DS_BYTES + k * 32, 16, 1024);
          const uint64_t db = make_smem_desc(t1 + k * 2048, BW_T * 128, 1024);
          umma_ss(tmem + L::TM_ACC2, da, db, idesc_a2, (u > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(bar(BB_T_EMPTY0 + st));
        umma_commit(bar(BB_DS_EMPTY0 + s));
        return true;
      };
      for (int it = 0; ok && it < n_iter; ++it) {
        const int s = it % NB, st = it % TS;
        if (!mbar_wait(bar(BB_T_FULL0 + st), (it / TS) & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) { ok = false; break; }
        if (it >= NB && !mbar_wait(bar(BB_XY_EMPTY0 + s), ((it / NB) - 1) & 1u, p.status, ST_TIMEOUT_ACC_EMPTY, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t1 = base + L::OFF_T1 + st * L::T1_BYTES, t2 = base + L::OFF_T2 + st * L::T2_BYTES;
#pragma unroll
        for (int k = 0; k < D1 / 16; ++k) {
          const uint64_t da = make_smem_desc(base + L::OFF_R1 + (k / 4) * (BW_R * 128) + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(t1 + (k / 4) * (BW_T * 128) + (k % 4) * 32, 16, 1024);
          umma_ss(tmem + L::TM_X + s * BW_T, da, db, idesc_xy, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D2 / 16; ++k) {
          const uint64_t da = make_smem_desc(base + L::OFF_R2 + (k / 4) * (BW_R * 128) + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(t2 + (k / 4) * (BW_T * 128) + (k % 4) * 32, 16, 1024);
          umma_ss(tmem + L::TM_Y + s * BW_T, da, db, idesc_xy, k > 0 ? 1u : 0u);
        }
        umma_commit(bar(BB_XY_FULL0 + s));
        if (it >= 1 && !issue_acc(it - 1)) { ok = false; break; }
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
    float my_lse2 = 0.f, my_delta = 0.f;
    if (!KV_MODE) {
      const long long o = (static_cast<long long>(b) * p.Hq + head_r) * p.S + r0 + row;
      my_lse2 = p.lse2[o];
      my_delta = p.delta[o];
    }
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it % NB;
      const int tr = t_row0(it);
      if (!mbar_wait(bar(BB_XY_FULL0 + s), (it / NB) & 1u, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) { ok = false; break; }
      if (it >= NB && !mbar_wait(bar(BB_DS_EMPTY0 + s), ((it / NB) - 1) & 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // rows are keys and columns queries in key mode, the other way round in query mode
      const bool diag = KV_MODE ? (tr < r0 + BW_R) : (tr + BW_T > r0);
      const float* lse_col = nullptr;
      const float* dl_col = nullptr;
      if (KV_MODE) {
        const long long o = (static_cast<long long>(b) * p.Hq + t_head(it)) * p.S + tr + c0;
        lse_col = p.lse2 + o;
        dl_col = p.delta + o;
      }
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
#pragma unroll
      for (int i8 = 0; i8 < CPT / 8; ++i8) {
        float l2[8], dl[8];
        if (KV_MODE) {
          // all threads read the same 8 query statistics: two broadcast 16-byte loads each
          const float4 a0 = __ldg(reinterpret_cast<const float4*>(lse_col + i8 * 8));
          const float4 a1 = __ldg(reinterpret_cast<const float4*>(lse_col + i8 * 8 + 4));
          const float4 b0 = __ldg(reinterpret_cast<const float4*>(dl_col + i8 * 8));
          const float4 b1 = __ldg(reinterpret_cast<const float4*>(dl_col + i8 * 8 + 4));
          l2[0] = a0.x; l2[1] = a0.y; l2[2] = a0.z; l2[3] = a0.w; l2[4] = a1.x; l2[5] = a1.y; l2[6] = a1.z; l2[7] = a1.w;
          dl[0] = b0.x; dl[1] = b0.y; dl[2] = b0.z; dl[3] = b0.w; dl[4] = b1.x; dl[5] = b1.y; dl[6] = b1.z; dl[7] = b1.w;
        }
        float pv[8], dv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int col = c0 + i8 * 8 + e;
          const int kv = KV_MODE ? r0 + row : tr + col;
          const int qi = KV_MODE ? tr + col : r0 + row;
          const bool valid = !diag || kv <= qi;
          const float pr = valid ? ex2_approx(__uint_as_float(x[i8 * 8 + e]) * p.scale_log2 - (KV_MODE ? l2[e] : my_lse2)) : 0.f;
          pv[e] = pr;
          dv[e] = pr * (__uint_as_float(y[i8 * 8 + e]) - (KV_MODE ? dl[e] : my_delta));
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          pp[i8 * 4 + e] = pack_bf16(pv[2 * e], pv[2 * e + 1]);
          ds[i8 * 4 + e] = pack_bf16(dv[2 * e], dv[2 * e + 1]);
        }
      }
#pragma unroll
      for (int q = 0; q < CPT / 8; ++q) {
        const int chunk = grp * (CPT / 8) + q;  // 16-byte chunk of the 128-byte row
        const uint32_t off = row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + L::OFF_DS + s * L::DS_BYTES + off),
                     "r"(ds[4 * q]), "r"(ds[4 * q + 1]), "r"(ds[4 * q + 2]), "r"(ds[4 * q + 3])
                     : "memory");
        if (KV_MODE)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + L::OFF_P + s * L::DS_BYTES + off),
                       "r"(pp[4 * q]), "r"(pp[4 * q + 1]), "r"(pp[4 * q + 2]), "r"(pp[4 * q + 3])
                       : "memory");
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(BB_XY_EMPTY0 + s));
        mbar_arrive(bar(BB_DS_FULL0 + s));
      }
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

// delta[b,h,s] = sum_d dO[b,s,h,d] * O[b,s,h,d];  lse2 = lse * log2(e).  One warp per (b, s, h) row.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  const float* __restrict__ lse, float* __restrict__ delta, float* __restrict__ lse2,
                                  long long o_bs, long long o_ss, long long o_hs, long long do_bs, long long do_ss,
                                  long long do_hs, int B, int S, int H, int Dv) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(B) * S * H) return;
  const int h = static_cast<int>(w % H);
  const int s = static_cast<int>((w / H) % S);
  const int b = static_cast<int>(w / (static_cast<long long>(H) * S));
  const __nv_bfloat16* orow = o + b * o_bs + s * o_ss + h * o_hs;
  const __nv_bfloat16* drow = dout + b * do_bs + s * do_ss + h * do_hs;
  float acc = 0.f;
  for (int c = lane * 8; c < Dv; c += 256) {
    const uint4 a = *reinterpret_cast<const uint4*>(orow + c);
    const uint4 g = *reinterpret_cast<const uint4*>(drow + c);
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack_bf16(av[i]), y = unpack_bf16(gv[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const long long idx = (static_cast<long long>(b) * H + h) * S + s;
    delta[idx] = acc;
    lse2[idx] = lse[idx] * 1.4426950408889634f;
  }
}

template <int D, int DV>
static int launch_bwd(const olb_attn_bwd_desc* d, cudaStream_t stream) {
  using LK = BwdCfg<D, DV, true>;
  using LQ = BwdCfg<D, DV, false>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<D, DV, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, LK::TOTAL) != cudaSuccess ||
        cudaFuncSetAttribute(attn_bwd_kernel<D, DV, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, LQ::TOTAL) != cudaSuccess)
      return -3;
    configured = true;
  }
  const long long n_rows = static_cast<long long>(d->B) * d->S * d->Hq;
  float* delta = d->delta;
  float* lse2 = d->delta + n_rows;
  attn_delta_kernel<<<static_cast<unsigned>((n_rows * 32 + 255) / 256), 256, 0, stream>>>(
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
