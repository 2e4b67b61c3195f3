// Causal flash attention for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
// Forward, one CTA per (batch, head, 128-row query tile):
//   warp 0    : TMA producer - Q once, then K tiles and V tiles through two 3- or 4-stage rings (4D tensor maps over
//               the strided [B, S, H, D] tensors, 128B swizzle)
//   warp 1    : one thread issues  S = Q K^T  (UMMA 128 x BKV x 16, K-major x K-major) into one of
//               two TMEM score buffers and  O += P V  (A = P read from TMEM, B = V MN-major)
//   warps 2-9 : softmax - two threads own query row r (half of the columns each): one tcgen05.ld pass of
//               the score row into registers, row maxima exchanged between the pair, online softmax
//               in base 2 with lazy rescaling (the running maximum only moves when it grows by
//               more than 2^8, so the TMEM accumulator is rarely rescaled), P written as packed
//               bf16 over the scores in TMEM, final normalisation and store of O and the
//               log-sum-exp.
// Head dims: D (q/k) in {64, 128, 192}, Dv in {64, 128}; D = 192 / Dv = 128 is DeepSeek-V3's MLA.
// The reference calls F.scaled_dot_product_attention (optimus/models/olmoe/modeling_olmoe.py:219-227)
// or materialises the S x S scores (optimus/models/deepseek_v3/modeling_deepseek_v3.py:359-369).
//
// Backward: two kernels so that every gradient has exactly one writer (deterministic, no atomics):
// dK/dV per key tile looping over query tiles, dQ per query tile looping over key tiles; both
// recompute P from the saved log-sum-exp.  See attention_bwd.cu.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>
#include <cstdlib>

#include "olb_api.h"
#include "ptx.cuh"

namespace olb {

int make_tmap_4d_bf16(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides_bytes[3],
                      const uint32_t box[4]);

constexpr int ATT_BQ = 128;
constexpr int ATT_THREADS = 320;  // TMA warp, MMA warp, 8 softmax warps

template <int D, int DV, int BKV>
struct AttnFwdSmem {
  static constexpr int Q_BYTES = ATT_BQ * D * 2;
  static constexpr int K_BYTES = BKV * D * 2;
  static constexpr int V_BYTES = BKV * DV * 2;
  // K tiles are released as soon as their Q K^T has run, V tiles only after P V: separate rings.  Their depth
  // has to cover the TMA latency at one tile pair per ~1000 cycles, so all of shared memory is used.
  static constexpr int KS = (D == 128) ? 3 : 4, VS = KS;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + KS * K_BYTES;
  static constexpr int OFF_PAIR = OFF_V + VS * V_BYTES;  // row statistics exchanged between warp pairs
  static constexpr int OFF_BAR = OFF_PAIR + 2 * 2 * ATT_BQ * 4;
  static constexpr int TOTAL = OFF_BAR + 256;  // no alignment slack: the kernel checks that the window is 1024-aligned
  static_assert(TOTAL <= 232448, "shared memory size");
};

struct AttnFwdParams {
  __nv_bfloat16* o;
  float* lse;
  long long o_bs, o_ss, o_hs;
  int B, S, Hq, Hkv;
  float scale_log2;  // softmax scale * log2(e)
  float scale;
  int* status;
};

// barrier slots
enum { AB_Q = 0, AB_K0 = 1, AB_KE0 = 5, AB_V0 = 9, AB_VE0 = 13, AB_S_FULL0 = 17, AB_P_FULL = 19, AB_O_DONE = 20, AB_PAIR0 = 21 };

template <int D, int DV, int BKV>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnFwdParams p) {
  using L = AttnFwdSmem<D, DV, BKV>;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t TM_S0 = 0, TM_S1 = BKV, TM_O = 2 * BKV;  // column offsets
  static_assert(2 * BKV + DV <= 512, "TMEM columns");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {  // swizzled tiles need a 1024-byte aligned window (uniform exit, nothing allocated yet)
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_ARG);
    return;
  }
  uint8_t* gen = smem_raw;
  auto bar = [&](int i) { return base + L::OFF_BAR + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::OFF_BAR + 8 * 26);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::OFF_BAR + 8 * 26 + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_q_tiles = p.S / ATT_BQ;
  const int qt = n_q_tiles - 1 - blockIdx.x;  // heavy tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * ATT_BQ;
  const int n_kv = (q0 + ATT_BQ + BKV - 1) / BKV;  // causal: key tiles up to the diagonal

  if (threadIdx.x == 0) {
    mbar_init(bar(AB_Q), 1);
    for (int s = 0; s < L::KS; ++s) {
      mbar_init(bar(AB_K0 + s), 1);
      mbar_init(bar(AB_KE0 + s), 1);
    }
    for (int s = 0; s < L::VS; ++s) {
      mbar_init(bar(AB_V0 + s), 1);
      mbar_init(bar(AB_VE0 + s), 1);
    }
    for (int s = 0; s < 2; ++s) mbar_init(bar(AB_S_FULL0 + s), 1);
    mbar_init(bar(AB_P_FULL), 8);
    mbar_init(bar(AB_O_DONE), 1);
    for (int g = 0; g < 4; ++g) mbar_init(bar(AB_PAIR0 + g), 2);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      mbar_expect_tx(bar(AB_Q), L::Q_BYTES);
#pragma unroll
      for (int a = 0; a < D / 64; ++a) tma_load_4d(base + L::OFF_Q + a * (ATT_BQ * 128), &tm_q, bar(AB_Q), a * 64, h, q0, b);
      // K runs two tiles ahead of V
      for (int i = 0; i < n_kv + 2; ++i) {
        if (i < n_kv) {
          const int s = i % L::KS;
          if (i >= L::KS && !mbar_wait(bar(AB_KE0 + s), ((i / L::KS) - 1) & 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) break;
          mbar_expect_tx(bar(AB_K0 + s), L::K_BYTES);
#pragma unroll
          for (int a = 0; a < D / 64; ++a)
            tma_load_4d(base + L::OFF_K + s * L::K_BYTES + a * (BKV * 128), &tm_k, bar(AB_K0 + s), a * 64, hk, i * BKV, b);
        }
        const int j = i - 2;
        if (j >= 0) {
          const int s = j % L::VS;
          if (j >= L::VS && !mbar_wait(bar(AB_VE0 + s), ((j / L::VS) - 1) & 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) break;
          mbar_expect_tx(bar(AB_V0 + s), L::V_BYTES);
#pragma unroll
          for (int a = 0; a < DV / 64; ++a)
            tma_load_4d(base + L::OFF_V + s * L::V_BYTES + a * (BKV * 128), &tm_v, bar(AB_V0 + s), a * 64, hk, j * BKV, b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc_bf16(ATT_BQ, BKV, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(ATT_BQ, DV, 0, 1);
      bool ok = mbar_wait(bar(AB_Q), 0, p.status, ST_TIMEOUT_FULL, abort_flag);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        const uint32_t kbase = base + L::OFF_K + (j % L::KS) * L::K_BYTES;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t da = make_smem_desc(base + L::OFF_Q + (k / 4) * (ATT_BQ * 128) + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(kbase + (k / 4) * (BKV * 128) + (k % 4) * 32, 16, 1024);
          umma_ss(tmem + (s ? TM_S1 : TM_S0), da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(bar(AB_S_FULL0 + s));
        umma_commit(bar(AB_KE0 + j % L::KS));
      };
      if (ok && n_kv > 0) {
        ok = mbar_wait(bar(AB_K0), 0, p.status, ST_TIMEOUT_FULL, abort_flag);
        tc_fence_after();
        if (ok) issue_s(0);
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const int s = j & 1;
        if (j + 1 < n_kv) {
          const int s1 = (j + 1) % L::KS;
          const uint32_t ph1 = ((j + 1) / L::KS) & 1u;
          // score buffer s1 held P of tile j-1, whose P V was issued before this MMA: tcgen05.mma of one
          // thread execute in issue order, so no barrier is needed before overwriting it
          if (!mbar_wait(bar(AB_K0 + s1), ph1, p.status, ST_TIMEOUT_FULL, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(bar(AB_P_FULL), j & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) break;
        const int sv = j % L::VS;
        if (!mbar_wait(bar(AB_V0 + sv), (j / L::VS) & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) break;
        tc_fence_after();
        const uint32_t vbase = base + L::OFF_V + sv * L::V_BYTES;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          // A = P read from TMEM: bf16 pairs packed in the first BKV/2 columns of the score buffer,
          // 8 columns per K = 16 step
          const uint64_t db = make_smem_desc(vbase + k * 2048, BKV * 128, 1024);
          umma_ts(tmem + TM_O, tmem + (s ? TM_S1 : TM_S0) + k * 8, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(bar(AB_VE0 + sv));
        umma_commit(bar(AB_O_DONE));
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue
    // Eight warps: warps w and w+4 share the 32 query rows (TMEM lanes) of lane group w % 4 and split the
    // columns of the score tile.  Each reads its half row from TMEM once, keeps it in registers, and the two
    // exchange their row maxima through shared memory so that both use the same running maximum.
    constexpr int CW = BKV / 2;        // score columns per thread
    constexpr int OW = DV / 2;         // output columns per thread
    const int lg = warp & 3;
    const int ch = (warp - 2) >> 2;    // column half
    const int row = lg * 32 + lane;    // query row inside the tile == TMEM lane
    const int qi = q0 + row;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(lg * 32) << 16);
    float* pair = reinterpret_cast<float*>(gen + L::OFF_PAIR);  // [2 buffers][2 halves][128 rows]
    float m_used = -FLT_MAX, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int s = j & 1;
      if (!mbar_wait(bar(AB_S_FULL0 + s), (j >> 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t s_addr = lane_addr + (s ? TM_S1 : TM_S0) + ch * CW;
      const int kv0 = j * BKV + ch * CW;
      const bool diag = kv0 + CW > q0;  // this half tile touches the causal boundary
      uint32_t xr[CW / 32][32];
#pragma unroll
      for (int c = 0; c < CW / 32; ++c) tmem_ld_32x32b_x32(s_addr + c * 32, xr[c]);
      tmem_ld_wait();
      float x[CW];
#pragma unroll
      for (int i = 0; i < CW; ++i) x[i] = __uint_as_float(xr[i / 32][i % 32]);
      if (diag) {
#pragma unroll
        for (int i = 0; i < CW; ++i)
          if (kv0 + i > qi) x[i] = -FLT_MAX;
      }
      float mx4[4] = {-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX};  // four independent chains
#pragma unroll
      for (int i = 0; i < CW; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], x[i]);
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float* pb = pair + (j & 1) * 256;
      pb[ch * 128 + row] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(AB_PAIR0 + lg));
      // probabilities as packed bf16 pairs and their sum, for a given (scaled) running maximum
      uint32_t packed[CW / 2];
      auto probabilities = [&](float m_scaled) {
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int e = 0; e < CW / 2; ++e) {
          const float a = ex2_approx(x[2 * e] * p.scale_log2 - m_scaled);  // masked entries give 0
          const float bb = ex2_approx(x[2 * e + 1] * p.scale_log2 - m_scaled);
          s4[e & 3] += a + bb;
          packed[e] = pack_bf16(a, bb);
        }
        return (s4[0] + s4[1]) + (s4[2] + s4[3]);
      };
      if (!mbar_wait(bar(AB_PAIR0 + lg), j & 1u, p.status, ST_TIMEOUT_PEER, abort_flag)) {
        ok = false;
        break;
      }
      mx = fmaxf(mx, pb[(ch ^ 1) * 128 + row]);
      // rescale decision (identical in both warps of a pair: same rows, same maxima)
      const bool grow = (j == 0) || ((mx - m_used) * p.scale_log2 > 8.f);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      if (any_grow) {
        const float m_new = grow ? fmaxf(m_used, mx) : m_used;
        const float alpha = (j == 0) ? 0.f : ex2_approx((m_used - m_new) * p.scale_log2);
        if (j > 0) {
          // the previous P V must be complete before O is rescaled
          if (!mbar_wait(bar(AB_O_DONE), (j - 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < OW / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(lane_addr + TM_O + ch * OW + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x32(lane_addr + TM_O + ch * OW + c * 32, r);
          }
          tmem_st_wait();
        }
        l_sum *= alpha;
        m_used = m_new;
      }
      l_sum += probabilities(m_used * p.scale_log2);
      // P goes back into the score buffer (first BKV/2 columns), from where the P V MMA reads it as its A
      // operand.  Both halves of the scores are in registers by now (the pair barrier came after the loads).
      const uint32_t p_addr = lane_addr + (s ? TM_S1 : TM_S0) + ch * (CW / 2);
#pragma unroll
      for (int c16 = 0; c16 < CW / 32; ++c16) {
        uint32_t part[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) part[e] = packed[c16 * 16 + e];
        tmem_st_32x32b_x16(p_addr + c16 * 16, part);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(AB_P_FULL));
    }
    // epilogue: O / l and the log-sum-exp; each warp of a pair stores half of the output columns
    if (ok && n_kv > 0 && mbar_wait(bar(AB_O_DONE), (n_kv - 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) {
      tc_fence_after();
      float* pb = pair + (n_kv & 1) * 256;
      pb[ch * 128 + row] = l_sum;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(AB_PAIR0 + lg));
      const bool paired = mbar_wait(bar(AB_PAIR0 + lg), n_kv & 1u, p.status, ST_TIMEOUT_PEER, abort_flag);
      l_sum += paired ? pb[(ch ^ 1) * 128 + row] : 0.f;
      const float inv = 1.f / l_sum;
      __nv_bfloat16* orow = p.o + static_cast<long long>(b) * p.o_bs + static_cast<long long>(qi) * p.o_ss +
                            static_cast<long long>(h) * p.o_hs + ch * OW;
#pragma unroll 1
      for (int c = 0; c < OW / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_addr + TM_O + ch * OW + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(r[8 * g]) * inv, __uint_as_float(r[8 * g + 1]) * inv);
          v.y = pack_bf16(__uint_as_float(r[8 * g + 2]) * inv, __uint_as_float(r[8 * g + 3]) * inv);
          v.z = pack_bf16(__uint_as_float(r[8 * g + 4]) * inv, __uint_as_float(r[8 * g + 5]) * inv);
          v.w = pack_bf16(__uint_as_float(r[8 * g + 6]) * inv, __uint_as_float(r[8 * g + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = v;
        }
      }
      if (ch == 0) p.lse[(static_cast<long long>(b) * p.Hq + h) * p.S + qi] = m_used * p.scale + __logf(l_sum);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Forward with two query tiles per CTA.  The single-tile kernel above is bound by the latency of its softmax
// chain (score ready -> TMEM read -> row maximum -> pair exchange -> exp -> P write): two warps per scheduler
// cannot hide it, and the tensor pipe idles while it runs.  Here a CTA owns 256 query rows as two 128-row tiles
// a and b, each with its own score buffer and output accumulator in TMEM (2 * BKV + 2 * DV columns) and its own
// group of four softmax warps (one thread per query row).  The issuing thread alternates  P_a V, S_a = Q_a K^T(next), P_b V, S_b(next),
// so that one group's softmax runs underneath the other group's matrix products, and every K / V tile that
// TMA brings in is used by both query tiles.  K and V tiles share one ring in consumption order K0 V0 K1 V1 ...
// Tile a ends one diagonal block (128 keys) before tile b.
constexpr int ATT2_THREADS = 64 + 2 * 128;  // TMA warp, MMA warp, 2 x 4 softmax warps

template <int D, int DV, int BKV>
struct AttnFwd2Smem {
  static constexpr int QT_BYTES = ATT_BQ * D * 2;  // one query tile
  static constexpr int K_BYTES = BKV * D * 2;
  static constexpr int V_BYTES = BKV * DV * 2;
  static constexpr int STAGE = K_BYTES > V_BYTES ? K_BYTES : V_BYTES;
  static constexpr int NS = (2 * QT_BYTES + 5 * STAGE + 256 <= 232448) ? 5 : 4;  // as deep as shared memory allows
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_RING = OFF_Q + 2 * QT_BYTES;
  static constexpr int OFF_BAR = OFF_RING + NS * STAGE;
  static constexpr int TOTAL = OFF_BAR + 256;
  static_assert(STAGE % 1024 == 0 && QT_BYTES % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
  static_assert(TOTAL <= 232448, "shared memory size");
};

// barrier slots of the two-tile kernel
enum { A2_Q = 0, A2_FULL0 = 1, A2_EMPTY0 = 7, A2_S_FULL0 = 13, A2_P_FULL0 = 15, A2_O_DONE0 = 17 };  // up to 6 stages

template <int D, int DV, int BKV, int EMU>
__global__ void __launch_bounds__(ATT2_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttnFwdParams p) {
  using L = AttnFwd2Smem<D, DV, BKV>;
  constexpr int NS = L::NS;
  constexpr uint32_t TMEM_COLS = 512;
  static_assert(2 * BKV + 2 * DV <= 512, "TMEM columns");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {  // uniform exit before anything is allocated
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_ARG);
    return;
  }
  uint8_t* gen = smem_raw;
  auto bar = [&](int i) { return base + L::OFF_BAR + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::OFF_BAR + 8 * 26);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::OFF_BAR + 8 * 26 + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_q2 = p.S / (2 * ATT_BQ);
  const int qt2 = n_q2 - 1 - blockIdx.x;  // heavy tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt2 * 2 * ATT_BQ;
  const int n_a = (q0 + ATT_BQ + BKV - 1) / BKV;      // key tiles of query tile a
  const int n_b = (q0 + 2 * ATT_BQ + BKV - 1) / BKV;  // ... of query tile b (all that the CTA loads)

  if (threadIdx.x == 0) {
    mbar_init(bar(A2_Q), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(A2_FULL0 + s), 1);
      mbar_init(bar(A2_EMPTY0 + s), 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(bar(A2_S_FULL0 + g), 1);
      mbar_init(bar(A2_P_FULL0 + g), 4);
      mbar_init(bar(A2_O_DONE0 + g), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      mbar_expect_tx(bar(A2_Q), 2 * L::QT_BYTES);
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int a = 0; a < D / 64; ++a)
          tma_load_4d(base + L::OFF_Q + g * L::QT_BYTES + a * (ATT_BQ * 128), &tm_q, bar(A2_Q), a * 64, h, q0 + g * ATT_BQ, b);
      for (int t = 0; t < 2 * n_b; ++t) {
        const int s = t % NS, j = t >> 1;
        if (t >= NS && !mbar_wait(bar(A2_EMPTY0 + s), ((t / NS) - 1) & 1u, p.status, ST_TIMEOUT_EMPTY, abort_flag)) break;
        const uint32_t dst = base + L::OFF_RING + s * L::STAGE;
        if ((t & 1) == 0) {
          mbar_expect_tx(bar(A2_FULL0 + s), L::K_BYTES);
#pragma unroll
          for (int a = 0; a < D / 64; ++a) tma_load_4d(dst + a * (BKV * 128), &tm_k, bar(A2_FULL0 + s), a * 64, hk, j * BKV, b);
        } else {
          mbar_expect_tx(bar(A2_FULL0 + s), L::V_BYTES);
#pragma unroll
          for (int a = 0; a < DV / 64; ++a) tma_load_4d(dst + a * (BKV * 128), &tm_v, bar(A2_FULL0 + s), a * 64, hk, j * BKV, b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc_bf16(ATT_BQ, BKV, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(ATT_BQ, DV, 0, 1);
      bool ok = mbar_wait(bar(A2_Q), 0, p.status, ST_TIMEOUT_FULL, abort_flag);
      auto wait_item = [&](int t) {
        const bool got = mbar_wait(bar(A2_FULL0 + t % NS), (t / NS) & 1u, p.status, ST_TIMEOUT_FULL, abort_flag);
        tc_fence_after();
        return got;
      };
      auto issue_s = [&](int g, int j) {  // S_g = Q_g K_j^T
        const uint32_t kbase = base + L::OFF_RING + ((2 * j) % NS) * L::STAGE;
        const uint32_t qbase = base + L::OFF_Q + g * L::QT_BYTES;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t da = make_smem_desc(qbase + (k / 4) * (ATT_BQ * 128) + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(kbase + (k / 4) * (BKV * 128) + (k % 4) * 32, 16, 1024);
          umma_ss(tmem + g * BKV, da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(bar(A2_S_FULL0 + g));
      };
      auto issue_pv = [&](int g, int j) {  // O_g += P_g V_j, P read from TMEM (packed bf16 over the scores)
        const uint32_t vbase = base + L::OFF_RING + ((2 * j + 1) % NS) * L::STAGE;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint64_t db = make_smem_desc(vbase + k * 2048, BKV * 128, 1024);
          umma_ts(tmem + 2 * BKV + g * DV, tmem + g * BKV + k * 8, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(bar(A2_O_DONE0 + g));
      };
      if (ok) ok = wait_item(0);
      if (ok) {
        issue_s(0, 0);
        issue_s(1, 0);
        umma_commit(bar(A2_EMPTY0 + 0));
      }
      for (int j = 0; ok && j < n_b; ++j) {
        // The K / V tiles an iteration needs are waited for before the probabilities, while this thread would idle
        // anyway; their loads depend on nothing that is still to come.
        if (!wait_item(2 * j + 1)) break;
        if (j + 1 < n_b && !wait_item(2 * j + 2)) break;
        if (j < n_a) {
          if (!mbar_wait(bar(A2_P_FULL0 + 0), j & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) break;
          tc_fence_after();
          issue_pv(0, j);
          // S_a of the next key tile overwrites P_a(j): its P V was issued just above, and the tcgen05.mma of
          // one thread execute in issue order
          if (j + 1 < n_a) issue_s(0, j + 1);
        }
        if (!mbar_wait(bar(A2_P_FULL0 + 1), j & 1u, p.status, ST_TIMEOUT_FULL, abort_flag)) break;
        tc_fence_after();
        issue_pv(1, j);
        umma_commit(bar(A2_EMPTY0 + (2 * j + 1) % NS));
        if (j + 1 < n_b) {
          issue_s(1, j + 1);
          umma_commit(bar(A2_EMPTY0 + (2 * j + 2) % NS));
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue, one group per query tile
    // Four warps per group, one thread per query row (TMEM lane): the whole score row sits in registers, so the
    // row maximum needs no exchange between threads and the exponentials of a row are one long independent
    // stream for the special-function unit.
    constexpr int CW = BKV;                  // score columns per thread
    const int g = (warp - 2) >> 2;           // query tile / softmax group
    const int lg = warp & 3;
    const int row = lg * 32 + lane;
    const int qg0 = q0 + g * ATT_BQ;
    const int qi = qg0 + row;
    const int n_kv = g ? n_b : n_a;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(lg * 32) << 16);
    const uint32_t tm_s = g * BKV, tm_o = 2 * BKV + g * DV;
    float m_used = -FLT_MAX, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      if (!mbar_wait(bar(A2_S_FULL0 + g), j & 1u, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int kv0 = j * BKV;
      const bool diag = kv0 + CW > qg0;  // this tile touches the causal boundary
      uint32_t xr[CW / 32][32];
#pragma unroll
      for (int c = 0; c < CW / 32; ++c) tmem_ld_32x32b_x32(lane_addr + tm_s + c * 32, xr[c]);
      tmem_ld_wait();
      float x[CW];
#pragma unroll
      for (int i = 0; i < CW; ++i) x[i] = __uint_as_float(xr[i / 32][i % 32]);
      if (diag) {
#pragma unroll
        for (int i = 0; i < CW; ++i)
          if (kv0 + i > qi) x[i] = -FLT_MAX;
      }
      float mx4[4];  // four chains of three-input maxima
#pragma unroll
      for (int c = 0; c < 4; ++c) mx4[c] = fmaxf(x[2 * c], x[2 * c + 1]);
#pragma unroll
      for (int i = 8; i < CW; i += 8) {
#pragma unroll
        for (int c = 0; c < 4; ++c) mx4[c] = max3(mx4[c], x[i + 2 * c], x[i + 2 * c + 1]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // lazy rescaling: the running maximum only moves when it grows by more than 2^8
      const bool grow = (j == 0) || ((mx - m_used) * p.scale_log2 > 8.f);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? fmaxf(m_used, mx) : m_used;
        const float alpha = (j == 0) ? 0.f : ex2_approx((m_used - m_new) * p.scale_log2);
        if (j > 0) {
          // the previous P V must be complete before O is rescaled
          if (!mbar_wait(bar(A2_O_DONE0 + g), (j - 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < DV / 16; ++c) {  // 16-column pieces: the score row is live in registers here
            uint32_t r[16];
            tmem_ld_32x32b_x16(lane_addr + tm_o + c * 16, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x16(lane_addr + tm_o + c * 16, r);
          }
          tmem_st_wait();
        }
        l_sum *= alpha;
        m_used = m_new;
      }
      // P = 2^(s * c - m) as packed bf16 pairs over the first BKV/2 columns of the score buffer (this thread's own
      // lane), written in 16-column pieces as they are produced; the P V product reads it from there as its A operand
      const float m_scaled = m_used * p.scale_log2;
      float2 s2[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m_scaled, -m_scaled);
#pragma unroll
      for (int c16 = 0; c16 < CW / 32; ++c16) {
        uint32_t part[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float2 t2 = fma2(make_float2(x[c16 * 32 + 2 * e], x[c16 * 32 + 2 * e + 1]), sc2, nm2);
          float2 pr;
          if ((e & 7) < EMU) {
            pr = ex2_poly2(t2);  // this share of the exponentials runs on the FMA pipe
          } else {
            pr.x = ex2_approx(t2.x);  // masked entries give 0
            pr.y = ex2_approx(t2.y);
          }
          s2[e & 3] = add2(s2[e & 3], pr);
          part[e] = pack_bf16(pr.x, pr.y);
        }
        tmem_st_32x32b_x16(lane_addr + tm_s + c16 * 16, part);
      }
      {
        const float2 sa = add2(s2[0], s2[1]), sb = add2(s2[2], s2[3]);
        l_sum += (sa.x + sa.y) + (sb.x + sb.y);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(A2_P_FULL0 + g));
    }
    // epilogue: O / l and the log-sum-exp
    if (ok && n_kv > 0 && mbar_wait(bar(A2_O_DONE0 + g), (n_kv - 1) & 1u, p.status, ST_TIMEOUT_ACC_FULL, abort_flag)) {
      tc_fence_after();
      const float inv = 1.f / l_sum;
      __nv_bfloat16* orow = p.o + static_cast<long long>(b) * p.o_bs + static_cast<long long>(qi) * p.o_ss +
                            static_cast<long long>(h) * p.o_hs;
#pragma unroll 1
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_addr + tm_o + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(r[8 * q4]) * inv, __uint_as_float(r[8 * q4 + 1]) * inv);
          v.y = pack_bf16(__uint_as_float(r[8 * q4 + 2]) * inv, __uint_as_float(r[8 * q4 + 3]) * inv);
          v.z = pack_bf16(__uint_as_float(r[8 * q4 + 4]) * inv, __uint_as_float(r[8 * q4 + 5]) * inv);
          v.w = pack_bf16(__uint_as_float(r[8 * q4 + 6]) * inv, __uint_as_float(r[8 * q4 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = v;
        }
      }
      p.lse[(static_cast<long long>(b) * p.Hq + h) * p.S + qi] = m_used * p.scale + __logf(l_sum);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// [B, S, H, Dh] view -> 4D tensor map with box {64, 1, rows, 1}
int attn_tmap(CUtensorMap* map, const void* ptr, int Dh, int H, int S, int B, long long bs, long long ss, long long hs,
              int box_rows) {
  const uint64_t dims[4] = {static_cast<uint64_t>(Dh), static_cast<uint64_t>(H), static_cast<uint64_t>(S),
                            static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(hs) * 2, static_cast<uint64_t>(ss) * 2, static_cast<uint64_t>(bs) * 2};
  const uint32_t box[4] = {64, 1, static_cast<uint32_t>(box_rows), 1};
  return make_tmap_4d_bf16(map, ptr, dims, strides, box);
}

template <int D, int DV, int BKV>
static int launch_fwd(const olb_attn_fwd_desc* d, cudaStream_t stream) {
  using L = AttnFwdSmem<D, DV, BKV>;
  // the attribute belongs to the function on one device: once per device, not once per process
  static bool configured_on[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  bool& configured = configured_on[dev];
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<D, DV, BKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return -3;
    configured = true;
  }
  CUtensorMap tq, tk, tv;
  if (attn_tmap(&tq, d->q, D, d->Hq, d->S, d->B, d->q_bs, d->q_ss, d->q_hs, ATT_BQ)) return -4;
  if (attn_tmap(&tk, d->k, D, d->Hkv, d->S, d->B, d->k_bs, d->k_ss, d->k_hs, BKV)) return -4;
  if (attn_tmap(&tv, d->v, DV, d->Hkv, d->S, d->B, d->v_bs, d->v_ss, d->v_hs, BKV)) return -4;
  AttnFwdParams p;
  p.o = static_cast<__nv_bfloat16*>(d->o);
  p.lse = d->lse;
  p.o_bs = d->o_bs;
  p.o_ss = d->o_ss;
  p.o_hs = d->o_hs;
  p.B = d->B;
  p.S = d->S;
  p.Hq = d->Hq;
  p.Hkv = d->Hkv;
  p.scale = d->scale;
  p.scale_log2 = d->scale * 1.4426950408889634f;
  p.status = d->status;
  dim3 grid(d->S / ATT_BQ, d->Hq, d->B);
  attn_fwd_kernel<D, DV, BKV><<<grid, ATT_THREADS, L::TOTAL, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

template <int D, int DV, int BKV, int EMU>
static int launch_fwd2(const olb_attn_fwd_desc* d, cudaStream_t stream) {
  using L = AttnFwd2Smem<D, DV, BKV>;
  // the attribute belongs to the function on one device: once per device, not once per process
  static bool configured_on[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  bool& configured = configured_on[dev];
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd2_kernel<D, DV, BKV, EMU>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return -3;
    configured = true;
  }
  CUtensorMap tq, tk, tv;
  if (attn_tmap(&tq, d->q, D, d->Hq, d->S, d->B, d->q_bs, d->q_ss, d->q_hs, ATT_BQ)) return -4;
  if (attn_tmap(&tk, d->k, D, d->Hkv, d->S, d->B, d->k_bs, d->k_ss, d->k_hs, BKV)) return -4;
  if (attn_tmap(&tv, d->v, DV, d->Hkv, d->S, d->B, d->v_bs, d->v_ss, d->v_hs, BKV)) return -4;
  AttnFwdParams p;
  p.o = static_cast<__nv_bfloat16*>(d->o);
  p.lse = d->lse;
  p.o_bs = d->o_bs;
  p.o_ss = d->o_ss;
  p.o_hs = d->o_hs;
  p.B = d->B;
  p.S = d->S;
  p.Hq = d->Hq;
  p.Hkv = d->Hkv;
  p.scale = d->scale;
  p.scale_log2 = d->scale * 1.4426950408889634f;
  p.status = d->status;
  dim3 grid(d->S / (2 * ATT_BQ), d->Hq, d->B);
  attn_fwd2_kernel<D, DV, BKV, EMU><<<grid, ATT2_THREADS, L::TOTAL, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Two query tiles per CTA wherever the sequence is a multiple of 256 rows; OLB_ATTN_FWD2=0 keeps the
// single-tile kernel (A/B measurements).
static bool fwd2_enabled() {
  static const bool on = [] {
    const char* e = getenv("OLB_ATTN_FWD2");
    return !(e && e[0] == '0');
  }();
  return on;
}

}  // namespace olb

extern "C" int olb_attn_fwd(const olb_attn_fwd_desc* d, cudaStream_t stream) {
  using namespace olb;
  if (d->S % ATT_BQ || d->Hq % d->Hkv) return -1;
  auto bad = [](long long s) { return (s % 8) != 0; };
  if (bad(d->q_bs) || bad(d->q_ss) || bad(d->q_hs) || bad(d->k_bs) || bad(d->k_ss) || bad(d->k_hs) || bad(d->v_bs) ||
      bad(d->v_ss) || bad(d->v_hs) || bad(d->o_bs) || bad(d->o_ss) || bad(d->o_hs))
    return -2;
  if ((reinterpret_cast<uintptr_t>(d->q) | reinterpret_cast<uintptr_t>(d->k) | reinterpret_cast<uintptr_t>(d->v) |
       reinterpret_cast<uintptr_t>(d->o)) & 15)
    return -2;
  if (d->variant == 2 && d->S % (2 * ATT_BQ)) return -7;
  if (d->S % (2 * ATT_BQ) == 0 && (d->variant == 2 || (d->variant == 0 && fwd2_enabled()))) {
    // a quarter of the exponentials on the FMA pipe measured fastest for 128 x 128 tiles (0.303 ms against 0.308 with
    // none and 0.318 / 0.333 with three / four eighths, B4 S4096 H16)
    if (d->D == 128 && d->Dv == 128) return launch_fwd2<128, 128, 128, 2>(d, stream);
    if (d->D == 64 && d->Dv == 64) return launch_fwd2<64, 64, 128, 0>(d, stream);
    if (d->D == 192 && d->Dv == 128) return launch_fwd2<192, 128, 64, 0>(d, stream);
  }
  if (d->D == 128 && d->Dv == 128) return launch_fwd<128, 128, 128>(d, stream);
  if (d->D == 64 && d->Dv == 64) return launch_fwd<64, 64, 128>(d, stream);
  if (d->D == 192 && d->Dv == 128) return launch_fwd<192, 128, 64>(d, stream);
  return -6;
}
