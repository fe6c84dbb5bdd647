// Fused causal prefill attention on int8 operands, one kernel instead of
//   bmm_s8t_s8n_f32t (scores) -> mask + softmax + x127 + round -> bmm_s8t_s8n_s8t (context)
// (torch_int/models/opt.py:131-181), with the same arithmetic per element:
//   s_tj  = alpha_qk * float(q_t . k_j)                       int8 dot products, int32 accumulators
//   p_tj  = int8(rne(127 * exp(s_tj - max_j s_tj) / sum_j exp(s_tj - max_j s_tj)))   for j <= t + past
//   ctx_t = int8(sat_rne(alpha_pv * float(sum_j p_tj * v_j)))
// The probabilities are quantised from the softmax of the FULL row, so the row maximum and the row
// sum must be known before the first p is formed: the kernel makes two passes over the key tiles.
//   pass 1: S = Q.K_j^T on the tensor cores (tcgen05.mma kind::i8, accumulator in TMEM) -> running
//           row maximum m and row sum l (rescaled when the maximum grows);
//   pass 2: S again -> p -> the int8 P tile is written to shared memory in the 128-byte-swizzled
//           K-major layout and multiplied with the V^T tile: O += P.V_j (second TMEM accumulator).
// Neither the fp32 scores (4 S^2 bytes per head, written and read) nor the int8 probabilities
// (S^2, written and read) touch HBM; the price is computing Q.K^T twice, which the tensor cores
// have room for (the kernel is bound by the exponentials).
//
// One CTA per (sequence, head, 128 query rows); 320 threads: warp 0 = TMA producer, warp 1 = MMA
// issuer, warps 2-9 = softmax / epilogue.  Two threads share a query row (TMEM lane = row): one owns
// keys [0, 64) of every tile, the other keys [64, 128); each keeps a running maximum and sum of its
// keys, the two are combined once after pass 1.  A thread copies its 64 accumulators into registers
// and releases S immediately, so the next Q.K^T runs while the exponentials of this tile are evaluated.
// The accumulators become fp32 scores in place, with the causal mask folded in as -FLT_MAX on the diagonal
// tile only; all later loops are the same code for every tile (small enough for the instruction cache).  TMEM: 128 columns S + up to 128
// columns O = 256 of 512, shared memory 99 KB: two CTAs per SM.  Only keys j <= t + past are visited
// (causal); an explicit additive mask is not supported - callers with padding masks use the
// three-kernel path.  Every wait is bounded (2 s) and reports through the status word.
//
// Rounding: every probability is rne(127 * expf(s - m) / l) with IEEE-exact division (a multiply by
// RN(1/l) plus two residual corrections); the row sum l is accumulated per thread with ex2.approx and
// in tile order, so it can differ from a sequential expf sum in its last bits, which moves a
// probability by one unit only where 127 * e / l sits on a rounding tie.
#include <cuda.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#define TI_PTX_EXTERNAL_STATUS 1
#include "attention_prefill.h"
#include "gemm_i8.h"
#include "sm100_ptx.cuh"

namespace ti {
namespace {

constexpr int TILE_ROWS = 128;             // query rows per CTA, keys per tile
constexpr int TILE_BYTES = 128 * 128;      // one 128-row x 128-byte swizzled operand tile
constexpr int NSLOT = 4;                   // ring of K / V^T tiles
constexpr int SOFTMAX_WARPS = 8;           // two threads per query row: each owns 64 of a tile's 128 keys
constexpr int SOFTMAX_THREADS = SOFTMAX_WARPS * 32;
constexpr int ATT_THREADS = 64 + SOFTMAX_THREADS;
constexpr int TMEM_COLS = 256;
constexpr int STATS_BYTES = 2 * 2 * TILE_ROWS * 4;  // (m, l) of both column halves of every row
constexpr int SMEM_BYTES = 1024 + (2 + NSLOT) * TILE_BYTES + STATS_BYTES + 256;

enum : int {
  TI_ERR_ATT_RING_EMPTY = 121,  // producer waited for a free ring slot
  TI_ERR_ATT_RING_FULL = 122,   // MMA warp waited for a K / V tile
  TI_ERR_ATT_Q = 123,           // MMA warp waited for the Q tile
  TI_ERR_ATT_S_EMPTY = 124,     // MMA warp waited for the softmax warps to drain S
  TI_ERR_ATT_S_FULL = 125,      // softmax warps waited for S
  TI_ERR_ATT_P_FULL = 126,      // MMA warp waited for the P tile
  TI_ERR_ATT_P_EMPTY = 127,     // softmax warps waited for the P tile to be consumed
  TI_ERR_ATT_O_FULL = 128,      // epilogue waited for the context accumulator
};

struct AttnParams {
  int T;       // query rows per sequence
  int S;       // keys per sequence = past + T
  int past;    // row t sees keys j <= t + past
  float alpha_qk, alpha_pv;
  int8_t* ctx;             // [B, T, *]: row stride ld_ctx, head h at column h * D
  long long ld_ctx;
  long long ctx_batch_stride;
  int* status;
};

// Generic-proxy writes to shared memory (the P tile) -> visible to the async proxy (UMMA reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 2^x to about 2 ulp; used for the row sum only (every probability is formed with expf).
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Four values, each already rounded to an integer, clamped to [-128, 127] and packed into bytes.
__device__ __forceinline__ uint32_t pack_sat_s8x4(int a, int b, int c, int d) {
  uint32_t lo, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(lo) : "r"(d), "r"(c));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(lo));
  return out;
}

// e / l rounded to nearest, given r = RN(1 / l): a product and two residual corrections (Markstein's
// scheme) reproduce IEEE division for the operands that occur here (0 <= e <= 1 <= l, both normal
// or e so small that the probability is 0 either way) without a reciprocal per element.
__device__ __forceinline__ float div_by_row_sum(float e, float l, float r) {
  float q = __fmul_rn(e, r);
  float rem = __fmaf_rn(-q, l, e);
  q = __fmaf_rn(rem, r, q);
  rem = __fmaf_rn(-q, l, e);
  return __fmaf_rn(rem, r, q);
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attention_prefill_s8_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  static_assert(D == 64 || D == 128, "head_dim 64 or 128");
  constexpr uint32_t V_BYTES = D * 128;  // V^T tile: D rows x 128 keys
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                     // [128 rows][128 B]  (D = 64: upper half of each row zero)
  uint8_t* sP = smem + TILE_BYTES;        // [128 rows][128 keys]
  uint8_t* ring = smem + 2 * TILE_BYTES;  // NSLOT tiles
  float* stats = reinterpret_cast<float*>(ring + NSLOT * TILE_BYTES);  // [half][m | l][row]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(stats) + STATS_BYTES);
  uint64_t* full_bar = bars;              // [NSLOT]
  uint64_t* empty_bar = bars + NSLOT;     // [NSLOT]
  uint64_t* q_full = bars + 2 * NSLOT;
  uint64_t* s_full = q_full + 1;
  uint64_t* s_empty = q_full + 2;
  uint64_t* p_full = q_full + 3;
  uint64_t* p_empty = q_full + 4;
  uint64_t* o_full = q_full + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heavy query tiles (those that see most keys) first
  const int qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int t0 = qt * TILE_ROWS;
  const int kv_end = min(p.S, min(t0 + TILE_ROWS, p.T) + p.past);  // keys [0, kv_end) are visible to some row
  const int nt = (kv_end + TILE_ROWS - 1) / TILE_ROWS;             // >= 1

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSLOT; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(q_full), 1);
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(s_empty), SOFTMAX_THREADS);
    mbar_init(smem_u32(p_full), SOFTMAX_THREADS);
    mbar_init(smem_u32(p_empty), 1);
    mbar_init(smem_u32(o_full), 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;        // S: 128 columns
  const uint32_t tmem_o = tmem_base + 128;  // O: D columns

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // Tile order = the order in which the MMA warp consumes them:
    //   pass 1: K_0 .. K_{nt-1};   pass 2: K_0, then for every j: K_{j+1} (if any), V_j.
    if (lane == 0) {
      mbar_expect_tx(smem_u32(q_full), TILE_BYTES);
      tma_load_4d(smem_u32(sQ), &tmap_q, smem_u32(q_full), 0, t0, h, b);
      int slot = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto push = [&](const CUtensorMap* map, int c0, int c1, uint32_t bytes) {
        ok = mbar_wait_status(smem_u32(&empty_bar[slot]), phase ^ 1, abort_flag, p.status, TI_ERR_ATT_RING_EMPTY);
        if (!ok) return;
        const uint32_t fb = smem_u32(&full_bar[slot]);
        mbar_expect_tx(fb, bytes);
        tma_load_4d(smem_u32(ring + slot * TILE_BYTES), map, fb, c0, c1, h, b);
        if (++slot == NSLOT) {
          slot = 0;
          phase ^= 1;
        }
      };
      for (int j = 0; j < nt && ok; ++j) push(&tmap_k, 0, j * TILE_ROWS, TILE_BYTES);
      if (ok) push(&tmap_k, 0, 0, TILE_BYTES);
      for (int j = 0; j < nt && ok; ++j) {
        if (j + 1 < nt) push(&tmap_k, 0, (j + 1) * TILE_ROWS, TILE_BYTES);
        if (ok) push(&tmap_v, j * TILE_ROWS, 0, V_BYTES);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_s8s8s32(128, 128);
      constexpr uint32_t idesc_o = make_idesc_s8s8s32(128, D);
      int slot = 0;
      uint32_t phase = 0;
      uint32_t g = 0;  // S tiles issued so far (both passes)
      bool ok = mbar_wait_status(smem_u32(q_full), 0, abort_flag, p.status, TI_ERR_ATT_Q);
      const uint64_t dq = make_smem_desc_sw128(smem_u32(sQ));
      const uint64_t dp = make_smem_desc_sw128(smem_u32(sP));
      auto advance = [&]() {
        if (++slot == NSLOT) {
          slot = 0;
          phase ^= 1;
        }
      };
      // S = Q . K^T for the K tile in the next ring slot
      auto issue_s = [&]() {
        ok = mbar_wait_status(smem_u32(&full_bar[slot]), phase, abort_flag, p.status, TI_ERR_ATT_RING_FULL);
        if (!ok) return;
        // the softmax warps have copied the previous S into registers (the first wait passes at once)
        ok = mbar_wait_status(smem_u32(s_empty), (g & 1) ^ 1, abort_flag, p.status, TI_ERR_ATT_S_EMPTY);
        if (!ok) return;
        tc_fence_after();
        const uint64_t dk = make_smem_desc_sw128(smem_u32(ring + slot * TILE_BYTES));
#pragma unroll
        for (int k = 0; k < D / 32; ++k) umma_i8<1>(tmem_s, dq + 2 * k, dk + 2 * k, idesc_s, k != 0);
        umma_commit(smem_u32(&empty_bar[slot]));
        umma_commit(smem_u32(s_full));
        advance();
        ++g;
      };
      for (int j = 0; j < nt && ok; ++j) issue_s();  // pass 1
      if (ok) issue_s();                             // pass 2, tile 0
      for (int j = 0; j < nt && ok; ++j) {
        if (j + 1 < nt) issue_s();                   // S_{j+1}: the softmax of tile j+1 overlaps P_j . V_j
        if (!ok) break;
        ok = mbar_wait_status(smem_u32(&full_bar[slot]), phase, abort_flag, p.status, TI_ERR_ATT_RING_FULL);
        if (!ok) break;
        ok = mbar_wait_status(smem_u32(p_full), j & 1, abort_flag, p.status, TI_ERR_ATT_P_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dv = make_smem_desc_sw128(smem_u32(ring + slot * TILE_BYTES));
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_i8<1>(tmem_o, dp + 2 * k, dv + 2 * k, idesc_o, (j != 0) || (k != 0));
        umma_commit(smem_u32(&empty_bar[slot]));
        umma_commit(smem_u32(p_empty));
        advance();
      }
      if (ok) umma_commit(smem_u32(o_full));
    }
  } else {
    // --------------------------------------------------------- softmax and epilogue
    // Two threads per query row: warps 2-5 own keys [0, 64) of every tile, warps 6-9 keys [64, 128).
    // A thread copies its 64 accumulators into registers and releases S at once, so the tensor core
    // computes the next S while the exponentials of this one run.
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter + 32)
    const int half = (warp - 2) >> 2;        // which 64 keys of a tile
    const int r = quarter * 32 + lane;       // row of the tile = TMEM lane
    const int rg = t0 + r;                   // row of the sequence
    const bool valid = rg < p.T;
    const int lim = valid ? rg + p.past : -1;  // last visible key
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_s + lane_off + half * 64;
    const float alpha = p.alpha_qk;
    constexpr float kLog2e = 1.4426950408889634f;
    // the fp32 score exactly as the unfused path stores it: one rounded multiply (never contracted
    // into the following subtraction)
    auto score = [alpha](uint32_t acc) { return __fmul_rn(alpha, __int2float_rn(static_cast<int>(acc))); };
    float m = -FLT_MAX, l = 0.f;
    uint32_t g = 0;
    bool ok = true;
    uint32_t va[32], vb[32];
    auto fetch_s = [&]() {
      ok = mbar_wait_status(smem_u32(s_full), g & 1, abort_flag, p.status, TI_ERR_ATT_S_FULL);
      if (!ok) return;
      tc_fence_after();
      tmem_ld_32x32(s_addr, va);
      tmem_ld_32x32(s_addr + 32, vb);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(s_empty));
      ++g;
    };
    // Accumulators -> fp32 scores in place (the registers keep the float bits), with the causal mask
    // folded in as -FLT_MAX: everything after this step is the same code for tiles below and on the
    // diagonal, which keeps the unrolled loops small enough for the instruction cache.
    auto to_scores = [&](int c0, bool all_visible) {
      if (all_visible) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          va[i] = __float_as_uint(score(va[i]));
          vb[i] = __float_as_uint(score(vb[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          va[i] = __float_as_uint(c0 + i <= lim ? score(va[i]) : -FLT_MAX);
          vb[i] = __float_as_uint(c0 + 32 + i <= lim ? score(vb[i]) : -FLT_MAX);
        }
      }
    };
    // ---- pass 1: row maximum and row sum over this thread's keys
#pragma unroll 1
    for (int j = 0; j < nt && ok; ++j) {
      fetch_s();
      if (!ok) break;
      const int c0 = j * TILE_ROWS + half * 64;
      const bool all_visible = c0 + 63 <= t0 + p.past;  // for every valid row of the CTA (uniform)
      if (!all_visible && c0 > lim) continue;  // none of this thread's keys of this tile is visible to its row
      to_scores(c0, all_visible);
      float t0m = -FLT_MAX, t1m = -FLT_MAX;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        t0m = fmaxf(t0m, __uint_as_float(va[i]));
        t1m = fmaxf(t1m, __uint_as_float(vb[i]));
      }
      const float mn = fmaxf(m, fmaxf(t0m, t1m));
      l *= ex2_approx((m - mn) * kLog2e);
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int i = 0; i < 32; i += 2) {  // masked keys: 2^(-inf) = 0
        a0 += ex2_approx((__uint_as_float(va[i]) - mn) * kLog2e);
        a1 += ex2_approx((__uint_as_float(va[i + 1]) - mn) * kLog2e);
        a2 += ex2_approx((__uint_as_float(vb[i]) - mn) * kLog2e);
        a3 += ex2_approx((__uint_as_float(vb[i + 1]) - mn) * kLog2e);
      }
      l += (a0 + a1) + (a2 + a3);
      m = mn;
    }
    // ---- the row's maximum and sum over all keys: combine the two halves (in a fixed order, so that
    //      both threads of a row hold identical values)
    stats[(half * 2 + 0) * TILE_ROWS + r] = m;
    stats[(half * 2 + 1) * TILE_ROWS + r] = l;
    asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_THREADS) : "memory");
    {
      const float m0 = stats[0 * TILE_ROWS + r], l0 = stats[1 * TILE_ROWS + r];
      const float m1 = stats[2 * TILE_ROWS + r], l1 = stats[3 * TILE_ROWS + r];
      m = fmaxf(m0, m1);
      l = l0 * expf(m0 - m) + l1 * expf(m1 - m);
    }
    const float rl = __frcp_rn(l);
    // ---- pass 2: probabilities -> P tile -> O += P . V
    uint8_t* prow = sP + r * 128;
    const int sw = r & 7;
#pragma unroll 1
    for (int j = 0; j < nt && ok; ++j) {
      fetch_s();
      if (!ok) break;
      const int c0 = j * TILE_ROWS + half * 64;
      const bool all_visible = c0 + 63 <= t0 + p.past;
      uint32_t w[16];
      to_scores(c0, all_visible);
      auto prob = [&](uint32_t sbits) {  // a masked key has score -FLT_MAX: expf gives 0, the probability is 0
        const float e = expf(__uint_as_float(sbits) - m);
        return __float2int_rn(__fmul_rn(div_by_row_sum(e, l, rl), 127.f));
      };
#pragma unroll
      for (int q4 = 0; q4 < 8; ++q4) {
        w[q4] = pack_sat_s8x4(prob(va[q4 * 4]), prob(va[q4 * 4 + 1]), prob(va[q4 * 4 + 2]), prob(va[q4 * 4 + 3]));
        w[8 + q4] = pack_sat_s8x4(prob(vb[q4 * 4]), prob(vb[q4 * 4 + 1]), prob(vb[q4 * 4 + 2]), prob(vb[q4 * 4 + 3]));
      }
      // P_{j-1} has been consumed by its MMAs (the first wait passes at once)
      ok = mbar_wait_status(smem_u32(p_empty), (j & 1) ^ 1, abort_flag, p.status, TI_ERR_ATT_P_EMPTY);
      if (!ok) break;
      // 16-byte chunk q of row r lives at chunk position q ^ (r % 8) (128-byte swizzle); this thread
      // owns chunks 4*half .. 4*half + 3
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *reinterpret_cast<uint4*>(prow + (((4 * half + q) ^ sw) << 4)) =
            make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(p_full));
    }
    // ---- epilogue: context rows (each thread D/2 columns of its row)
    if (ok) ok = mbar_wait_status(smem_u32(o_full), 0, abort_flag, p.status, TI_ERR_ATT_O_FULL);
    if (ok) {
      tc_fence_after();
      int8_t* orow = p.ctx + static_cast<long long>(b) * p.ctx_batch_stride + static_cast<long long>(rg) * p.ld_ctx +
                     h * D + half * (D / 2);
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        tmem_ld_32x32(tmem_o + lane_off + half * (D / 2) + c * 32, va);
        tmem_ld_wait();
        uint32_t w[8];
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4) {
          int o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            o[i] = __float2int_rn(p.alpha_pv * __int2float_rn(static_cast<int>(va[q4 * 4 + i])));
          w[q4] = pack_sat_s8x4(o[0], o[1], o[2], o[3]);
        }
        if (valid) {
          *reinterpret_cast<uint4*>(orow + c * 32) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(orow + c * 32 + 16) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
    }
  }

  // -------------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up: give copies and MMAs that may still be in flight a bounded grace period
    // before shared memory and TMEM are released.
    const uint64_t t_start = global_timer_ns();
    while (global_timer_ns() - t_start < 200000ull) {
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

template <int D>
int launch(const AttnProblem& a, cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  // Q rows of one sequence and head: [B][Hl][T][D] view of the query columns
  if (!make_operand_map(&tq, a.q, D, a.T, a.heads, a.batch, a.ld_q, D, a.q_batch_stride, TILE_ROWS)) return TI_E_INVALID;
  // key rows: [B][Hl][S][D]
  if (!make_operand_map(&tk, a.k, D, a.S, a.heads, a.batch, a.ld_k, D, a.k_batch_stride, TILE_ROWS)) return TI_E_INVALID;
  // transposed values: [B][Hl][D][S], keys contiguous
  if (!make_operand_map(&tv, a.vt, a.S, D, a.heads, a.batch, a.ld_vt, D * a.ld_vt, a.heads * D * a.ld_vt, D))
    return TI_E_INVALID;
  AttnParams p;
  p.T = static_cast<int>(a.T);
  p.S = static_cast<int>(a.S);
  p.past = static_cast<int>(a.S - a.T);
  p.alpha_qk = a.alpha_qk;
  p.alpha_pv = a.alpha_pv;
  p.ctx = a.ctx;
  p.ld_ctx = a.ld_ctx;
  p.ctx_batch_stride = a.ctx_batch_stride;
  p.status = status_word_ptr();
  if (!p.status) {
    set_error("attention_prefill_s8: cannot resolve the device status word");
    return TI_E_CUDA;
  }
  auto kernel = attention_prefill_s8_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) {
    set_error("attention_prefill_s8: cannot reserve %d bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(e));
    return TI_E_CUDA;
  }
  // two CTAs per SM need 2 x 97 KB: ask for the largest shared-memory carve-out (a hint)
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  const dim3 grid(static_cast<unsigned>((a.T + TILE_ROWS - 1) / TILE_ROWS), static_cast<unsigned>(a.heads),
                  static_cast<unsigned>(a.batch));
  kernel<<<grid, ATT_THREADS, SMEM_BYTES, stream>>>(tq, tk, tv, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("attention_prefill_s8 launch failed: %s", cudaGetErrorString(e));
    return TI_E_CUDA;
  }
  return TI_OK;
}

}  // namespace

int attention_prefill_s8(const AttnProblem& a, cudaStream_t stream) {
  if (a.batch < 0 || a.heads <= 0 || a.T < 0 || a.S < a.T || (a.head_dim != 64 && a.head_dim != 128)) {
    set_error("attention_prefill_s8: head_dim must be 64 or 128 and S >= T >= 0 (got T=%lld S=%lld D=%lld)",
              (long long)a.T, (long long)a.S, (long long)a.head_dim);
    return TI_E_INVALID;
  }
  if (a.batch == 0 || a.T == 0) return TI_OK;
  if (!a.q || !a.k || !a.vt || !a.ctx) {
    set_error("attention_prefill_s8: null pointer");
    return TI_E_INVALID;
  }
  const int64_t el = a.heads * a.head_dim;
  auto misaligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; };
  if (misaligned(a.q) || misaligned(a.k) || misaligned(a.vt) || misaligned(a.ctx) || a.ld_q % 16 || a.ld_k % 16 ||
      a.ld_vt % 16 || a.ld_ctx % 16 || a.q_batch_stride % 16 || a.k_batch_stride % 16 || a.ctx_batch_stride % 16) {
    set_error("attention_prefill_s8: pointers and strides must be multiples of 16 bytes");
    return TI_E_INVALID;
  }
  if (a.ld_q < el || a.ld_k < el || a.ld_ctx < el || a.ld_vt < a.S) {
    set_error("attention_prefill_s8: a row stride is smaller than the row");
    return TI_E_INVALID;
  }
  if (a.batch > 65535 || a.heads > 65535 || a.S > (1 << 24)) {
    set_error("attention_prefill_s8: batch and heads are limited to 65535, S to 2^24");
    return TI_E_INVALID;
  }
  return a.head_dim == 128 ? launch<128>(a, stream) : launch<64>(a, stream);
}

}  // namespace ti
