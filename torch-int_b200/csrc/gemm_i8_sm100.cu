// W8A8 contraction for sm_100a: C[b] = epilogue(A[b] * B[b]^T), A [M,K] and
// B [N,K] int8 with K contiguous (both "K-major"), int32 accumulation.
//
// One persistent CTA per SM walks a list of 128 x BN output tiles.  Inside a
// CTA the work is split by warp:
//   warp 0    TMA producer: cp.async.bulk.tensor loads of a 128 x 128-byte A
//             tile and a BN x 128-byte B tile into a ring of 128B-swizzled
//             shared-memory stages, completion counted on "full" mbarriers;
//   warp 1    MMA issuer: one thread issues tcgen05.mma.kind::i8 (M=128, N=BN,
//             K=32) over each stage, accumulating in TMEM, and hands stages
//             back through tcgen05.commit on "empty" mbarriers;
//   warps 2-5 epilogue: tcgen05.ld the int32 accumulator (one TMEM lane = one
//             output row per thread), apply the fp32 epilogue and store.
// TMEM holds two accumulators (2 x BN columns), so the epilogue of tile i runs
// while the mainloop of tile i+1 fills the other one.
//
// Replaces the CUTLASS 2.x device::Gemm / device::GemmBatched instantiations of
// the reference (torch_int/kernels/linear.cu:34-45,163-172,270-279,393-401,
// 500-519; torch_int/kernels/bmm.cu:33-41,133-141,233-241).  The bias is read
// as a length-N vector in the epilogue instead of a materialised M x N matrix
// (linear.cu:83,420).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include <mutex>

#include "gemm_i8.h"
#include "sm100_ptx.cuh"

namespace ti {

namespace {

constexpr int BM = 128;        // rows of C per tile = TMEM lanes
constexpr int BK = 128;        // bytes (= int8 elements) of K per stage: one swizzle row
constexpr int UMMA_K = 32;     // K per tcgen05.mma for 8-bit operands
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int SMEM_BUDGET = 227 * 1024;

struct KernelParams {
  void* C;
  const void* bias;
  int M, N, K;
  int num_kb;               // ceil(K / BK)
  int m_tiles, n_tiles;     // per batch entry
  int batch, batch2;
  long long ldc, strideC, stride2C;
  long long total_tiles;
  float alpha, beta;
  const float* alpha_vec;
  const float* beta_vec;
  int group_m;              // rasterisation: M tiles per column sweep
  int a_b1, a_b2, b_b1, b_b2;  // 0 where an operand is broadcast over a batch index (stride 0), else 1
  // Row-block scatter of the output (tensor-parallel reduce-scatter fused into the epilogue):
  // rows [i*scatter_rows, (i+1)*scatter_rows) go to scatter[i], which may be another GPU's memory
  // reached by plain peer stores.  scatter_rows == 0: everything goes to C.
  void* scatter[8];
  int scatter_rows;
  // Split-K (small M): the K blocks of a tile are divided over `splits` work items that add their
  // int32 partial accumulators into `ws` ([M][N], zero on entry and on exit); the work item that
  // arrives last at the tile's counter applies the epilogue.  splits == 1: off.
  int splits, kb_per_split;
  int32_t* ws;
  int* counters;
  // 1: launched with programmatic stream serialisation (small-M problems): the kernel may start while
  // the kernel before it still runs.  The B operand is model weights, which no kernel writes, so the
  // producer fetches the B tiles of its first stages at once; everything else (A, the outputs, the
  // split-K scratch) is touched only after grid_dep_wait().
  int pdl;
};

// PAIR = false: one CTA computes a 128 x BN tile (tcgen05 cta_group::1).
// PAIR = true : two CTAs of a cluster compute a 256 x BN tile together
//               (cta_group::2): each loads its own 128 rows of A and its own
//               BN/2 rows of B, the leader CTA issues M=256 MMAs that read both
//               CTAs' shared memory and write 128 accumulator rows into each
//               CTA's TMEM.  Per CTA this halves the B bytes that TMA writes to
//               and the tensor core reads from shared memory.
// AROWS = rows of A that a stage holds.  128 is the tile height.  16 serves problems of at most 16 rows
// (decode steps): the TMA box of A is 16 rows, so a stage is 2 KB + the B tile instead of 16 KB + the B
// tile, and half as many more weight bytes are in flight per SM.  The MMA is still 128 rows high: rows 16
// and up of its A operand are whatever follows in shared memory (the stage's own B tile), which gives
// arbitrary integers in accumulator rows that no epilogue reads.
template <int BN, bool PAIR, int AROWS = BM>
struct Cfg {
  static constexpr int A_BYTES = AROWS * BK;
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;
  static constexpr int B_BYTES = B_ROWS * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // flag word + per epilogue warp with valid rows: 32 rows x (128 + 16) bytes
  static constexpr int XPOSE_BYTES = 16 + (AROWS > 32 ? 4 : 1) * 32 * 144;
  static constexpr int AUX_BYTES = 4 * BN * 4 + 256 + XPOSE_BYTES;  // bias + alpha tiles, barriers, store staging
  static constexpr int STAGES_RAW = (SMEM_BUDGET - 1024 - AUX_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 12 ? 12 : STAGES_RAW;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + AUX_BYTES;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int TILE_M = PAIR ? 2 * BM : BM;
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN must be 32..256, multiple of 32");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM columns must be a power of two");
  static_assert(STAGES >= 2, "need at least two stages");
  static_assert(AROWS == BM || (!PAIR && AROWS == 16 && B_BYTES >= BM * BK - A_BYTES),
                "a narrow A stage needs a B tile behind it that covers the MMA's 128-row read");
  static_assert((2 * STAGES + 4) * 8 + 8 <= 256, "barrier area");
};

struct TileCoord {
  int m_tile, n_tile, b1, b2;
  int kb0, kb1;  // K blocks [kb0, kb1) of this work item
  int parts;     // work items that share this tile (1: this one computes all of it)
};

__device__ __forceinline__ TileCoord decode_tile(long long t, const KernelParams& p) {
  int kb0 = 0, kb1 = p.num_kb;
  if (p.splits > 1) {
    const int split = static_cast<int>(t % p.splits);
    t /= p.splits;
    kb0 = split * p.kb_per_split;
    kb1 = min(p.num_kb, kb0 + p.kb_per_split);
  }
  const int per_batch = p.m_tiles * p.n_tiles;
  const long long bidx = t / per_batch;
  int r = static_cast<int>(t - bidx * per_batch);
  TileCoord c;
  c.b1 = static_cast<int>(bidx % p.batch);
  c.b2 = static_cast<int>(bidx / p.batch);
  // Grouped order: sweep all N tiles for a band of `group_m` M tiles, so CTAs
  // that run at the same time share A rows and B rows in L2.
  const int group_size = p.group_m * p.n_tiles;
  const int g = r / group_size;
  const int first_m = g * p.group_m;
  const int gm = min(p.m_tiles - first_m, p.group_m);
  r -= g * group_size;
  c.m_tile = first_m + r % gm;
  c.n_tile = r / gm;
  c.kb0 = kb0;
  c.kb1 = kb1;
  c.parts = p.splits;
  return c;
}

// The work items of one CTA (or CTA pair), in order: every warp role walks the same sequence.
struct WorkIter {
  long long t, step;
  __device__ WorkIter(long long first, long long stride) : t(first), step(stride) {}
  __device__ bool next(const KernelParams& p, TileCoord& c) {
    if (t >= p.total_tiles) return false;
    c = decode_tile(t, p);
    t += step;
    return true;
  }
};

// Fire-and-forget integer add to global memory: `red` returns nothing, so a thread keeps issuing
// the next ones while these are on their way to L2.
__device__ __forceinline__ void red_add_s32(int32_t* addr, int v) {
  asm volatile("red.relaxed.gpu.global.add.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ int sat_rne_s8(float y) {
  int v = __float2int_rn(y);  // cvt.rni.s32.f32: RNE, saturating, NaN -> 0
  return max(-128, min(127, v));
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  return (static_cast<uint32_t>(a) & 0xFFu) | ((static_cast<uint32_t>(b) & 0xFFu) << 8) |
         ((static_cast<uint32_t>(c) & 0xFFu) << 16) | ((static_cast<uint32_t>(d) & 0xFFu) << 24);
}

template <int EPI>
struct EpiTraits {
  static constexpr bool kOutS8 =
      EPI == EPI_S8_BIAS_S8 || EPI == EPI_S8_BIAS_S8_RELU || EPI == EPI_S8_ALPHA || EPI == EPI_S8_BIAS_S8_VEC;
  static constexpr bool kHasBias = EPI == EPI_S8_BIAS_S8 || EPI == EPI_S8_BIAS_S8_RELU ||
                                   EPI == EPI_F32_BIAS_F32 || EPI == EPI_S32_BIAS_S32_ADD ||
                                   EPI == EPI_S32_BIAS_S32_SCALE || EPI == EPI_S8_BIAS_S8_VEC ||
                                   EPI == EPI_F32_BIAS_F32_ACC;
  static constexpr bool kAddToC = EPI == EPI_F32_BIAS_F32_ACC;  // the fp32 result is added to what C holds
  static constexpr bool kVecAlpha = EPI == EPI_S8_BIAS_S8_VEC;
  static constexpr int kOutBytes = kOutS8 ? 1 : 4;
};

// One accumulator value -> one output value (as raw 32 bits; int8 outputs are
// returned as an int in [-128,127]).  `t` is the bias term prepared per column:
// beta*float(bias) as float bits for the scaled forms, the raw int32 bias for
// EPI_S32_BIAS_S32_ADD.
template <int EPI>
__device__ __forceinline__ uint32_t epilogue_one(uint32_t acc_bits, uint32_t t, float alpha) {
  const int acc = static_cast<int>(acc_bits);
  if constexpr (EPI == EPI_S32_RAW) {
    return acc_bits;
  } else if constexpr (EPI == EPI_S32_BIAS_S32_ADD) {
    return acc_bits + t;  // two's-complement wrap-around
  } else {
    const float a = __int2float_rn(acc);
    float y;
    if constexpr (EPI == EPI_F32_ALPHA || EPI == EPI_S8_ALPHA)
      y = alpha * a;  // (EPI_S8_BIAS_S8_VEC takes the fma branch with its per-column alpha)
    else
      y = __fmaf_rn(alpha, a, __uint_as_float(t));
    if constexpr (EPI == EPI_S8_BIAS_S8_RELU) y = fmaxf(y, 0.f);
    if constexpr (EpiTraits<EPI>::kOutS8)
      return static_cast<uint32_t>(sat_rne_s8(y));
    else if constexpr (EPI == EPI_S32_BIAS_S32_SCALE)
      return static_cast<uint32_t>(__float2int_rn(y));
    else
      return __float_as_uint(y);
  }
}

template <int BN, int EPI, bool PAIR, int AROWS = BM>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const KernelParams p) {
  using C = Cfg<BN, PAIR, AROWS>;
  using T = EpiTraits<EPI>;
  constexpr int CG = PAIR ? 2 : 1;
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* aux = smem + C::STAGES * C::STAGE_BYTES;
  uint32_t* bias_smem = reinterpret_cast<uint32_t*>(aux);  // [2][BN]
  uint32_t* alpha_smem = bias_smem + 2 * BN;               // [2][BN], per-column alphas (VEC epilogue)
  uint64_t* bars = reinterpret_cast<uint64_t*>(aux + 4 * BN * 4);
  uint8_t* xpose = aux + 4 * BN * 4 + 256;  // [4 warps][32 rows][144 bytes]
  uint64_t* full_bar = bars;                    // [STAGES]  (PAIR: only the leader's are used)
  uint64_t* empty_bar = bars + C::STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * C::STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;         // [2]       (PAIR: only the leader's are used)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0;  // 0 = leader of the CTA pair
  const long long first_tile = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  const long long tile_step = PAIR ? (gridDim.x >> 1) : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tfull_bar[b]), 1);
      mbar_init(smem_u32(&tempty_bar[b]), (PAIR ? 2 : 1) * (EPI_THREADS / 32));
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc<CG>(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish<CG>();
  }
  tc_fence_before();
  if constexpr (PAIR)
    cluster_sync_all();  // the peer's barriers must be initialised before any remote arrive
  else
    __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) grid_dep_launch();  // the next kernel may be scheduled as CTAs of this one drain

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int prefetched = 0;  // K blocks (over the first work items) whose stages were filled before the loop
      WorkIter work(first_tile, tile_step);
      if constexpr (!PAIR) {
        if (p.pdl) {
          // Weights of the first K blocks of this CTA's work first: they do not depend on the kernel before
          // this one.  The activations follow once that kernel has completed.
          int a_kb[C::STAGES], a_b1[C::STAGES], a_b2[C::STAGES];
          int n = 0;
          {
            WorkIter ahead = work;
            TileCoord c;
            while (n < C::STAGES && ahead.next(p, c)) {
              for (int kb = c.kb0; kb < c.kb1 && n < C::STAGES; ++kb, ++n) {
                const uint32_t fb = smem_u32(&full_bar[n]);
                mbar_expect_tx(fb, C::STAGE_BYTES);
                tma_load_4d(smem_u32(smem + n * C::STAGE_BYTES + C::A_BYTES), &tmap_b, fb, kb * BK, c.n_tile * BN,
                            c.b1 * p.b_b1, c.b2 * p.b_b2);
                a_kb[n] = kb;
                a_b1[n] = c.b1 * p.a_b1;
                a_b2[n] = c.b2 * p.a_b2;
              }
            }
          }
          grid_dep_wait();
          for (int i = 0; i < n; ++i)  // one M tile (M <= 128): row 0
            tma_load_4d(smem_u32(smem + i * C::STAGE_BYTES), &tmap_a, smem_u32(&full_bar[i]), a_kb[i] * BK, 0, a_b1[i],
                        a_b2[i]);
          prefetched = n;
          stage = n == C::STAGES ? 0 : n;
          phase = n == C::STAGES ? 1 : 0;
        }
      }
      TileCoord tc;
      while (ok && work.next(p, tc)) {
        const int row_a = tc.m_tile * C::TILE_M + static_cast<int>(rank) * BM;
        const int row_b = tc.n_tile * BN + static_cast<int>(rank) * C::B_ROWS;
        const int skip = min(prefetched, tc.kb1 - tc.kb0);
        prefetched -= skip;
        const int kb_first = tc.kb0 + skip;
        for (int kb = kb_first; kb < tc.kb1; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, TI_ERR_WAIT_EMPTY);
          if (!ok) break;
          uint8_t* sa = smem + stage * C::STAGE_BYTES;
          if constexpr (PAIR) {
            // Both CTAs' loads count their bytes on the LEADER's barrier, which
            // therefore completes when the operands of the whole 256-row MMA are in
            // place.  Only the leader arrives on it, expecting the bytes of both CTAs
            // (the peer's bytes may be counted before or after that arrive; the phase
            // cannot complete until the arrive has happened).  A remote
            // arrive.expect_tx with cluster-scope release from the peer was measured
            // to halve the throughput of the whole kernel.
            const uint32_t fb = mapa_shared(smem_u32(&full_bar[stage]), 0);
            if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[stage]), 2 * C::STAGE_BYTES);
            tma_load_4d_pair(smem_u32(sa), &tmap_a, fb, kb * BK, row_a, tc.b1 * p.a_b1, tc.b2 * p.a_b2);
            tma_load_4d_pair(smem_u32(sa + C::A_BYTES), &tmap_b, fb, kb * BK, row_b, tc.b1 * p.b_b1,
                             tc.b2 * p.b_b2);
          } else {
            const uint32_t fb = smem_u32(&full_bar[stage]);
            mbar_expect_tx(fb, C::STAGE_BYTES);
            tma_load_4d(smem_u32(sa), &tmap_a, fb, kb * BK, row_a, tc.b1 * p.a_b1, tc.b2 * p.a_b2);
            tma_load_4d(smem_u32(sa + C::A_BYTES), &tmap_b, fb, kb * BK, row_b, tc.b1 * p.b_b1, tc.b2 * p.b_b2);
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_s8s8s32(C::TILE_M, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      WorkIter work(first_tile, tile_step);
      TileCoord tc;
      for (; ok && work.next(p, tc); ++it) {
        const int buf = it & 1;
        const int kb0 = tc.kb0, kb1 = tc.kb1;
        ok = mbar_wait<PAIR>(smem_u32(&tempty_bar[buf]), ((it >> 1) & 1) ^ 1, abort_flag,
                             TI_ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, TI_ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint64_t da = make_smem_desc_sw128(sa);
          const uint64_t db = make_smem_desc_sw128(sa + C::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // +32 bytes of K inside the 128-byte swizzle row = +2 in the
            // (address >> 4) field of the descriptor.
            umma_i8<CG>(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb != kb0) || (k != 0));
          }
          // Hand the stage back to the producer(s) once these MMAs have read it.
          if constexpr (PAIR) {
            umma_commit_pair_both(smem_u32(&empty_bar[stage]));
          } else {
            umma_commit(smem_u32(&empty_bar[stage]));
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          if constexpr (PAIR) {
            umma_commit_pair_both(smem_u32(&tfull_bar[buf]));
          } else {
            umma_commit(smem_u32(&tfull_bar[buf]));
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    if (p.pdl) grid_dep_wait();  // outputs and the split-K scratch may still be in use by the kernel before
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    const int et = threadIdx.x - 64;
    int it = 0;
    bool ok = true;
    WorkIter work(first_tile, tile_step);
    TileCoord tc;
    for (; ok && work.next(p, tc); ++it) {
      const int buf = it & 1;
      const int n0 = tc.n_tile * BN;
      if constexpr (T::kHasBias) {
        uint32_t* bs = bias_smem + buf * BN;
        for (int j = et; j < BN; j += EPI_THREADS) {
          const int n = n0 + j;
          uint32_t v = 0;
          if (n < p.N) {
            if constexpr (EPI == EPI_S8_BIAS_S8_VEC) {
              v = __float_as_uint(p.beta_vec[n] * static_cast<float>(static_cast<const int8_t*>(p.bias)[n]));
              alpha_smem[buf * BN + j] = __float_as_uint(p.alpha_vec[n]);
            } else if constexpr (EPI == EPI_S8_BIAS_S8 || EPI == EPI_S8_BIAS_S8_RELU)
              v = __float_as_uint(p.beta * static_cast<float>(static_cast<const int8_t*>(p.bias)[n]));
            else if constexpr (EPI == EPI_F32_BIAS_F32 || EPI == EPI_F32_BIAS_F32_ACC)
              v = __float_as_uint(p.beta * static_cast<const float*>(p.bias)[n]);
            else if constexpr (EPI == EPI_S32_BIAS_S32_SCALE)
              v = __float_as_uint(p.beta *
                                  __int2float_rn(static_cast<const int32_t*>(p.bias)[n]));
            else
              v = static_cast<uint32_t>(static_cast<const int32_t*>(p.bias)[n]);
          }
          bs[j] = v;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
      }
      ok = mbar_wait(smem_u32(&tfull_bar[buf]), (it >> 1) & 1, abort_flag, TI_ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();

      const int row0 = tc.m_tile * C::TILE_M + static_cast<int>(rank) * BM + quarter * 32;  // first row of this warp
      // Address of output row r (this tile's column 0).
      auto row_ptr = [&](int r) -> uint8_t* {
        if (p.scatter_rows > 0) {
          const int owner = min(r / p.scatter_rows, 7);
          return static_cast<uint8_t*>(p.scatter[owner]) +
                 (static_cast<long long>(r - owner * p.scatter_rows) * p.ldc + n0) * T::kOutBytes;
        }
        return static_cast<uint8_t*>(p.C) +
               (static_cast<long long>(tc.b2) * p.stride2C + static_cast<long long>(tc.b1) * p.strideC +
                static_cast<long long>(r) * p.ldc + n0) *
                   T::kOutBytes;
      };
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
      const uint32_t* bs = bias_smem + buf * BN;
      if (tc.parts > 1) {
        // ---- split-K: add this work item's partial sums into the workspace ----
        // Rows are transposed through the warp's shared-memory patch so that lane L adds column L of
        // every valid row: each warp-wide reduction touches 128 contiguous bytes of the workspace.
        const int valid = min(32, p.M - row0);  // valid rows of this warp (<= 0: none)
        uint8_t* patch = xpose + 16 + quarter * (32 * 144);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if (n0 + c * 32 >= p.N || valid <= 0) break;
          uint32_t v[32];
          __syncwarp();
          tmem_ld_32x32(taddr + c * 32, v);
          tmem_ld_wait();
          if (valid > 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4*>(patch + lane * 144 + q * 16) =
                  make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            __syncwarp();
            const int col = n0 + c * 32 + lane;
            if (col < p.N) {
              int32_t* wcol = p.ws + static_cast<long long>(row0) * p.N + col;
#pragma unroll 4
              for (int r = 0; r < valid; ++r)
                red_add_s32(wcol + static_cast<long long>(r) * p.N,
                            *reinterpret_cast<const int*>(patch + r * 144 + lane * 4));
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[buf]));  // the accumulator is drained
        // ---- the last work item of the tile finishes it ----
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        if (et == 0) {
          const int old = atomicAdd(p.counters + tc.n_tile, 1);
          *reinterpret_cast<volatile int*>(xpose) = (old == tc.parts - 1) ? 1 : 0;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        const bool last = *reinterpret_cast<volatile int*>(xpose) != 0;
        if (last) {
          __threadfence();
          for (int j = et; j < BN; j += EPI_THREADS) {
            const int col = n0 + j;
            if (col >= p.N) continue;
            uint32_t tb = 0;
            float al = p.alpha;
            if constexpr (T::kHasBias) tb = bs[j];
            if constexpr (T::kVecAlpha) al = __uint_as_float(alpha_smem[buf * BN + j]);
            for (int r0 = 0; r0 < p.M; r0 += 8) {
              int acc[8];
#pragma unroll
              for (int i = 0; i < 8; ++i)  // eight independent loads in flight
                acc[i] = r0 + i < p.M ? __ldcg(p.ws + static_cast<long long>(r0 + i) * p.N + col) : 0;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int r = r0 + i;
                if (r >= p.M) break;
                p.ws[static_cast<long long>(r) * p.N + col] = 0;  // leave the workspace clean
                const uint32_t o = epilogue_one<EPI>(static_cast<uint32_t>(acc[i]), tb, al);
                uint8_t* dst =
                    static_cast<uint8_t*>(p.C) + (static_cast<long long>(r) * p.ldc + col) * T::kOutBytes;
                if constexpr (T::kOutS8)
                  *reinterpret_cast<int8_t*>(dst) = static_cast<int8_t>(static_cast<int>(o));
                else if constexpr (T::kAddToC)
                  *reinterpret_cast<float*>(dst) = *reinterpret_cast<const float*>(dst) + __uint_as_float(o);
                else
                  *reinterpret_cast<uint32_t*>(dst) = o;
              }
            }
          }
          if (et == 0) p.counters[tc.n_tile] = 0;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");  // xpose[0] is reused by the next tile
        continue;
      }
      if constexpr (T::kOutS8) {
        // int8 rows: a thread owns one row and writes its 32 bytes of each chunk as two 16-byte stores
        // (one full 32-byte sector).
        const int row = row0 + lane;
        const bool row_ok = row < p.M;
        uint8_t* crow = row_ptr(row_ok ? row : 0);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if (n0 + c * 32 >= p.N || row0 >= p.M) break;  // uniform over the warp
          uint32_t v[32];
          __syncwarp();
          tmem_ld_32x32(taddr + c * 32, v);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              uint4 tb = make_uint4(0, 0, 0, 0);
              if constexpr (T::kHasBias) tb = reinterpret_cast<const uint4*>(bs)[c * 8 + q];
              float a0 = p.alpha, a1 = p.alpha, a2 = p.alpha, a3 = p.alpha;
              if constexpr (T::kVecAlpha) {
                const uint4 ta = reinterpret_cast<const uint4*>(alpha_smem + buf * BN)[c * 8 + q];
                a0 = __uint_as_float(ta.x); a1 = __uint_as_float(ta.y);
                a2 = __uint_as_float(ta.z); a3 = __uint_as_float(ta.w);
              }
              v[q * 4 + 0] = epilogue_one<EPI>(v[q * 4 + 0], tb.x, a0);
              v[q * 4 + 1] = epilogue_one<EPI>(v[q * 4 + 1], tb.y, a1);
              v[q * 4 + 2] = epilogue_one<EPI>(v[q * 4 + 2], tb.z, a2);
              v[q * 4 + 3] = epilogue_one<EPI>(v[q * 4 + 3], tb.w, a3);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (n0 + c * 32 + h * 16 < p.N) {
                uint4 o;
                o.x = pack4(v[h * 16 + 0], v[h * 16 + 1], v[h * 16 + 2], v[h * 16 + 3]);
                o.y = pack4(v[h * 16 + 4], v[h * 16 + 5], v[h * 16 + 6], v[h * 16 + 7]);
                o.z = pack4(v[h * 16 + 8], v[h * 16 + 9], v[h * 16 + 10], v[h * 16 + 11]);
                o.w = pack4(v[h * 16 + 12], v[h * 16 + 13], v[h * 16 + 14], v[h * 16 + 15]);
                *reinterpret_cast<uint4*>(crow + c * 32 + h * 16) = o;
              }
            }
          }
        }
      } else {
        // 32-bit outputs: the 32 rows x 128 bytes of a chunk are transposed through a per-warp
        // shared-memory patch so that eight lanes write one row's 128 contiguous bytes - full lines
        // for local HBM and efficient packets when the destination is a peer GPU.
        uint8_t* patch = xpose + 16 + quarter * (32 * 144);
        const int sub = lane >> 3, piece = lane & 7;  // this lane stores piece `piece` of rows sub, sub+4, ...
        uint8_t* rp[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = row0 + i * 4 + sub;
          rp[i] = r < p.M ? row_ptr(r) + piece * 16 : nullptr;
        }
        // EPI_F32_BIAS_F32_ACC: the values of C this lane adds to, fetched one chunk ahead of their use
        uint4 held[8];
        auto fetch_c = [&](int c, uint4 (&dst)[8]) {
          const bool in_range = n0 + c * 32 + piece * 4 < p.N;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = (in_range && rp[i] != nullptr) ? *reinterpret_cast<const uint4*>(rp[i] + c * 128)
                                                   : make_uint4(0, 0, 0, 0);
        };
        if constexpr (T::kAddToC) {
          if (row0 < p.M && n0 < p.N) fetch_c(0, held);
        }
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if (n0 + c * 32 >= p.N) break;  // uniform over the CTA
          if (row0 >= p.M) break;  // no valid row in this warp (its patch may not exist: narrow A stages)
          uint4 ahead[8];
          if constexpr (T::kAddToC) {
            if (c + 1 < BN / 32) fetch_c(c + 1, ahead);  // zeros beyond N
          }
          uint32_t v[32];
          __syncwarp();
          tmem_ld_32x32(taddr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            uint4 tb = make_uint4(0, 0, 0, 0);
            if constexpr (T::kHasBias) tb = reinterpret_cast<const uint4*>(bs)[c * 8 + q];
            uint4 o;
            o.x = epilogue_one<EPI>(v[q * 4 + 0], tb.x, p.alpha);
            o.y = epilogue_one<EPI>(v[q * 4 + 1], tb.y, p.alpha);
            o.z = epilogue_one<EPI>(v[q * 4 + 2], tb.z, p.alpha);
            o.w = epilogue_one<EPI>(v[q * 4 + 3], tb.w, p.alpha);
            *reinterpret_cast<uint4*>(patch + lane * 144 + q * 16) = o;
          }
          __syncwarp();
          const bool col_ok = n0 + c * 32 + piece * 4 < p.N;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint4 o = *reinterpret_cast<const uint4*>(patch + (i * 4 + sub) * 144 + piece * 16);
            if constexpr (T::kAddToC) {
              o.x = __float_as_uint(__uint_as_float(held[i].x) + __uint_as_float(o.x));
              o.y = __float_as_uint(__uint_as_float(held[i].y) + __uint_as_float(o.y));
              o.z = __float_as_uint(__uint_as_float(held[i].z) + __uint_as_float(o.z));
              o.w = __float_as_uint(__uint_as_float(held[i].w) + __uint_as_float(o.w));
            }
            if (col_ok && rp[i] != nullptr) *reinterpret_cast<uint4*>(rp[i] + c * 128) = o;
          }
          if constexpr (T::kAddToC) {
            if (c + 1 < BN / 32) {
#pragma unroll
              for (int i = 0; i < 8; ++i) held[i] = ahead[i];
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR)
          mbar_arrive_remote(mapa_shared(smem_u32(&tempty_bar[buf]), 0));
        else
          mbar_arrive(smem_u32(&tempty_bar[buf]));
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before();
  // In a CTA pair neither CTA may release shared memory or TMEM while the other
  // can still signal its barriers or the leader's MMAs can still read its tiles.
  if constexpr (PAIR)
    cluster_sync_all();
  else
    __syncthreads();
  if (*abort_flag) {
    // A wait gave up: give copies and MMAs that may still be in flight a bounded
    // grace period before shared memory and TMEM are released.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  if constexpr (PAIR)
    cluster_sync_all();
  else
    __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CG>(tmem_base, C::TMEM_COLS);
  }
}

// ----------------------------------------------------------------- host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

}  // namespace

// K-major int8 operand [batch2, batch, rows, K] -> 4-D tensor map with a
// (128 bytes of K) x box_rows x 1 x 1 box, 128-byte swizzle, zero fill.
bool make_operand_map(void* tensor_map, const int8_t* ptr, int64_t K, int64_t rows, int64_t batch,
                      int64_t batch2, int64_t ld, int64_t stride, int64_t stride2, int box_rows) {
  CUtensorMap* map = static_cast<CUtensorMap*>(tensor_map);
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return false;
  }
  // A batch index with stride 0 (broadcast operand) becomes a dimension of extent 1;
  // the kernel then always passes coordinate 0 for it.
  if (stride == 0 || batch == 1) {
    batch = 1;
    stride = ld * rows;
  }
  if (stride2 == 0 || batch2 == 1) {
    batch2 = 1;
    stride2 = stride * batch;
  }
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(batch), static_cast<cuuint64_t>(batch2)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ld), static_cast<cuuint64_t>(stride),
                           static_cast<cuuint64_t>(stride2)};
  cuuint32_t box[4] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (CUresult %d) for K=%lld rows=%lld batch=%lld x %lld "
              "ld=%lld stride=%lld stride2=%lld",
              static_cast<int>(r), (long long)K, (long long)rows, (long long)batch,
              (long long)batch2, (long long)ld, (long long)stride, (long long)stride2);
    return false;
  }
  return true;
}

namespace {

// Upper bound on the SMs the persistent GEMM grid occupies (0 = all).  A caller that
// overlaps collectives with the GEMMs lowers it so that the collective's CTAs find free SMs.
int g_sm_limit = 0;
// Rasterisation band override for tuning (0 = choose automatically).
int g_group_m = 0;
// Small-M launches use programmatic dependent launch (1) or ordinary stream order (0).
int g_pdl = 1;
// Problems of at most 16 rows use 16-row A stages (1) or the full 128-row ones (0).
int g_narrow_a = 1;

int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  const int n = cached[dev];
  return (g_sm_limit > 0 && g_sm_limit < n) ? g_sm_limit : n;
}

// Split-K workspace layout: one int counter per N tile (sized for the narrowest tile, 256-byte
// padded), then the [M][N] int32 accumulator.
int64_t counter_bytes(int bn, int64_t N) {
  (void)bn;
  const int64_t tiles = (N + 31) / 32;
  return (tiles * 4 + 255) / 256 * 256;
}

template <int BN, int EPI, bool PAIR, int AROWS = BM>
int launch_one(const GemmProblem& g, int splits, cudaStream_t stream) {
  using C = Cfg<BN, PAIR, AROWS>;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_i8_kernel<BN, EPI, PAIR, AROWS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(%d bytes) failed: %s", C::SMEM_BYTES, cudaGetErrorString(e));
      return TI_E_CUDA;
    }
    attr_done[dev] = true;
  }
  CUtensorMap ta, tb;
  if (!make_operand_map(&ta, g.A, g.K, g.M, g.batch, g.batch2, g.lda, g.strideA, g.stride2A, AROWS))
    return TI_E_CUDA;
  if (!make_operand_map(&tb, g.B, g.K, g.N, g.batch, g.batch2, g.ldb, g.strideB, g.stride2B, C::B_ROWS))
    return TI_E_CUDA;
  KernelParams p;
  p.C = g.C;
  p.bias = g.bias;
  p.M = static_cast<int>(g.M);
  p.N = static_cast<int>(g.N);
  p.K = static_cast<int>(g.K);
  p.num_kb = static_cast<int>((g.K + BK - 1) / BK);
  p.m_tiles = static_cast<int>((g.M + C::TILE_M - 1) / C::TILE_M);
  p.n_tiles = static_cast<int>((g.N + BN - 1) / BN);
  p.batch = static_cast<int>(g.batch);
  p.batch2 = static_cast<int>(g.batch2);
  p.ldc = g.ldc;
  p.strideC = g.strideC;
  p.stride2C = g.stride2C;
  p.total_tiles = static_cast<long long>(p.m_tiles) * p.n_tiles * g.batch * g.batch2;
  p.alpha = g.alpha;
  p.beta = g.beta;
  p.alpha_vec = g.alpha_vec;
  p.beta_vec = g.beta_vec;
  // Rasterisation band: M tiles swept per pass over the N tiles.  Wide bands re-read B less often but
  // need the band's A rows to stay in L2.  Measured on the model shapes (M = 4096): a band of 16 pair
  // tiles wins while its A rows stay below about 32 MB (K <= 8192: out_proj 165 -> 147 us, q/k/v
  // 479 -> 440 us), bands of 8 win beyond (K = 12288, 28672).
  p.group_m = PAIR ? 8 : 16;
  if (g_group_m > 0) {
    p.group_m = g_group_m;
  } else if (PAIR) {
    const int gm = p.m_tiles < 32 ? p.m_tiles : 32;
    if (gm > 8 && static_cast<long long>(gm) * C::TILE_M * g.K <= (32ll << 20)) p.group_m = gm;
  }
  p.a_b1 = (g.strideA != 0 && g.batch > 1) ? 1 : 0;
  p.a_b2 = (g.stride2A != 0 && g.batch2 > 1) ? 1 : 0;
  p.b_b1 = (g.strideB != 0 && g.batch > 1) ? 1 : 0;
  p.b_b2 = (g.stride2B != 0 && g.batch2 > 1) ? 1 : 0;
  p.scatter_rows = static_cast<int>(g.scatter_rows);
  for (int i = 0; i < 8; ++i) p.scatter[i] = g.scatter_rows > 0 ? g.scatter_ptrs[i] : nullptr;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.ws = nullptr;
  p.counters = nullptr;
  p.pdl = (!PAIR && g_pdl && g.M <= BM && g.scatter_rows == 0) ? 1 : 0;
  if (!PAIR && splits > 1) {
    p.kb_per_split = (p.num_kb + splits - 1) / splits;
    p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
    if (p.splits > 1) {
      p.counters = static_cast<int*>(g.ws);
      p.ws = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(g.ws) + counter_bytes(BN, g.N));
      p.total_tiles *= p.splits;
    } else {
      p.kb_per_split = p.num_kb;
    }
  }
  const int sms = num_sms();
  const long long workers = PAIR ? sms / 2 : sms;  // CTAs, or CTA pairs
  const int grid = static_cast<int>(p.total_tiles < workers ? p.total_tiles : workers) * (PAIR ? 2 : 1);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_i8_kernel<BN, EPI, PAIR, AROWS>, ta, tb, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_error("gemm_i8_kernel<%d,%d,%d> launch failed: %s", BN, EPI, PAIR ? 1 : 0, cudaGetErrorString(e));
    return TI_E_CUDA;
  }
  return TI_OK;
}

template <int EPI>
int launch_bn(const GemmProblem& g, int bn, bool pair, int splits, cudaStream_t stream) {
  if (pair) return launch_one<256, EPI, true>(g, 1, stream);
  if (g_narrow_a && g.M <= 16) {  // decode steps: narrow A stages, deeper weight pipeline
    if (bn == 256) return launch_one<256, EPI, false, 16>(g, splits, stream);
    if (bn == 128) return launch_one<128, EPI, false, 16>(g, splits, stream);
  }
  switch (bn) {
    case 256: return launch_one<256, EPI, false>(g, splits, stream);
    case 128: return launch_one<128, EPI, false>(g, splits, stream);
    case 64: return launch_one<64, EPI, false>(g, splits, stream);
    case 32: return launch_one<32, EPI, false>(g, splits, stream);
  }
  set_error("unsupported N tile %d", bn);
  return TI_E_INVALID;
}

// Pick the tile shape.  The cost of a configuration is (waves over the SMs) x
// (cycles one 32-byte K slice of one tile takes).  A slice is bound either by
// the tensor pipe (N/2 cycles for 128 rows) or by shared-memory bandwidth
// (128 B/cycle, shared by the TMA writes and the tensor core's reads of A and
// B).  The CTA-pair form does 256 rows per slice with only half of B per CTA.
void choose_tile(const GemmProblem& g, int* bn_out, bool* pair_out) {
  const int cands[4] = {256, 128, 64, 32};
  const int sms = num_sms();
  const long long m_tiles = (g.M + BM - 1) / BM;
  const long long nb = g.batch * g.batch2;
  double best = 1e300;
  int best_bn = 256;
  bool best_pair = false;
  for (int i = 0; i < 4; ++i) {
    const int bn = cands[i];
    if (bn > 32 && bn / 2 >= g.N) continue;  // tile mostly padding
    const long long tiles = m_tiles * ((g.N + bn - 1) / bn) * nb;
    const long long waves = (tiles + sms - 1) / sms;
    const double mma = bn / 2.0;
    const double smem = 2.0 * (4096.0 + 32.0 * bn) / 128.0;
    const double cost = static_cast<double>(waves) * (mma > smem ? mma : smem);
    if (cost < best * 0.999) {
      best = cost;
      best_bn = bn;
    }
  }
  if (g.force_pair != 1 && g.M > BM && g.N > 128) {
    const long long tiles = ((g.M + 2 * BM - 1) / (2 * BM)) * ((g.N + 255) / 256) * nb;
    const long long pairs = sms / 2;
    const long long waves = (tiles + pairs - 1) / pairs;
    const double cost = static_cast<double>(waves) * 128.0;  // mma 128 = smem 2*(4096+4096)/128
    if (cost < best * 1.001 || g.force_pair == 2) {
      best_bn = 256;
      best_pair = true;
    }
  }
  *bn_out = best_bn;
  *pair_out = best_pair;
}

// Tile width and number of K splits for a small-M problem (weights streamed once, HBM bound).  Model, in
// microseconds, fitted to measurements at M = 8 on the OPT-30B decode shapes: a work item costs
// (K blocks per item) x (bytes of B per K block = 128 x bn) / (an SM's share of HBM bandwidth, 44 B/ns)
// plus 4.3 us for the pipeline fill, the partial-sum reduction and the last-CTA epilogue; the launch
// takes as many such rounds as the busiest CTA of the persistent grid has items.  `force_bn` != 0
// restricts the tile width, `wanted` > 1 asks for that many splits (capped so that a split keeps at
// least 8 K blocks).
void choose_small_m(int64_t N, int64_t K, int force_bn, int wanted, int* bn_out, int* splits_out) {
  const long long num_kb = (K + BK - 1) / BK;
  const long long sms = num_sms();
  long long max_splits = num_kb / 8 > 0 ? num_kb / 8 : 1;
  if (max_splits > 64) max_splits = 64;
  const int cands[3] = {256, 128, 64};
  double best = 1e300;
  int best_bn = force_bn ? force_bn : 128, best_sp = 1;
  for (int i = 0; i < 3; ++i) {
    const int bn = cands[i];
    if (force_bn && bn != force_bn) continue;
    if (!force_bn && bn > 64 && bn / 2 >= N) continue;  // tile mostly padding
    const long long tiles = (N + bn - 1) / bn;
    const long long lo = wanted > 1 ? (wanted < max_splits ? wanted : max_splits) : 1;
    const long long hi = wanted > 1 ? lo : (wanted == 1 ? 1 : max_splits);
    for (long long sp = lo; sp <= hi; ++sp) {
      const long long per = (num_kb + sp - 1) / sp;
      const long long eff = (num_kb + per - 1) / per;  // no empty split
      const long long rounds = (tiles * eff + sms - 1) / sms;
      const double cost = static_cast<double>(rounds) * (static_cast<double>(per) * bn * 0.0029 + 4.3) +
                          (eff > 1 ? 0.0 : -1.0);  // no scratch traffic at all without a split
      if (cost < best * 0.999) {
        best = cost;
        best_bn = bn;
        best_sp = static_cast<int>(eff);
      }
    }
  }
  *bn_out = best_bn;
  *splits_out = best_sp;
}

}  // namespace

int split_k_auto_splits(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || M > BM || N <= 0 || K <= 0) return 1;
  int bn = 0, splits = 1;
  choose_small_m(N, K, 0, 0, &bn, &splits);
  return splits;
}

int launch_gemm_i8(const GemmProblem& g, cudaStream_t stream) {
  if (g.M < 0 || g.N < 0 || g.K < 0 || g.batch < 0 || g.batch2 < 0) {
    set_error("negative dimension");
    return TI_E_INVALID;
  }
  if (g.M == 0 || g.N == 0 || g.batch == 0 || g.batch2 == 0) return TI_OK;  // empty output
  if (g.K == 0) {
    set_error("K must be positive");
    return TI_E_INVALID;
  }
  if (!g.A || !g.B || (!g.C && g.scatter_rows == 0)) {
    set_error("null operand pointer");
    return TI_E_INVALID;
  }
  if (g.scatter_rows != 0) {
    const int64_t blocks = g.scatter_rows > 0 ? (g.M + g.scatter_rows - 1) / g.scatter_rows : 0;
    if (g.scatter_rows < 0 || blocks > 8 || g.batch != 1 || g.batch2 != 1) {
      set_error("output scatter needs batch == 1 and at most 8 row blocks");
      return TI_E_INVALID;
    }
    for (int64_t i = 0; i < blocks; ++i)
      if (!g.scatter_ptrs[i] || (reinterpret_cast<uintptr_t>(g.scatter_ptrs[i]) & 15)) {
        set_error("output scatter pointers must be non-null and 16-byte aligned");
        return TI_E_INVALID;
      }
  }
  const bool out_s8 = g.epilogue == EPI_S8_BIAS_S8 || g.epilogue == EPI_S8_BIAS_S8_RELU ||
                      g.epilogue == EPI_S8_ALPHA || g.epilogue == EPI_S8_BIAS_S8_VEC;
  const bool has_bias = g.epilogue == EPI_S8_BIAS_S8 || g.epilogue == EPI_S8_BIAS_S8_RELU ||
                        g.epilogue == EPI_F32_BIAS_F32 || g.epilogue == EPI_S32_BIAS_S32_ADD ||
                        g.epilogue == EPI_S32_BIAS_S32_SCALE || g.epilogue == EPI_S8_BIAS_S8_VEC ||
                        g.epilogue == EPI_F32_BIAS_F32_ACC;
  if (g.epilogue == EPI_F32_BIAS_F32_ACC && g.scatter_rows != 0) {
    set_error("the epilogue that adds to C cannot scatter its output");
    return TI_E_INVALID;
  }
  if (g.epilogue == EPI_S8_BIAS_S8_VEC && (!g.alpha_vec || !g.beta_vec)) {
    set_error("the per-column epilogue needs alpha and beta vectors");
    return TI_E_INVALID;
  }
  if (has_bias && !g.bias) {
    set_error("this epilogue needs a bias vector");
    return TI_E_INVALID;
  }
  // The shape rules of the reference kernels (128-bit vector accesses): K a
  // multiple of 16, N a multiple of 16 for int8 outputs and of 4 for 32-bit
  // outputs.  They are also what TMA (16-byte strides) and the 16-byte stores
  // of the epilogue need.
  if (g.K % 16 != 0) {
    set_error("K=%lld must be a multiple of 16", (long long)g.K);
    return TI_E_INVALID;
  }
  const int nmult = out_s8 ? 16 : 4;
  if (g.N % nmult != 0) {
    set_error("N=%lld must be a multiple of %d for this output type", (long long)g.N, nmult);
    return TI_E_INVALID;
  }
  if (g.lda % 16 || g.ldb % 16 || g.strideA % 16 || g.strideB % 16 || g.stride2A % 16 ||
      g.stride2B % 16 || g.lda < g.K || g.ldb < g.K) {
    set_error("operand strides must be multiples of 16 elements and >= K");
    return TI_E_INVALID;
  }
  if (g.ldc % nmult || g.strideC % nmult || g.stride2C % nmult || g.ldc < g.N) {
    set_error("output strides must be multiples of %d elements and ldc >= N", nmult);
    return TI_E_INVALID;
  }
  if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.B) |
       (g.scatter_rows ? 0 : reinterpret_cast<uintptr_t>(g.C))) & 15) {
    set_error("operand and output pointers must be 16-byte aligned");
    return TI_E_INVALID;
  }
  if (g.M > 0x7FFFFFFF - 256 || g.N > 0x7FFFFFFF - 256 || g.K > 0x7FFFFFFF - 256 ||
      g.batch > 0x7FFFFFFF || g.batch2 > 0x7FFFFFFF) {
    set_error("dimension too large");
    return TI_E_INVALID;
  }
  int bn = 256;
  bool pair = false;
  if (g.force_bn) {
    bn = g.force_bn;
    pair = g.force_pair == 2 && bn == 256;
  } else {
    choose_tile(g, &bn, &pair);
  }
  // Split-K for small M: with one M tile and few N tiles most SMs would idle while a few stream
  // all of the weights; splitting K puts every SM to work.  Needs a workspace.
  int splits = 1;
  if (g.ws != nullptr && !pair && g.M <= BM && g.batch == 1 && g.batch2 == 1 && g.scatter_rows == 0 &&
      g.splits != 1) {
    if (g.ws_bytes < split_k_workspace_bytes(g.M, g.N)) {
      set_error("split-K workspace too small: %lld bytes given, %lld needed", (long long)g.ws_bytes,
                (long long)split_k_workspace_bytes(g.M, g.N));
      return TI_E_INVALID;
    }
    if ((reinterpret_cast<uintptr_t>(g.ws) & 255) != 0) {
      set_error("split-K workspace must be 256-byte aligned");
      return TI_E_INVALID;
    }
    int bn_small = bn;
    choose_small_m(g.N, g.K, g.force_bn, g.splits, &bn_small, &splits);
    bn = bn_small;  // with or without a split: the width that streams the weights fastest
  }
  switch (g.epilogue) {
    case EPI_S8_BIAS_S8: return launch_bn<EPI_S8_BIAS_S8>(g, bn, pair, splits, stream);
    case EPI_S8_BIAS_S8_RELU: return launch_bn<EPI_S8_BIAS_S8_RELU>(g, bn, pair, splits, stream);
    case EPI_F32_BIAS_F32: return launch_bn<EPI_F32_BIAS_F32>(g, bn, pair, splits, stream);
    case EPI_S32_BIAS_S32_ADD: return launch_bn<EPI_S32_BIAS_S32_ADD>(g, bn, pair, splits, stream);
    case EPI_S32_BIAS_S32_SCALE: return launch_bn<EPI_S32_BIAS_S32_SCALE>(g, bn, pair, splits, stream);
    case EPI_F32_ALPHA: return launch_bn<EPI_F32_ALPHA>(g, bn, pair, splits, stream);
    case EPI_S8_ALPHA: return launch_bn<EPI_S8_ALPHA>(g, bn, pair, splits, stream);
    case EPI_S32_RAW: return launch_bn<EPI_S32_RAW>(g, bn, pair, splits, stream);
    case EPI_S8_BIAS_S8_VEC: return launch_bn<EPI_S8_BIAS_S8_VEC>(g, bn, pair, splits, stream);
    case EPI_F32_BIAS_F32_ACC: return launch_bn<EPI_F32_BIAS_F32_ACC>(g, bn, pair, splits, stream);
  }
  set_error("unknown epilogue %d", g.epilogue);
  return TI_E_INVALID;
}

// ------------------------------------------------- entry point that allocates nothing
//
// ti_linear_a8_w8_b8_o8_static: the int8-output linear for few rows (decode steps) with its
// split-K scratch taken from a fixed array inside this library instead of from the caller.
//
// Who needs this: hosts that are not allowed to allocate device memory when they call us.
// Examples are an inference server that reserves the whole GPU up front and hands plug-ins no
// allocator; a latency-critical serving loop in which cudaMalloc (an implicit device
// synchronisation) is banned after start-up; and code that runs after the framework's
// caching allocator has been frozen.  Such a caller cannot provide ti_gemm_desc.workspace,
// yet without split-K a 16-row problem keeps most SMs idle.  So the scratch lives here, as a
// file-scope device array: every GPU that loads this library holds its kStaticScratchBytes
// (4 MiB) until the process exits, whether or not the entry point is ever called.
//
// Rules that follow from sharing one array:
//   * sizes whose scratch need (ti_split_k_workspace_bytes(M, N)) exceeds the array, or
//     M > 128, are refused with an error - nothing is allocated as a fallback;
//   * the array keeps whatever the last call left in it.  The split-K kernel needs it all zero
//     on entry and restores every word it touched to zero before it ends, and the array starts
//     zeroed when the library is loaded, so consecutive calls on one stream are safe;
//   * the one exception: a launch whose bounded wait gave up (ti_device_status reports non-zero)
//     may leave partial sums and counters behind.  ti_device_status(reset != 0) clears the array
//     together with the status word; until then results of this entry point are not trustworthy;
//   * two calls that overlap on the GPU (different streams, or different host threads feeding
//     different streams) would add into the same words: do not do that - serialise them;
//   * the array's name is only a host-side handle; the device address is looked up with
//     cudaGetSymbolAddress the first time the entry point runs on a device (with that device
//     current) and cached.  Make that first call before any stream capture begins.
namespace {
constexpr long long kStaticScratchBytes = 4ll << 20;
}
static __device__ __align__(256) unsigned char ti_static_scratch[kStaticScratchBytes];

namespace {
std::mutex g_static_scratch_mutex;
void* g_static_scratch_ptr[64] = {nullptr};

// Device address of ti_static_scratch on the current device (set up once per device).
int static_scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("ti_linear_a8_w8_b8_o8_static: cannot identify the current device");
    return TI_E_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), ti_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_error("ti_linear_a8_w8_b8_o8_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return TI_E_CUDA;
    }
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return TI_OK;
}
}  // namespace

// Device address of the status word, for kernels of other translation units.
int* status_word_ptr() {
  static int* cached[64] = {nullptr};  // resolved once per device (not during stream capture)
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, ti_kernel_status) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}

int64_t split_k_workspace_bytes(int64_t M, int64_t N) { return counter_bytes(32, N) + M * N * 4; }

void set_sm_limit(int sms) { g_sm_limit = sms > 0 ? sms : 0; }

void set_group_m(int tiles) { g_group_m = tiles > 0 ? tiles : 0; }

void set_dependent_launch(int on) { g_pdl = on ? 1 : 0; }

void set_narrow_a(int on) { g_narrow_a = on ? 1 : 0; }

// Reads (and optionally clears) the status word the kernels of this file set
// when a bounded wait gives up.  Synchronises the device.
int device_status(int* status, bool reset) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_error("cudaDeviceSynchronize failed: %s", cudaGetErrorString(e));
    return TI_E_CUDA;
  }
  int v = 0;
  e = cudaMemcpyFromSymbol(&v, ti_kernel_status, sizeof(int));
  if (e != cudaSuccess) {
    set_error("cudaMemcpyFromSymbol failed: %s", cudaGetErrorString(e));
    return TI_E_CUDA;
  }
  if (reset && v != 0) {
    // A kernel whose wait gave up may have left partial sums and tile counters in the split-K scratch,
    // which every later launch expects to find all zero: clear the built-in array along with the word
    // (the device is idle here; a caller-provided workspace must be cleared by its owner).
    const int zero = 0;
    cudaMemcpyToSymbol(ti_kernel_status, &zero, sizeof(int));
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
      std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
      if (g_static_scratch_ptr[dev] != nullptr) {
        cudaMemset(g_static_scratch_ptr[dev], 0, static_cast<size_t>(kStaticScratchBytes));
        cudaDeviceSynchronize();
      }
    }
  }
  *status = v;
  return TI_OK;
}

}  // namespace ti

#pragma GCC visibility push(default)
extern "C" int ti_linear_a8_w8_b8_o8_static(const int8_t* input, const int8_t* weight, const int8_t* bias,
                                            int8_t* out, int64_t M, int64_t N, int64_t K, float alpha,
                                            float beta, void* stream) {
  using namespace ti;
  if (M < 0 || N < 0 || K < 0) {
    set_error("ti_linear_a8_w8_b8_o8_static: negative dimension");
    return TI_E_INVALID;
  }
  if (M > 128) {
    set_error("ti_linear_a8_w8_b8_o8_static: M=%lld exceeds the 128 rows this entry point handles "
              "(use ti_linear_a8_w8_b8_o8, which needs no scratch for large M)", (long long)M);
    return TI_E_INVALID;
  }
  const long long need = split_k_workspace_bytes(M, N);
  if (need > kStaticScratchBytes) {
    set_error("ti_linear_a8_w8_b8_o8_static: M=%lld x N=%lld needs %lld bytes of scratch, the built-in array "
              "holds %lld; nothing is allocated as a fallback",
              (long long)M, (long long)N, need, kStaticScratchBytes);
    return TI_E_INVALID;
  }
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != TI_OK) return rc;
  GemmProblem g;
  g.A = input;
  g.B = weight;
  g.C = out;
  g.bias = bias;
  g.M = M;
  g.N = N;
  g.K = K;
  g.lda = K;
  g.ldb = K;
  g.ldc = N;
  g.strideA = M * K;
  g.strideB = N * K;
  g.strideC = M * N;
  g.stride2A = g.strideA;
  g.stride2B = g.strideB;
  g.stride2C = g.strideC;
  g.alpha = alpha;
  g.beta = beta;
  g.epilogue = EPI_S8_BIAS_S8;
  g.ws = scratch;  // the looked-up device address, never the symbol itself
  g.ws_bytes = kStaticScratchBytes;
  g.splits = 0;
  return launch_gemm_i8(g, static_cast<cudaStream_t>(stream));
}
#pragma GCC visibility pop

namespace ti {

// ------------------------------------------------------------ error plumbing
namespace {
thread_local char g_err[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

const char* last_error() { return g_err; }

}  // namespace ti
