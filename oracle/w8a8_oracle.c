/* TEST INFRASTRUCTURE - CPU restatement of the reference's W8A8 arithmetic.
 *
 * Only tests/, __graft_entry__.smoke() and the CPU-baseline / reference arms of
 * bench.py may build, load or call this file.  The product (libtorch_int_b200.so
 * and the torch_int package) never does.
 *
 * What it restates (reference = Guangxuan-Xiao/torch-int):
 *   - the int8 x int8 -> int32 contraction every op starts with: A [M,K] row-major
 *     times B [N,K] row-major, i.e. RowMajor x ColumnMajor with int32 accumulation
 *     (torch_int/kernels/linear.cu:30-32, bmm.cu:22-24);
 *   - the per-op epilogues chosen by the reference's CUTLASS template arguments
 *     (linear.cu:41-44, 169-171, 276-278, 399-400, 500-511; bmm.cu:33-35, 133-135,
 *     233-235).  CUTLASS itself (NVIDIA/cutlass, an un-vendored git submodule with
 *     no recoverable pinned commit, .gitmodules:1-4) is absent from the reference
 *     tree, so the epilogue arithmetic follows its published semantics:
 *       a = float(acc)                (round to nearest)
 *       t = beta * float(bias[n])     (one rounding)
 *       y = fma(alpha, a, t)          (one rounding; nvcc contracts alpha*a + t)
 *       no-bias forms: y = alpha * a
 *       int8  out: round to nearest even, saturate to [-128, 127]
 *       int32 out: round to nearest even, saturate to int32
 *       ReLU: y = max(y, 0) before the conversion.
 *
 * Parity pins: the int32 paths are pinned exactly and the int8/fp32 paths to the
 * reference tests' own tolerances by tests/golden (built from the formulas of the
 * reference's tests); the exact rounding order of the float epilogues is pinned
 * only by the CUTLASS semantics above - "parity unpinned" at the last bit of the
 * int8 rounding, because the reference kernels cannot run without a GPU and
 * without CUTLASS.
 *
 * Build: see oracle/Makefile (gcc -O3 -mavx2 -mfma -fopenmp -ffp-contract=off).
 */
#include <immintrin.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define TI_ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ contraction */

/* dot products of RB rows of A against CB rows of B, int16 operands. */
#define RB 2
#define CB 4

__attribute__((target("avx2"))) static void tile_avx2(const int16_t* a, const int16_t* b,
                                                       int64_t K16, int64_t lda, int64_t ldb,
                                                       int32_t out[RB][CB]) {
  __m256i acc[RB][CB];
  for (int r = 0; r < RB; ++r)
    for (int c = 0; c < CB; ++c) acc[r][c] = _mm256_setzero_si256();
  for (int64_t k = 0; k < K16; k += 16) {
    __m256i bv[CB];
    for (int c = 0; c < CB; ++c) bv[c] = _mm256_loadu_si256((const __m256i*)(b + c * ldb + k));
    for (int r = 0; r < RB; ++r) {
      const __m256i av = _mm256_loadu_si256((const __m256i*)(a + r * lda + k));
      for (int c = 0; c < CB; ++c)
        acc[r][c] = _mm256_add_epi32(acc[r][c], _mm256_madd_epi16(av, bv[c]));
    }
  }
  for (int r = 0; r < RB; ++r)
    for (int c = 0; c < CB; ++c) {
      int32_t tmp[8];
      _mm256_storeu_si256((__m256i*)tmp, acc[r][c]);
      int32_t s = 0;
      for (int i = 0; i < 8; ++i) s += tmp[i];
      out[r][c] = s;
    }
}

__attribute__((target("avx512bw"))) static void tile_avx512(const int16_t* a, const int16_t* b,
                                                             int64_t K32, int64_t lda, int64_t ldb,
                                                             int32_t out[RB][CB]) {
  __m512i acc[RB][CB];
  for (int r = 0; r < RB; ++r)
    for (int c = 0; c < CB; ++c) acc[r][c] = _mm512_setzero_si512();
  for (int64_t k = 0; k < K32; k += 32) {
    __m512i bv[CB];
    for (int c = 0; c < CB; ++c) bv[c] = _mm512_loadu_si512((const void*)(b + c * ldb + k));
    for (int r = 0; r < RB; ++r) {
      const __m512i av = _mm512_loadu_si512((const void*)(a + r * lda + k));
      for (int c = 0; c < CB; ++c)
        acc[r][c] = _mm512_add_epi32(acc[r][c], _mm512_madd_epi16(av, bv[c]));
    }
  }
  for (int r = 0; r < RB; ++r)
    for (int c = 0; c < CB; ++c) out[r][c] = _mm512_reduce_add_epi32(acc[r][c]);
}

static int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

static void widen(const int8_t* src, int64_t rows, int64_t K, int64_t ld_src, int16_t* dst,
                  int64_t rows_pad, int64_t Kp) {
  for (int64_t r = 0; r < rows_pad; ++r) {
    int16_t* d = dst + r * Kp;
    if (r < rows) {
      const int8_t* s = src + r * ld_src;
      for (int64_t k = 0; k < K; ++k) d[k] = s[k];
      for (int64_t k = K; k < Kp; ++k) d[k] = 0;
    } else {
      memset(d, 0, (size_t)Kp * sizeof(int16_t));
    }
  }
}

/* C[b][m][n] = sum_k A[b][m][k] * B[b][n][k], exact int32 accumulation (wraps
 * like the hardware would for K >= 131072; no op of the reference gets there).
 * Plain triple loop semantics; blocking and SIMD only change the order of the
 * exact integer additions. */
TI_ORACLE_API void ti_oracle_gemm_acc(const int8_t* A, const int8_t* B, int32_t* C, int64_t batch,
                                      int64_t M, int64_t N, int64_t K) {
  if (batch <= 0 || M <= 0 || N <= 0) return;
  const int use512 = __builtin_cpu_supports("avx512bw");
  const int use256 = __builtin_cpu_supports("avx2");
  const int64_t Kp = round_up(K, 32);
  const int64_t Mp = round_up(M, RB), Np = round_up(N, CB);
  for (int64_t b = 0; b < batch; ++b) {
    const int8_t* Ab = A + b * M * K;
    const int8_t* Bb = B + b * N * K;
    int32_t* Cb = C + b * M * N;
    int16_t* a16 = (int16_t*)aligned_alloc(64, (size_t)(Mp * Kp) * sizeof(int16_t));
    int16_t* b16 = (int16_t*)aligned_alloc(64, (size_t)(Np * Kp) * sizeof(int16_t));
    widen(Ab, M, K, K, a16, Mp, Kp);
    widen(Bb, N, K, K, b16, Np, Kp);
    const int64_t mt = Mp / RB, nt = Np / CB;
    /* 64-column panels of B stay in L2 while all rows of A stream past them. */
    const int64_t NPANEL = 64 / CB;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int64_t np = 0; np < (nt + NPANEL - 1) / NPANEL; ++np) {
      for (int64_t mi = 0; mi < mt; ++mi) {
        const int64_t n_end = (np + 1) * NPANEL < nt ? (np + 1) * NPANEL : nt;
        for (int64_t ni = np * NPANEL; ni < n_end; ++ni) {
          int32_t out[RB][CB];
          const int16_t* ap = a16 + mi * RB * Kp;
          const int16_t* bp = b16 + ni * CB * Kp;
          if (use512) {
            tile_avx512(ap, bp, Kp, Kp, Kp, out);
          } else if (use256) {
            tile_avx2(ap, bp, Kp, Kp, Kp, out);
          } else {
            for (int r = 0; r < RB; ++r)
              for (int c = 0; c < CB; ++c) {
                int32_t s = 0;
                for (int64_t k = 0; k < Kp; ++k) s += (int32_t)ap[r * Kp + k] * (int32_t)bp[c * Kp + k];
                out[r][c] = s;
              }
          }
          for (int r = 0; r < RB; ++r) {
            const int64_t m = mi * RB + r;
            if (m >= M) break;
            for (int c = 0; c < CB; ++c) {
              const int64_t n = ni * CB + c;
              if (n < N) Cb[m * N + n] = out[r][c];
            }
          }
        }
      }
    }
    free(a16);
    free(b16);
  }
}

/* Unblocked scalar form of the same contraction, for cross-checking the SIMD one. */
TI_ORACLE_API void ti_oracle_gemm_acc_naive(const int8_t* A, const int8_t* B, int32_t* C,
                                            int64_t batch, int64_t M, int64_t N, int64_t K) {
  for (int64_t b = 0; b < batch; ++b)
    for (int64_t m = 0; m < M; ++m)
      for (int64_t n = 0; n < N; ++n) {
        int32_t s = 0;
        for (int64_t k = 0; k < K; ++k)
          s += (int32_t)A[(b * M + m) * K + k] * (int32_t)B[(b * N + n) * K + k];
        C[(b * M + m) * N + n] = s;
      }
}

/* -------------------------------------------------------------------- epilogues */

static inline int32_t rne_sat_s32(float y) {
  if (y != y) return 0; /* NaN -> 0, as the device conversion does */
  if (y >= 2147483648.0f) return INT32_MAX;
  if (y <= -2147483648.0f) return INT32_MIN;
  return (int32_t)nearbyintf(y); /* round-to-nearest-even in the default mode */
}

static inline int8_t rne_sat_s8(float y) {
  int32_t v = rne_sat_s32(y);
  if (v > 127) v = 127;
  if (v < -128) v = -128;
  return (int8_t)v;
}

/* linear_a8_w8_b8_o8 (relu = 0, linear.cu:369-473) and linear_relu_a8_w8_b8_o8
 * (relu = 1, linear.cu:476-625): int8 bias, int8 output. */
TI_ORACLE_API void ti_oracle_epi_s8_bias_s8(const int32_t* acc, const int8_t* bias, int8_t* out,
                                            int64_t rows, int64_t N, float alpha, float beta,
                                            int relu) {
#pragma omp parallel for
  for (int64_t m = 0; m < rows; ++m)
    for (int64_t n = 0; n < N; ++n) {
      const float t = beta * (float)bias[n];
      float y = fmaf(alpha, (float)acc[m * N + n], t);
      if (relu) y = y > 0.f ? y : (y != y ? y : 0.f);
      out[m * N + n] = rne_sat_s8(y);
    }
}

/* linear_a8_w8_bfp32_ofp32 (linear.cu:246-365): fp32 bias, fp32 output. */
TI_ORACLE_API void ti_oracle_epi_f32_bias_f32(const int32_t* acc, const float* bias, float* out,
                                              int64_t rows, int64_t N, float alpha, float beta) {
#pragma omp parallel for
  for (int64_t m = 0; m < rows; ++m)
    for (int64_t n = 0; n < N; ++n) {
      const float t = beta * bias[n];
      out[m * N + n] = fmaf(alpha, (float)acc[m * N + n], t);
    }
}

/* linear_a8_w8_b32_o32 (linear.cu:13-136): int32 add with wrap-around. */
TI_ORACLE_API void ti_oracle_epi_s32_bias_s32_add(const int32_t* acc, const int32_t* bias,
                                                  int32_t* out, int64_t rows, int64_t N) {
#pragma omp parallel for
  for (int64_t m = 0; m < rows; ++m)
    for (int64_t n = 0; n < N; ++n)
      out[m * N + n] = (int32_t)((uint32_t)acc[m * N + n] + (uint32_t)bias[n]);
}

/* linear_a8_w8_b32_o32_with_scaling (linear.cu:139-243): int32 bias, int32 output. */
TI_ORACLE_API void ti_oracle_epi_s32_bias_s32_scale(const int32_t* acc, const int32_t* bias,
                                                    int32_t* out, int64_t rows, int64_t N,
                                                    float alpha, float beta) {
#pragma omp parallel for
  for (int64_t m = 0; m < rows; ++m)
    for (int64_t n = 0; n < N; ++n) {
      const float t = beta * (float)bias[n];
      out[m * N + n] = rne_sat_s32(fmaf(alpha, (float)acc[m * N + n], t));
    }
}

/* bmm_s8t_s8n_f32t (bmm.cu:10-108): out = alpha * float(acc). */
TI_ORACLE_API void ti_oracle_epi_f32_alpha(const int32_t* acc, float* out, int64_t count,
                                           float alpha) {
#pragma omp parallel for
  for (int64_t i = 0; i < count; ++i) out[i] = alpha * (float)acc[i];
}

/* bmm_s8t_s8n_s8t (bmm.cu:110-208): out = sat_rne(alpha * float(acc)). */
TI_ORACLE_API void ti_oracle_epi_s8_alpha(const int32_t* acc, int8_t* out, int64_t count,
                                          float alpha) {
#pragma omp parallel for
  for (int64_t i = 0; i < count; ++i) out[i] = rne_sat_s8(alpha * (float)acc[i]);
}

TI_ORACLE_API int ti_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
