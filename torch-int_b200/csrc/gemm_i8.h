// Host-side description of one (batched) int8 x int8 -> int32 contraction with
// a fused epilogue, and the launcher that runs it on the current device.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/torch_int_b200.h"  // TI_OK / TI_E_* status codes

namespace ti {

// Epilogue kinds.  acc = sum_k A[m,k] * B[n,k] in int32; a = float(acc) (RN).
// The float forms compute t = beta * float(bias[n]) (one rounding) and then
// y = fma(alpha, a, t) (one rounding); the *_ALPHA forms compute y = alpha * a.
enum Epilogue : int {
  EPI_S8_BIAS_S8 = 0,      // int8  out = sat_rne(y),            bias int8
  EPI_S8_BIAS_S8_RELU,     // int8  out = sat_rne(max(y, 0)),    bias int8
  EPI_F32_BIAS_F32,        // fp32  out = y,                     bias fp32
  EPI_S32_BIAS_S32_ADD,    // int32 out = acc + bias (wraps),    bias int32
  EPI_S32_BIAS_S32_SCALE,  // int32 out = sat_rne(y),            bias int32
  EPI_F32_ALPHA,           // fp32  out = alpha * a
  EPI_S8_ALPHA,            // int8  out = sat_rne(alpha * a)
  EPI_S32_RAW,             // int32 out = acc
  EPI_S8_BIAS_S8_VEC,      // int8  out = sat_rne(fma(alpha[n], a, beta[n] * f32(bias[n]))): per-column scales
  EPI_F32_BIAS_F32_ACC,    // fp32  out = out + y (C is read and added to),  bias fp32
  EPI_COUNT
};

// A is [batch2, batch, M, K], B is [batch2, batch, N, K], C is
// [batch2, batch, M, N]; all strides are in elements, K and N are contiguous.
struct GemmProblem {
  const int8_t* A = nullptr;
  const int8_t* B = nullptr;
  void* C = nullptr;
  const void* bias = nullptr;  // N elements (type per epilogue) or nullptr
  int64_t M = 0, N = 0, K = 0;
  int64_t batch = 1, batch2 = 1;
  int64_t lda = 0, ldb = 0, ldc = 0;
  int64_t strideA = 0, strideB = 0, strideC = 0;     // per `batch` index
  int64_t stride2A = 0, stride2B = 0, stride2C = 0;  // per `batch2` index
  float alpha = 1.f, beta = 0.f;
  const float* alpha_vec = nullptr;  // EPI_S8_BIAS_S8_VEC: N per-column alphas
  const float* beta_vec = nullptr;   // EPI_S8_BIAS_S8_VEC: N per-column betas
  int epilogue = EPI_S32_RAW;
  int force_bn = 0;    // 0 = choose the N tile automatically
  int force_pair = 0;  // 0 = automatic, 1 = single-CTA tiles only, 2 = CTA-pair tiles (256 x 256)
  // Optional row-block scatter of the output: rows [i*scatter_rows, (i+1)*scatter_rows) are
  // written to scatter_ptrs[i] (row stride ldc) instead of C.  0 = off.
  // Optional split-K workspace for small-M problems (M <= 128, batch 1): zero-filled on first use,
  // left zero-filled by every launch; ws_bytes >= split_k_workspace_bytes(M, N).  nullptr: no split-K.
  void* ws = nullptr;
  int64_t ws_bytes = 0;
  int splits = 0;  // 0 = choose; 1 = off; else the number of K splits wanted
  int64_t scatter_rows = 0;
  void* scatter_ptrs[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
};

// Returns 0 or a negative TI_E_* code (message via set_error()).
int launch_gemm_i8(const GemmProblem& p, cudaStream_t stream);

// Bytes of split-K workspace a problem with M rows and N columns needs.
int64_t split_k_workspace_bytes(int64_t M, int64_t N);

// K splits the automatic choice makes for an M x N x K problem that is given a workspace (1 = no split:
// M > 128, or enough N tiles to fill the SMs).
int split_k_auto_splits(int64_t M, int64_t N, int64_t K);

// Caps the number of SMs the persistent GEMM grids use (0 = all SMs of the device).
void set_sm_limit(int sms);

// Tuning knob: M tiles per rasterisation band of the GEMM tile order (0 = automatic).
void set_group_m(int tiles);

// Small-M GEMMs (decode steps) are launched with programmatic stream serialisation (default on): they
// start fetching weights while the kernel before them drains.  0 turns that off.
void set_dependent_launch(int on);

// Problems of at most 16 rows stage 16 rows of A per pipeline stage instead of 128 (default on), which
// leaves room for half as many more weight bytes in flight per SM.  0: the 128-row stages.
void set_narrow_a(int on);

// Tensor map (CUtensorMap, 128 bytes, passed as an opaque pointer so that this header needs no
// driver API types) of a K-major int8 operand [batch2, batch, rows, K]: box = 128 bytes of K x
// box_rows x 1 x 1, 128-byte swizzle, out-of-range elements read as zero.  A batch index of extent
// 1 or stride 0 becomes a dimension of extent 1.  Returns false after set_error().
bool make_operand_map(void* tensor_map, const int8_t* ptr, int64_t K, int64_t rows, int64_t batch,
                      int64_t batch2, int64_t ld, int64_t stride, int64_t stride2, int box_rows);

// Status word set by kernels whose bounded waits gave up (0 = ok).
int* status_word_ptr();
int device_status(int* status, bool reset);

// Error plumbing shared by all host entry points.
void set_error(const char* fmt, ...);
const char* last_error();


}  // namespace ti
