// Host launchers of the bandwidth-bound row kernels (LayerNorm-quantise,
// dequant-add-LayerNorm-quantise, softmax-quantise).  All return 0 or a
// negative TI_E_* code with the message in last_error().
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ti {

// Row kernels on at most 32 rows (decode steps) are launched as programmatic dependents of the kernel before
// them (default on): their launch latency overlaps that kernel's last CTAs and they pull their per-layer
// parameters toward L2 before they wait for it.
void set_row_dependent_launch(int on);

int layernorm_q(const void* x, int x_is_half, const float* gamma, const float* beta, float eps,
                int8_t* q, int64_t rows, int64_t H, cudaStream_t stream);

// `in_bias` (fp32, H elements) is optional; see the kernel for its meaning.
int dq_add_layernorm_q(const int32_t* in, float scale, const void* res, int res_is_half,
                       const float* in_bias, const float* gamma, const float* beta, float eps,
                       void* res_out, int8_t* q, int64_t rows, int64_t H, cudaStream_t stream);

// scores [batch_heads, T, S] fp32 (row stride lds), optional additive mask
// [batch_heads / heads, T, S] fp32, out int8 [batch_heads, T, S] (row stride
// ldo).  causal < 0: no generated mask.
int softmax_q(const float* scores, const float* mask, int8_t* out, int64_t batch_heads, int64_t heads,
              int64_t T, int64_t S, int64_t lds, int64_t ldo, int causal, cudaStream_t stream);

// Tensor-parallel exchange kernels (see the kernels in norm_quant.cu).
// Optional synchronisation folded into tp_reduce_layernorm_q (nullptr: none): the kernel announces this
// rank's partial sums to all ranks, waits for theirs, reduces, and ends only when every rank's reduction
// is complete.  pads[i] = rank i's pad of 16 zero-initialised 32-bit words (peer accessible); epoch grows
// by one per call; counter = a zero-initialised int in this GPU's memory; waits are bounded by limit_ms.
struct TpSync {
  void* const* pads;
  int rank, n;
  uint32_t epoch;
  int* counter;
  int* status;
  int64_t limit_ms;
};
int tp_reduce_layernorm_q(const int32_t* stage, int n_partials, int64_t partial_stride, float scale,
                          const float* in_bias, const float* res, const float* gamma, const float* beta,
                          float eps, float* res_out, void* const* q_dst, int n_dst, int64_t q_row_offset,
                          int64_t rows, int64_t H, const TpSync* sync, cudaStream_t stream);
int tp_barrier(void* const* pads, int rank, int n, uint32_t epoch, int* status_word, int64_t limit_ms,
               cudaStream_t stream);

// int8 v [B, T, H, D] (token rows ld_in elements apart) -> vt [B, H, D, ld_out], written at
// columns [col0, col0 + T).
int transpose_values(const int8_t* v, int8_t* vt, int64_t B, int64_t T, int64_t H, int64_t D,
                     int64_t ld_in, int64_t ld_out, int64_t col0, cudaStream_t stream);

// One-token attention over the int8 cache with the position read from device memory
// (decode_attention.cu).
int decode_attention_s8(const int8_t* qkv, int64_t ld_qkv, int8_t* keys, int8_t* values_t, int64_t batch,
                        int64_t local_heads, int64_t head_dim, int64_t cap, const int* pos, float alpha_qk,
                        float alpha_pv, int8_t* ctx, int64_t ld_ctx, cudaStream_t stream);
int advance_position(int* pos, int by, cudaStream_t stream);

}  // namespace ti
