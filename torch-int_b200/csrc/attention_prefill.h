// Host-side description of one fused causal prefill attention call (attention_prefill_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ti {

// All strides in bytes (= int8 elements).  Query row t of sequence b, head h starts at
// q + b * q_batch_stride + t * ld_q + h * head_dim; key row j likewise with the k strides;
// vt is [batch][heads][head_dim][ld_vt] with the keys contiguous (the transposed value cache);
// ctx row t of sequence b, head h at ctx + b * ctx_batch_stride + t * ld_ctx + h * head_dim.
// Row t sees keys j <= t + (S - T).
struct AttnProblem {
  const int8_t* q = nullptr;
  const int8_t* k = nullptr;
  const int8_t* vt = nullptr;
  int8_t* ctx = nullptr;
  int64_t batch = 0, heads = 0, head_dim = 0;
  int64_t T = 0;  // query rows per sequence
  int64_t S = 0;  // keys per sequence (cached + new), S >= T
  int64_t ld_q = 0, q_batch_stride = 0;
  int64_t ld_k = 0, k_batch_stride = 0;
  int64_t ld_vt = 0;
  int64_t ld_ctx = 0, ctx_batch_stride = 0;
  float alpha_qk = 1.f, alpha_pv = 1.f;
};

// Returns 0 or a negative TI_E_* code (message via set_error()).
int attention_prefill_s8(const AttnProblem& a, cudaStream_t stream);

}  // namespace ti
