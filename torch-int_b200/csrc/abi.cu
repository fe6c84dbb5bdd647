// extern "C" entry points of libtorch_int_b200.so (declared in
// include/torch_int_b200.h).  Each one fills a GemmProblem or calls a row-kernel
// launcher; nothing here allocates or synchronises.
#include "../../include/torch_int_b200.h"

#include "attention_prefill.h"
#include "gemm_i8.h"
#include "norm_quant.h"

using namespace ti;

namespace {

int linear(const int8_t* x, const int8_t* w, const void* bias, void* out, int64_t M, int64_t N,
           int64_t K, float alpha, float beta, int epi, void* stream) {
  GemmProblem g;
  g.A = x;
  g.B = w;
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
  g.epilogue = epi;
  return launch_gemm_i8(g, static_cast<cudaStream_t>(stream));
}

int bmm(const int8_t* A, const int8_t* B, void* C, int64_t batch, int64_t M, int64_t N, int64_t K,
        float alpha, int epi, void* stream) {
  GemmProblem g;
  g.A = A;
  g.B = B;
  g.C = C;
  g.M = M;
  g.N = N;
  g.K = K;
  g.batch = batch;
  g.lda = K;
  g.ldb = K;
  g.ldc = N;
  g.strideA = M * K;
  g.strideB = N * K;
  g.strideC = M * N;
  g.stride2A = batch * g.strideA;
  g.stride2B = batch * g.strideB;
  g.stride2C = batch * g.strideC;
  g.alpha = alpha;
  g.epilogue = epi;
  return launch_gemm_i8(g, static_cast<cudaStream_t>(stream));
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

int ti_linear_a8_w8_b8_o8(const int8_t* input, const int8_t* weight, const int8_t* bias,
                          int8_t* out, int64_t M, int64_t N, int64_t K, float alpha, float beta,
                          void* stream) {
  return linear(input, weight, bias, out, M, N, K, alpha, beta, EPI_S8_BIAS_S8, stream);
}

int ti_linear_relu_a8_w8_b8_o8(const int8_t* input, const int8_t* weight, const int8_t* bias,
                               int8_t* out, int64_t M, int64_t N, int64_t K, float alpha,
                               float beta, void* stream) {
  return linear(input, weight, bias, out, M, N, K, alpha, beta, EPI_S8_BIAS_S8_RELU, stream);
}

int ti_linear_a8_w8_bfp32_ofp32(const int8_t* input, const int8_t* weight, const float* bias,
                                float* out, int64_t M, int64_t N, int64_t K, float alpha,
                                float beta, void* stream) {
  return linear(input, weight, bias, out, M, N, K, alpha, beta, EPI_F32_BIAS_F32, stream);
}

int ti_linear_a8_w8_b32_o32(const int8_t* input, const int8_t* weight, const int32_t* bias,
                            int32_t* out, int64_t M, int64_t N, int64_t K, void* stream) {
  return linear(input, weight, bias, out, M, N, K, 1.f, 1.f, EPI_S32_BIAS_S32_ADD, stream);
}

int ti_linear_a8_w8_b32_o32_with_scaling(const int8_t* input, const int8_t* weight,
                                         const int32_t* bias, int32_t* out, int64_t M, int64_t N,
                                         int64_t K, float alpha, float beta, void* stream) {
  return linear(input, weight, bias, out, M, N, K, alpha, beta, EPI_S32_BIAS_S32_SCALE, stream);
}

int ti_bmm_s8t_s8n_f32t(const int8_t* A, const int8_t* B, float* C, int64_t batch, int64_t M,
                        int64_t N, int64_t K, float alpha, void* stream) {
  return bmm(A, B, C, batch, M, N, K, alpha, EPI_F32_ALPHA, stream);
}

int ti_bmm_s8t_s8n_s8t(const int8_t* A, const int8_t* B, int8_t* C, int64_t batch, int64_t M,
                       int64_t N, int64_t K, float alpha, void* stream) {
  return bmm(A, B, C, batch, M, N, K, alpha, EPI_S8_ALPHA, stream);
}

int ti_bmm_s8t_s8n_s32t(const int8_t* A, const int8_t* B, int32_t* C, int64_t batch, int64_t M,
                        int64_t N, int64_t K, void* stream) {
  return bmm(A, B, C, batch, M, N, K, 1.f, EPI_S32_RAW, stream);
}

int ti_gemm_i8_ex(const ti_gemm_desc* d, void* stream) {
  if (d == nullptr) {
    set_error("ti_gemm_i8_ex: null descriptor");
    return TI_E_INVALID;
  }
  if (d->epilogue < 0 || d->epilogue >= EPI_COUNT) {
    set_error("ti_gemm_i8_ex: unknown epilogue %d", d->epilogue);
    return TI_E_INVALID;
  }
  if (d->tile_n != 0 && d->tile_n != 32 && d->tile_n != 64 && d->tile_n != 128 && d->tile_n != 256) {
    set_error("ti_gemm_i8_ex: tile_n must be 0, 32, 64, 128 or 256");
    return TI_E_INVALID;
  }
  if (d->cta_pair < 0 || d->cta_pair > 2) {
    set_error("ti_gemm_i8_ex: cta_pair must be 0, 1 or 2");
    return TI_E_INVALID;
  }
  GemmProblem g;
  g.A = d->A;
  g.B = d->B;
  g.C = d->C;
  g.bias = d->bias;
  g.M = d->M;
  g.N = d->N;
  g.K = d->K;
  g.batch = d->batch;
  g.batch2 = d->batch2;
  g.lda = d->lda;
  g.ldb = d->ldb;
  g.ldc = d->ldc;
  g.strideA = d->strideA;
  g.strideB = d->strideB;
  g.strideC = d->strideC;
  g.stride2A = d->stride2A;
  g.stride2B = d->stride2B;
  g.stride2C = d->stride2C;
  g.alpha = d->alpha;
  g.beta = d->beta;
  g.ws = d->workspace;
  g.ws_bytes = d->workspace_bytes;
  g.splits = d->splits;
  g.alpha_vec = d->alpha_vec;
  g.beta_vec = d->beta_vec;
  g.epilogue = d->epilogue;
  g.force_bn = d->tile_n;
  g.force_pair = d->cta_pair;
  g.scatter_rows = d->scatter_rows;
  for (int i = 0; i < 8; ++i) g.scatter_ptrs[i] = d->scatter_ptrs[i];
  return launch_gemm_i8(g, static_cast<cudaStream_t>(stream));
}

int ti_dq_add_layernorm_q(const int32_t* input, float input_scale, const void* residual,
                          int residual_is_half, const float* gamma, const float* beta, float eps,
                          void* residual_out, int8_t* q, int64_t rows, int64_t H, void* stream) {
  return dq_add_layernorm_q(input, input_scale, residual, residual_is_half, nullptr, gamma, beta, eps,
                            residual_out, q, rows, H, static_cast<cudaStream_t>(stream));
}

int ti_dq_add_layernorm_q_bias(const int32_t* input, float input_scale, const float* input_bias,
                               const void* residual, int residual_is_half, const float* gamma,
                               const float* beta, float eps, void* residual_out, int8_t* q,
                               int64_t rows, int64_t H, void* stream) {
  if (input_bias == nullptr) {
    set_error("ti_dq_add_layernorm_q_bias: null bias");
    return TI_E_INVALID;
  }
  return dq_add_layernorm_q(input, input_scale, residual, residual_is_half, input_bias, gamma, beta,
                            eps, residual_out, q, rows, H, static_cast<cudaStream_t>(stream));
}

int ti_layernorm_q(const void* x, int x_is_half, const float* gamma, const float* beta, float eps,
                   int8_t* q, int64_t rows, int64_t H, void* stream) {
  return layernorm_q(x, x_is_half, gamma, beta, eps, q, rows, H, static_cast<cudaStream_t>(stream));
}

int ti_softmax_q(const float* scores, const float* mask, int8_t* probs, int64_t batch_heads,
                 int64_t heads, int64_t T, int64_t S, int64_t lds, int64_t ldp, int causal,
                 void* stream) {
  return softmax_q(scores, mask, probs, batch_heads, heads, T, S, lds, ldp, causal,
                   static_cast<cudaStream_t>(stream));
}

int ti_transpose_values(const int8_t* v, int8_t* vt, int64_t B, int64_t T, int64_t H, int64_t D,
                        int64_t ld_in, int64_t ld_out, int64_t col0, void* stream) {
  return transpose_values(v, vt, B, T, H, D, ld_in, ld_out, col0, static_cast<cudaStream_t>(stream));
}

int ti_decode_attention_s8(const int8_t* qkv, int64_t ld_qkv, int8_t* keys, int8_t* values_t, int64_t batch,
                           int64_t local_heads, int64_t head_dim, int64_t capacity, const int32_t* position,
                           float alpha_qk, float alpha_pv, int8_t* ctx, int64_t ld_ctx, void* stream) {
  return decode_attention_s8(qkv, ld_qkv, keys, values_t, batch, local_heads, head_dim, capacity, position,
                             alpha_qk, alpha_pv, ctx, ld_ctx, static_cast<cudaStream_t>(stream));
}

int ti_advance_position(int32_t* position, int32_t by, void* stream) {
  return advance_position(position, by, static_cast<cudaStream_t>(stream));
}

int ti_attention_prefill_s8(const int8_t* q, int64_t ld_q, int64_t q_batch_stride, const int8_t* k, int64_t ld_k,
                            int64_t k_batch_stride, const int8_t* vt, int64_t ld_vt, int8_t* ctx, int64_t ld_ctx,
                            int64_t ctx_batch_stride, int64_t batch, int64_t heads, int64_t head_dim, int64_t T,
                            int64_t S, float alpha_qk, float alpha_pv, void* stream) {
  AttnProblem a;
  a.q = q;
  a.k = k;
  a.vt = vt;
  a.ctx = ctx;
  a.batch = batch;
  a.heads = heads;
  a.head_dim = head_dim;
  a.T = T;
  a.S = S;
  a.ld_q = ld_q;
  a.q_batch_stride = q_batch_stride;
  a.ld_k = ld_k;
  a.k_batch_stride = k_batch_stride;
  a.ld_vt = ld_vt;
  a.ld_ctx = ld_ctx;
  a.ctx_batch_stride = ctx_batch_stride;
  a.alpha_qk = alpha_qk;
  a.alpha_pv = alpha_pv;
  return attention_prefill_s8(a, static_cast<cudaStream_t>(stream));
}

const char* ti_last_error(void) { return last_error(); }

int ti_device_status(int* status, int reset) {
  if (status == nullptr) {
    set_error("ti_device_status: null pointer");
    return TI_E_INVALID;
  }
  return device_status(status, reset != 0);
}

int ti_check_device(int reset) {
  int v = 0;
  const int rc = device_status(&v, reset != 0);
  if (rc != TI_OK) return rc;
  if (v != 0) {
    set_error("a kernel's bounded wait gave up (status %d)", v);
    return TI_E_DEVICE;
  }
  return TI_OK;
}

int ti_tp_reduce_layernorm_q(const int32_t* stage, int32_t n_partials, int64_t partial_stride,
                             float scale, const float* bias, const float* residual, const float* gamma,
                             const float* beta, float eps, float* residual_out, void* const* q_dst,
                             int32_t n_dst, int64_t q_row_offset, int64_t rows, int64_t H, void* stream) {
  return tp_reduce_layernorm_q(stage, n_partials, partial_stride, scale, bias, residual, gamma, beta, eps,
                               residual_out, q_dst, n_dst, q_row_offset, rows, H, nullptr,
                               static_cast<cudaStream_t>(stream));
}

int ti_tp_exchange_reduce_layernorm_q(const int32_t* stage, int32_t n_partials, int64_t partial_stride,
                                      float scale, const float* bias, const float* residual, const float* gamma,
                                      const float* beta, float eps, float* residual_out, void* const* q_dst,
                                      int32_t n_dst, int64_t q_row_offset, int64_t rows, int64_t H,
                                      void* const* pads, int32_t rank, int32_t n, uint32_t epoch,
                                      int32_t* counter, int64_t limit_ms, void* stream) {
  TpSync sync;
  sync.pads = pads;
  sync.rank = rank;
  sync.n = n;
  sync.epoch = epoch;
  sync.counter = counter;
  sync.status = status_word_ptr();
  sync.limit_ms = limit_ms;
  if (sync.status == nullptr) {
    set_error("ti_tp_exchange_reduce_layernorm_q: cannot resolve the device status word");
    return TI_E_CUDA;
  }
  return tp_reduce_layernorm_q(stage, n_partials, partial_stride, scale, bias, residual, gamma, beta, eps,
                               residual_out, q_dst, n_dst, q_row_offset, rows, H, &sync,
                               static_cast<cudaStream_t>(stream));
}

int ti_tp_barrier_limit(void* const* pads, int32_t rank, int32_t n, uint32_t epoch, int64_t limit_ms,
                        void* stream) {
  int* status = status_word_ptr();
  if (status == nullptr) {
    set_error("ti_tp_barrier: cannot resolve the device status word");
    return TI_E_CUDA;
  }
  return tp_barrier(pads, rank, n, epoch, status, limit_ms, static_cast<cudaStream_t>(stream));
}

int ti_tp_barrier(void* const* pads, int32_t rank, int32_t n, uint32_t epoch, void* stream) {
  return ti_tp_barrier_limit(pads, rank, n, epoch, 2000, stream);
}

int64_t ti_split_k_workspace_bytes(int64_t M, int64_t N) { return split_k_workspace_bytes(M, N); }

int ti_split_k_splits(int64_t M, int64_t N, int64_t K) { return split_k_auto_splits(M, N, K); }

int ti_set_sm_limit(int sms) {
  set_sm_limit(sms);
  return TI_OK;
}

int ti_set_dependent_launch(int on) {
  set_dependent_launch(on);
  set_row_dependent_launch(on);
  return TI_OK;
}

int ti_set_narrow_a(int on) {
  set_narrow_a(on);
  return TI_OK;
}

int ti_set_group_m(int tiles) {
  set_group_m(tiles);
  return TI_OK;
}

int ti_abi_version(void) { return 1; }

}  // extern "C"
#pragma GCC visibility pop
