/* C ABI of libtorch_int_b200.so: the W8A8 operator set of torch-int for
 * NVIDIA B200 (sm_100a).
 *
 * Every entry point takes raw DEVICE pointers of the CURRENT CUDA device,
 * sizes as int64_t, scalars as float and a cudaStream_t passed as void*
 * (NULL = the legacy default stream).  Nothing is allocated, nothing
 * synchronises, outputs are written in place by kernels enqueued on `stream`.
 * Return value: 0 on success, negative on error (TI_E_*); the message of the
 * last error of the calling thread is returned by ti_last_error().
 *
 * The ops mirror, one to one, the functions the reference exports from its
 * pybind11 module `torch_int._CUDA` (torch_int/kernels/bindings.cpp:5-20); the
 * citation on each declaration is the reference function it replaces.  Tensor
 * arguments of the reference become (pointer, sizes); the output tensor the
 * reference allocates and returns becomes a caller-provided `out` pointer.
 *
 * Shape rules (the same ones the reference kernels impose through their
 * 128-bit vector accesses): K % 16 == 0; N % 16 == 0 for int8 outputs and
 * N % 4 == 0 for int32 / fp32 outputs; all pointers 16-byte aligned.  M (rows)
 * and the batch count are arbitrary, including 0 (no-op) and 1.
 */
#ifndef TORCH_INT_B200_H
#define TORCH_INT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TI_OK 0
#define TI_E_INVALID (-1) /* bad shape, alignment or pointer */
#define TI_E_CUDA (-2)    /* a CUDA runtime / driver call failed */
#define TI_E_DEVICE (-3)  /* returned by ti_check_device: a kernel's bounded wait gave up */

/* ---- linear layers: out[M,N] = epilogue(input[M,K] . weight[N,K]^T, bias[N]) ---- */

/* int8 out = sat_rne(fma(alpha, float(acc), beta * float(bias))), bias int8.
 * Replaces linear_a8_w8_b8_o8 (torch_int/kernels/linear.cu:369-473). */
int ti_linear_a8_w8_b8_o8(const int8_t* input, const int8_t* weight, const int8_t* bias,
                          int8_t* out, int64_t M, int64_t N, int64_t K, float alpha, float beta,
                          void* stream);

/* Same with max(., 0) before rounding.
 * Replaces linear_relu_a8_w8_b8_o8 (torch_int/kernels/linear.cu:476-625). */
int ti_linear_relu_a8_w8_b8_o8(const int8_t* input, const int8_t* weight, const int8_t* bias,
                               int8_t* out, int64_t M, int64_t N, int64_t K, float alpha,
                               float beta, void* stream);

/* fp32 out = fma(alpha, float(acc), beta * bias), bias fp32.
 * Replaces linear_a8_w8_bfp32_ofp32 (torch_int/kernels/linear.cu:246-365). */
int ti_linear_a8_w8_bfp32_ofp32(const int8_t* input, const int8_t* weight, const float* bias,
                                float* out, int64_t M, int64_t N, int64_t K, float alpha,
                                float beta, void* stream);

/* int32 out = acc + bias (two's-complement wrap), bias int32.
 * Replaces linear_a8_w8_b32_o32 (torch_int/kernels/linear.cu:13-136). */
int ti_linear_a8_w8_b32_o32(const int8_t* input, const int8_t* weight, const int32_t* bias,
                            int32_t* out, int64_t M, int64_t N, int64_t K, void* stream);

/* int32 out = sat_rne(fma(alpha, float(acc), beta * float(bias))), bias int32.
 * Replaces linear_a8_w8_b32_o32_with_scaling (torch_int/kernels/linear.cu:139-243). */
int ti_linear_a8_w8_b32_o32_with_scaling(const int8_t* input, const int8_t* weight,
                                         const int32_t* bias, int32_t* out, int64_t M, int64_t N,
                                         int64_t K, float alpha, float beta, void* stream);

/* Same result as ti_linear_a8_w8_b8_o8 for M <= 128 rows, for callers that may not allocate device
 * memory (an inference server that owns the whole GPU and gives plug-ins no allocator, a serving loop
 * where cudaMalloc's implicit synchronisation is banned after start-up, code running after the
 * framework's allocator was frozen).  The split-K scratch such small problems want is a 4 MiB array
 * built into the library (held by every GPU that loads it until exit); nothing is allocated, here or
 * by any library this calls.  Refused with an error: M > 128, or ti_split_k_workspace_bytes(M, N) >
 * 4 MiB (e.g. M = 16 allows N up to 65024).  The array is shared by all calls and keeps the last
 * call's contents: the kernel re-zeroes what it used, so back-to-back calls on one stream are fine, but
 * calls that overlap on the GPU race on it - serialise them.  If a launch gave up on a bounded wait
 * (ti_device_status reports non-zero) the array may be left non-zero: ti_device_status(reset != 0)
 * clears it together with the status word.  The first call on each device resolves
 * the array's device address (cudaGetSymbolAddress, with that device current); make that first call
 * before starting any stream capture.
 * No counterpart in the reference, which allocates a fresh output and workspace in every call
 * (torch_int/kernels/linear.cu:420,450). */
int ti_linear_a8_w8_b8_o8_static(const int8_t* input, const int8_t* weight, const int8_t* bias,
                                 int8_t* out, int64_t M, int64_t N, int64_t K, float alpha, float beta,
                                 void* stream);

/* ---- batched products: C[b] = epilogue(A[b][M,K] . B[b][N,K]^T), packed tensors ---- */

/* fp32 C = alpha * float(acc).
 * Replaces bmm_s8t_s8n_f32t (torch_int/kernels/bmm.cu:10-108). */
int ti_bmm_s8t_s8n_f32t(const int8_t* A, const int8_t* B, float* C, int64_t batch, int64_t M,
                        int64_t N, int64_t K, float alpha, void* stream);

/* int8 C = sat_rne(alpha * float(acc)).
 * Replaces bmm_s8t_s8n_s8t (torch_int/kernels/bmm.cu:110-208). */
int ti_bmm_s8t_s8n_s8t(const int8_t* A, const int8_t* B, int8_t* C, int64_t batch, int64_t M,
                       int64_t N, int64_t K, float alpha, void* stream);

/* int32 C = acc.
 * Replaces bmm_s8t_s8n_s32t (torch_int/kernels/bmm.cu:210-295). */
int ti_bmm_s8t_s8n_s32t(const int8_t* A, const int8_t* B, int32_t* C, int64_t batch, int64_t M,
                        int64_t N, int64_t K, void* stream);

/* ---- strided form of all of the above ---- */

/* Epilogue selector of ti_gemm_i8_ex. */
enum ti_epilogue {
  TI_EPI_S8_BIAS_S8 = 0,     /* ti_linear_a8_w8_b8_o8 */
  TI_EPI_S8_BIAS_S8_RELU = 1, /* ti_linear_relu_a8_w8_b8_o8 */
  TI_EPI_F32_BIAS_F32 = 2,   /* ti_linear_a8_w8_bfp32_ofp32 */
  TI_EPI_S32_BIAS_S32_ADD = 3, /* ti_linear_a8_w8_b32_o32 */
  TI_EPI_S32_BIAS_S32_SCALE = 4, /* ti_linear_a8_w8_b32_o32_with_scaling */
  TI_EPI_F32_ALPHA = 5,      /* ti_bmm_s8t_s8n_f32t */
  TI_EPI_S8_ALPHA = 6,       /* ti_bmm_s8t_s8n_s8t */
  TI_EPI_S32_RAW = 7,        /* ti_bmm_s8t_s8n_s32t */
  TI_EPI_S8_BIAS_S8_VEC = 8, /* ti_linear_a8_w8_b8_o8 with per-column alpha[n], beta[n] (alpha_vec, beta_vec):
                                several such linears that share their input, e.g. q/k/v, run as one GEMM */
  TI_EPI_F32_BIAS_F32_ACC = 9 /* C (fp32) += fma(alpha, acc, beta * bias): ti_linear_a8_w8_bfp32_ofp32 followed by the
                                in-place residual add of Int8OPTDecoderLayer (torch_int/models/opt.py:281,289:
                                residual.add_(hidden_states)), in the epilogue; C is read and written */
};

/* A [batch2][batch][M][K], B [batch2][batch][N][K], C [batch2][batch][M][N];
 * strides in ELEMENTS; K and N are the contiguous dimensions.  A zero batch
 * stride broadcasts the operand.  Operand strides must be multiples of 16,
 * output strides multiples of 16 (int8 out) or 4 (32-bit out). */
typedef struct ti_gemm_desc {
  const int8_t* A;
  const int8_t* B;
  void* C;
  const void* bias; /* N elements, type per epilogue; NULL when the epilogue has no bias */
  int64_t M, N, K;
  int64_t batch, batch2;
  int64_t lda, ldb, ldc;
  int64_t strideA, strideB, strideC;
  int64_t stride2A, stride2B, stride2C;
  float alpha, beta;
  int32_t epilogue; /* enum ti_epilogue */
  int32_t tile_n;   /* 0 = automatic; else 32, 64, 128 or 256 */
  int32_t cta_pair; /* 0 = automatic; 1 = single-CTA tiles; 2 = 256x256 tiles on CTA pairs (tile_n 0 or 256) */
  /* Optional row-block scatter of the output (batch == batch2 == 1): rows [i*scatter_rows,
   * (i+1)*scatter_rows) are written to scatter_ptrs[i] with row stride ldc instead of C; the
   * pointers may be peer-GPU memory (plain stores).  scatter_rows == 0: off.  This is the
   * reduce-scatter step of a row-parallel linear fused into the GEMM epilogue. */
  int64_t scatter_rows;
  void* scatter_ptrs[8];
  const float* alpha_vec; /* TI_EPI_S8_BIAS_S8_VEC only: N per-column alphas, else NULL */
  const float* beta_vec;  /* TI_EPI_S8_BIAS_S8_VEC only: N per-column betas, else NULL */
  /* Optional split-K scratch for small-M problems (M <= 128, batch == batch2 == 1, no scatter):
   * device memory of at least ti_split_k_workspace_bytes(M, N) bytes, 256-byte aligned, all zero
   * before its first use; every launch leaves it all zero again.  With it, the K dimension of each
   * output tile is divided over several CTAs, which add int32 partial sums into the scratch; the CTA
   * that finishes a tile last applies the epilogue.  Launches that share a workspace must not overlap
   * on the GPU.  NULL: no split-K.  splits: 0 = choose, 1 = off, n = at most n splits. */
  void* workspace;
  int64_t workspace_bytes;
  int32_t splits;
} ti_gemm_desc;

/* The reference has no strided entry point: its wrappers assume packed tensors
 * (torch_int/kernels/linear.cu:429-434, bmm.cu:18-20,71-73) and the attention
 * module makes contiguous copies to satisfy that (torch_int/models/opt.py:80-81,
 * 180,191-196).  This form lets a caller skip those copies. */
int ti_gemm_i8_ex(const ti_gemm_desc* desc, void* stream);

/* Scratch bytes ti_gemm_desc.workspace must provide for an M x N output. */
int64_t ti_split_k_workspace_bytes(int64_t M, int64_t N);

/* Number of K splits the library chooses for an M x N x K problem that is given split-K scratch (a
 * workspace in ti_gemm_desc, or the built-in array of ti_linear_a8_w8_b8_o8_static) on the current device:
 * 1 means the scratch is not touched (M > 128, or N alone fills the SMs).  A query; launches nothing. */
int ti_split_k_splits(int64_t M, int64_t N, int64_t K);

/* ---- LayerNorm-quantise ops ---- */

/* (residual_out, q) = dq_add_layernorm_q(input int32, input_scale, residual, gamma, beta, eps):
 *   residual_out = residual + input_scale * float(input)   (one fused multiply-add)
 *   q = int8(rne(clamp(LayerNorm(residual_out) * gamma + beta, -128, 127)))
 * rows x H row-major tensors; gamma, beta fp32 [H].  residual_is_half: 0 = fp32
 * residual / residual_out, 1 = fp16 (then, as torch::add and torch::layer_norm do for an fp16 tensor,
 * the int32 input is converted to fp16 first and the LayerNorm output is rounded to fp16 before it is
 * quantised; statistics are fp32).
 * Replaces dq_add_layernorm_q (torch_int/kernels/fused.cu:7-25), which issues
 * five ATen kernels. */
int ti_dq_add_layernorm_q(const int32_t* input, float input_scale, const void* residual,
                          int residual_is_half, const float* gamma, const float* beta, float eps,
                          void* residual_out, int8_t* q, int64_t rows, int64_t H, void* stream);

/* The residual update of Int8OPTDecoderLayer with the preceding fp32-output linear folded in
 * (torch_int/models/opt.py:281,289 after torch_int/nn/linear.py:213-214), then the next LayerNormQ:
 *   d = fma(input_scale, float(input), input_bias)     the linear's fp32 output from its int32 accumulator
 *   residual_out = residual + d                        fp32; with residual_is_half = 1, d is cast to fp16
 *                                                      and added in fp16, as residual.add_(d.to(fp16)) does
 *   q = int8(rne(clamp(LayerNorm(residual_out) * gamma + beta)))   in fp32 (LayerNormQ's fp32 parameters)
 * No single reference counterpart; `input` may be an accumulator summed across tensor-parallel ranks,
 * so that the bias of the row-parallel linear is added once, after the reduction. */
int ti_dq_add_layernorm_q_bias(const int32_t* input, float input_scale, const float* input_bias,
                               const void* residual, int residual_is_half, const float* gamma,
                               const float* beta, float eps, void* residual_out, int8_t* q,
                               int64_t rows, int64_t H, void* stream);

/* q = int8(clamp(rne(LayerNorm(x) * gamma + beta), -128, 127)); gamma/beta fp32.  x_is_half: 0 = fp32 x;
 * 2 = fp16 x normalised in fp32 (what LayerNormQ.forward computes with fp32 parameters: it casts x to
 * their dtype first); 1 = fp16 x with the LayerNorm output rounded to fp16 before quantising (parameters
 * cast to fp16 as well).
 * Replaces LayerNormQ.forward (torch_int/nn/fused.py:13-18), four ATen kernels. */
int ti_layernorm_q(const void* x, int x_is_half, const float* gamma, const float* beta, float eps,
                   int8_t* q, int64_t rows, int64_t H, void* stream);

/* probs int8 [batch_heads, T, S] = rne(127 * softmax(max(scores + mask, -FLT_MAX))) row-wise.
 * scores fp32 with row stride lds; mask: optional additive fp32 [batch_heads/heads, T, S]
 * (the reference's [bsz, 1, tgt, src] mask) or NULL; causal >= 0 generates the mask
 * "column j of row t is visible iff j <= t + causal" instead; causal < 0: none.
 * Replaces the mask / softmax / *127 / round / int8 chain of Int8OPTAttention.forward
 * (torch_int/models/opt.py:139-178), five to six ATen kernels. */
int ti_softmax_q(const float* scores, const float* mask, int8_t* probs, int64_t batch_heads,
                 int64_t heads, int64_t T, int64_t S, int64_t lds, int64_t ldp, int causal,
                 void* stream);

/* int8 values v [B, T, H, D] (what v_proj produces; consecutive tokens ld_in >= H*D elements apart,
 * so a column block of a wider projection output can be passed) -> vt [B, H, D, ld_out], written at
 * columns [col0, col0 + T): the transposed, K-major operand of the P.V product.
 * Replaces value_states.transpose(1, 2).contiguous() (torch_int/models/opt.py:180) and lets a
 * pre-allocated cache be filled in place. */
int ti_transpose_values(const int8_t* v, int8_t* vt, int64_t B, int64_t T, int64_t H, int64_t D,
                        int64_t ld_in, int64_t ld_out, int64_t col0, void* stream);

/* Attention of ONE new token per sequence over the int8 key/value cache, in one kernel: appends the
 * token's key row and value column at position *position, then
 *   s_j = alpha_qk * float(q . k_j),  p = int8(rne(127 * softmax(s))),  ctx = sat_rne(alpha_pv * float(p . v))
 * over positions 0 .. *position.  qkv [batch, >= 3*E] holds the token's q | k | v (E = local_heads *
 * head_dim, head_dim 64 or 128); keys [batch, capacity, E]; values_t [batch, local_heads, head_dim,
 * capacity]; ctx [batch, E] with row stride ld_ctx.  `position` is DEVICE memory (tokens already cached,
 * the same for all sequences), so the call has no per-step host parameters and a decode step can be
 * captured in a CUDA graph; ti_advance_position adds to it on the stream.  A full cache sets the status
 * word of ti_device_status to 201 and writes nothing.
 * Replaces, for tgt_len == 1, the torch.cat cache update, bmm_s8t_s8n_f32t, the softmax chain, the value
 * transpose and bmm_s8t_s8n_s8t of Int8OPTAttention.forward (torch_int/models/opt.py:113-116,131-181). */
int ti_decode_attention_s8(const int8_t* qkv, int64_t ld_qkv, int8_t* keys, int8_t* values_t, int64_t batch,
                           int64_t local_heads, int64_t head_dim, int64_t capacity, const int32_t* position,
                           float alpha_qk, float alpha_pv, int8_t* ctx, int64_t ld_ctx, void* stream);
int ti_advance_position(int32_t* position, int32_t by, void* stream);

/* Causal prefill attention in ONE kernel (scores, softmax and context never leave the SM):
 *   s_tj = alpha_qk * float(q_t . k_j),  p_tj = int8(rne(127 * softmax_j(s_tj)))  over j <= t + (S - T),
 *   ctx_t = sat_rne(alpha_pv * float(sum_j p_tj * v_j))
 * for `batch` sequences of T query rows and S >= T keys (S - T of them cached), `heads` heads of head_dim
 * 64 or 128.  Strides in bytes: query row t of sequence b, head h at q + b*q_batch_stride + t*ld_q +
 * h*head_dim; key rows likewise; vt = [batch][heads][head_dim][ld_vt] with the keys contiguous (the
 * transposed value cache); ctx row at ctx + b*ctx_batch_stride + t*ld_ctx + h*head_dim.  All pointers and
 * strides multiples of 16.  No additive mask: callers with padding masks use ti_gemm_i8_ex + ti_softmax_q.
 * Replaces bmm_s8t_s8n_f32t -> mask/softmax/x127/round -> bmm_s8t_s8n_s8t of Int8OPTAttention.forward
 * (torch_int/models/opt.py:131-181).  Rounding: the row sum is accumulated tile by tile, so p may differ
 * from the three-kernel path by one unit on rounding ties. */
int ti_attention_prefill_s8(const int8_t* q, int64_t ld_q, int64_t q_batch_stride, const int8_t* k, int64_t ld_k,
                            int64_t k_batch_stride, const int8_t* vt, int64_t ld_vt, int8_t* ctx, int64_t ld_ctx,
                            int64_t ctx_batch_stride, int64_t batch, int64_t heads, int64_t head_dim, int64_t T,
                            int64_t S, float alpha_qk, float alpha_pv, void* stream);

/* ---- status ---- */

/* Message of the last error raised on the calling thread ("" if none). */
const char* ti_last_error(void);

/* Synchronises the current device and stores the kernel status word in *status:
 * 0 = ok, else the code of the first in-kernel wait that ran into its time
 * limit (the kernels never spin forever).  reset != 0 clears it and, when it was
 * non-zero, also zeroes the built-in split-K scratch of ti_linear_a8_w8_b8_o8_static
 * (a launch that gave up may have left partial sums there).  A workspace the caller
 * passed through ti_gemm_desc.workspace must be zeroed by the caller in that case.
 * Returns TI_OK when the word could be read (whatever its value), TI_E_CUDA otherwise. */
int ti_device_status(int* status, int reset);

/* ti_device_status(&s, reset) as a plain check: TI_OK when the status word was 0, TI_E_DEVICE (with the
 * code in ti_last_error()) when a kernel's bounded wait had given up, TI_E_CUDA on a runtime error. */
int ti_check_device(int reset);

/* ---- tensor-parallel exchange (no reference counterpart: the reference is single-GPU) ---- */

/* For the `rows` rows this rank owns: sums `n_partials` int32 partial-sum slabs
 * (stage[s * partial_stride + row * H + col], written by the ranks' GEMM epilogues through
 * ti_gemm_desc.scatter_ptrs), then residual_out = residual + fma(scale, float(sum), bias) and
 * q = LayerNorm-quantise(residual_out) as ti_dq_add_layernorm_q_bias does, and writes q to row
 * (q_row_offset + row) of each of the n_dst buffers q_dst[i] (peer stores: the all-gather). */
int ti_tp_reduce_layernorm_q(const int32_t* stage, int32_t n_partials, int64_t partial_stride,
                             float scale, const float* bias, const float* residual, const float* gamma,
                             const float* beta, float eps, float* residual_out, void* const* q_dst,
                             int32_t n_dst, int64_t q_row_offset, int64_t rows, int64_t H, void* stream);

/* ti_tp_reduce_layernorm_q with the synchronisation of the exchange folded in, so that one exchange is
 * "copy the partial sums into the owners' stage slabs, then this one kernel".  The kernel (1) tells every
 * rank that this rank's partial sums have arrived (the copies precede it in stream order), (2) waits
 * until all ranks have said so, (3) reduces, normalises and stores the int8 rows into every rank's
 * buffer, and (4) its last CTA tells every rank that this rank is complete and waits for the same from
 * all ranks: when the kernel ends, every rank's rows are in this rank's buffer and every stage may be
 * overwritten.  pads[i] = rank i's pad of 16 zero-initialised 32-bit words in peer-accessible memory
 * (words [0, 8): arrival, [8, 16): completion); epoch must increase by one per call on every rank;
 * counter = one zero-initialised int32 in this GPU's memory, used by this call only while it runs.
 * Waits are bounded by limit_ms (<= 0: 2000; at most 60000); on expiry the status word of
 * ti_device_status is set to 105, no later wait of the process blocks, and the output of that pass is
 * invalid.  No reference counterpart (the reference is single-GPU). */
int ti_tp_exchange_reduce_layernorm_q(const int32_t* stage, int32_t n_partials, int64_t partial_stride,
                                      float scale, const float* bias, const float* residual, const float* gamma,
                                      const float* beta, float eps, float* residual_out, void* const* q_dst,
                                      int32_t n_dst, int64_t q_row_offset, int64_t rows, int64_t H,
                                      void* const* pads, int32_t rank, int32_t n, uint32_t epoch,
                                      int32_t* counter, int64_t limit_ms, void* stream);

/* Stream-ordered barrier over n <= 8 ranks.  pads[i] = rank i's pad (n 32-bit words, zeroed once,
 * peer-accessible); epoch must increase by one per call on every rank.  Peer stores made by earlier
 * work of `stream` are visible to the peers' work enqueued after their matching barrier.  The wait is
 * bounded (2 s); on expiry the status word of ti_device_status is set to 105. */
int ti_tp_barrier(void* const* pads, int32_t rank, int32_t n, uint32_t epoch, void* stream);
/* The same with the time limit of the wait given in milliseconds (<= 0: 2000; at most 60000): the first
 * barriers of a process tolerate the seconds by which ranks may reach them apart while kernels load. */
int ti_tp_barrier_limit(void* const* pads, int32_t rank, int32_t n, uint32_t epoch, int64_t limit_ms,
                        void* stream);

/* Caps the number of SMs the persistent GEMM/BMM grids of this process occupy (0 = all).  For callers
 * that run collectives concurrently with the GEMMs and want the collective's CTAs to find free SMs.
 * No reference counterpart (the reference has no multi-GPU path). */
int ti_set_sm_limit(int sms);

/* Tuning knob: number of M tiles per band of the GEMM tile order (0 = automatic: up to 32 CTA-pair tiles
 * while the band's A rows stay below 32 MB, else 8).  No reference counterpart. */
int ti_set_group_m(int tiles);

/* Small-M GEMMs (M <= 128: decode steps) are launched with programmatic stream serialisation by default:
 * their CTAs may become resident while the kernel before them in the stream drains and fetch their first
 * weight tiles (model constants that no kernel writes); activations, outputs and scratch are touched only after
 * the earlier kernel has completed.  The LayerNorm-quantise kernels on at most 32 rows are launched the same
 * way: they pull gamma, beta and the bias (constants as well) toward L2 and then wait.  A caller that
 * overwrites WEIGHTS or LayerNorm parameters with a kernel on the same stream right before such a call turns
 * this off (on = 0).  No reference counterpart. */
int ti_set_dependent_launch(int on);

/* GEMMs of at most 16 rows (decode steps) stage 16 rows of A per pipeline stage instead of the tile's 128
 * (default on = 1): the shared memory this frees holds more weight tiles in flight.  Results are identical.
 * No reference counterpart. */
int ti_set_narrow_a(int on);

/* ABI version of this header (bumped on incompatible changes). */
int ti_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TORCH_INT_B200_H */
