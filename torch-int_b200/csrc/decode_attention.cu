// One-token (decode step) attention over the int8 key/value cache, one kernel per layer:
//   append the new key row and value column at position *pos,
//   s_j = alpha_qk * float(q . k_j)                      j = 0 .. *pos          (int8 dot products)
//   p_j = int8(rne(127 * softmax(s)_j))
//   ctx = int8(sat_rne(alpha_pv * float(sum_j p_j * v_j)))
// i.e. what bmm_s8t_s8n_f32t -> softmax -> *127 -> round -> bmm_s8t_s8n_s8t compute for a single
// query row (torch_int/models/opt.py:131-181), with the same arithmetic as those ops' kernels.
// The position is read from DEVICE memory, so the launch has no per-step host parameters and a
// whole decode step can be captured in a CUDA graph and replayed.
//
// Layouts (those of the static cache): keys [B, cap, Hl*D] rows; values transposed
// [B, Hl, D, cap]; qkv [B, 3*Hl*D] = the fused projection output of the new token.
// One CTA of 256 threads per (sequence, head); HBM-bound on the cache: (D + D) * (*pos + 1) bytes.
// Key rows are read with one coalesced 128-byte row per 8 lanes and four rows in flight per lane, value
// rows with 512-byte segments per warp and four rows in flight, so that the kernel is bound by
// bandwidth rather than by a chain of dependent loads.
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "gemm_i8.h"
#include "grid_dependency.cuh"
#include "norm_quant.h"

namespace ti {
namespace {

__device__ __forceinline__ int dot16(const uint4& a, const uint4& b, int acc) {
  acc = __dp4a(static_cast<int>(a.x), static_cast<int>(b.x), acc);
  acc = __dp4a(static_cast<int>(a.y), static_cast<int>(b.y), acc);
  acc = __dp4a(static_cast<int>(a.z), static_cast<int>(b.z), acc);
  acc = __dp4a(static_cast<int>(a.w), static_cast<int>(b.w), acc);
  return acc;
}

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int DEC_THREADS = 256;
constexpr int DEC_WARPS = DEC_THREADS / 32;

// Loads a thread keeps in flight in the score loop (key rows) and in the context loop (value rows).  The
// kernel is bound by memory latency: a (sequence, head) pair holds 2 x S x D bytes and every pass over
// them costs one round trip.  Four CTAs must fit an SM (64 registers per thread): batch x heads = 448 CTAs
// of the OPT-30B decode step then run as one wave on 148 SMs.
constexpr int DEC_KEYS_IN_FLIGHT = 8;
constexpr int DEC_VALUE_ROWS_IN_FLIGHT = 8;

template <int D>
__global__ void __launch_bounds__(DEC_THREADS, 4)
decode_attention_s8_kernel(const int8_t* __restrict__ qkv, long long ld_qkv, int8_t* __restrict__ keys,
                           int8_t* __restrict__ values_t, int cap, int hl, const int* __restrict__ pos,
                           float alpha_qk, float alpha_pv, int8_t* __restrict__ ctx, long long ld_ctx,
                           int* status) {
  constexpr int PIECES = D / 16;        // 16-byte pieces of a key row
  constexpr int RPW = 32 / PIECES;      // key rows a warp covers with one load per lane
  extern __shared__ __align__(16) unsigned char dsm[];
  float* s_scores = reinterpret_cast<float*>(dsm);                 // [cap]
  int8_t* s_probs = reinterpret_cast<int8_t*>(dsm + cap * 4);      // [cap] (zero beyond the length)
  __shared__ float red[2 * DEC_WARPS];
  const int b = blockIdx.x / hl, h = blockIdx.x % hl;
  const int el = hl * D;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grid_dep_launch();  // the out_proj GEMM that follows may start fetching its weights now ...
  grid_dep_wait();    // ... and this kernel reads the q/k/v rows the GEMM before it wrote
  const int len = *pos;  // keys/values already cached; the new token goes to position `len`
  if (len < 0 || len >= cap) {
    if (tid == 0) atomicCAS(status, 0, 201);  // cache full: refuse instead of writing out of bounds
    return;
  }
  const int S = len + 1;
  const int8_t* qrow = qkv + b * ld_qkv + h * D;
  int8_t* krows = keys + (static_cast<long long>(b) * cap) * el + h * D;   // row j at + j*el
  int8_t* vrows = values_t + (static_cast<long long>(b) * hl + h) * D * static_cast<long long>(cap);

  // append the new key row (D bytes) and value column (one byte in each of D rows)
  if (tid < PIECES)
    reinterpret_cast<uint4*>(krows + static_cast<long long>(len) * el)[tid] =
        reinterpret_cast<const uint4*>(qrow + el)[tid];
  if (tid < D) vrows[static_cast<long long>(tid) * cap + len] = qrow[2 * el + tid];
  // this lane's 16 bytes of q
  const int piece = lane % PIECES, sub = lane / PIECES;
  const uint4 qp = reinterpret_cast<const uint4*>(qrow)[piece];
  __syncthreads();  // the new key row and value column are visible to the whole CTA

  // ---- scores: PIECES lanes share a key row (one coalesced row per load), KU rows in flight per lane
  constexpr int KU = DEC_KEYS_IN_FLIGHT;
  float mx = -FLT_MAX;
  for (int base = warp * RPW * KU; base < S; base += DEC_WARPS * RPW * KU) {
    uint4 kv[KU];
#pragma unroll
    for (int u = 0; u < KU; ++u) {
      const int j = base + u * RPW + sub;
      kv[u] = j < S ? reinterpret_cast<const uint4*>(krows + static_cast<long long>(j) * el)[piece]
                    : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < KU; ++u) {
      int acc = dot16(qp, kv[u], 0);
#pragma unroll
      for (int o = 1; o < PIECES; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      const int j = base + u * RPW + sub;
      if (piece == 0 && j < S) {
        const float sc = alpha_qk * __int2float_rn(acc);
        s_scores[j] = sc;
        mx = fmaxf(mx, sc);
      }
    }
  }
  mx = warp_max_f(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int w = 1; w < DEC_WARPS; ++w) mx = fmaxf(mx, red[w]);
  float sum = 0.f;
  for (int j = tid; j < S; j += DEC_THREADS) {
    const float e = expf(s_scores[j] - mx);
    s_scores[j] = e;
    sum += e;
  }
  sum = warp_sum_f(sum);
  if (lane == 0) red[DEC_WARPS + warp] = sum;
  __syncthreads();
  sum = ((red[DEC_WARPS] + red[DEC_WARPS + 1]) + (red[DEC_WARPS + 2] + red[DEC_WARPS + 3])) +
        ((red[DEC_WARPS + 4] + red[DEC_WARPS + 5]) + (red[DEC_WARPS + 6] + red[DEC_WARPS + 7]));
  const int s_pad = (S + 15) & ~15;
  for (int j = tid; j < s_pad; j += DEC_THREADS) {
    int p = 0;
    if (j < S) p = max(-128, min(127, __float2int_rn(__fdiv_rn(s_scores[j], sum) * 127.f)));
    s_probs[j] = static_cast<int8_t>(p);
  }
  __syncthreads();

  // ---- context: a warp owns D/8 value rows and takes VU at a time; lanes stride over the
  //      positions 16 bytes at a time (one coalesced 512-byte segment of a row per load)
  constexpr int ROWS = D / DEC_WARPS;
  constexpr int VU = ROWS < DEC_VALUE_ROWS_IN_FLIGHT ? ROWS : DEC_VALUE_ROWS_IN_FLIGHT;
#pragma unroll 1
  for (int dd = 0; dd < ROWS; dd += VU) {
    const int d0 = warp * ROWS + dd;
    int acc[VU];
#pragma unroll
    for (int u = 0; u < VU; ++u) acc[u] = 0;
    for (int j = lane * 16; j < s_pad; j += 512) {
      const uint4 pp = *reinterpret_cast<const uint4*>(s_probs + j);
      uint4 vv[VU];
#pragma unroll
      for (int u = 0; u < VU; ++u)
        vv[u] = *reinterpret_cast<const uint4*>(vrows + static_cast<long long>(d0 + u) * cap + j);
#pragma unroll
      for (int u = 0; u < VU; ++u) acc[u] = dot16(pp, vv[u], acc[u]);
    }
#pragma unroll
    for (int u = 0; u < VU; ++u) acc[u] = warp_sum_i(acc[u]);
    int a = acc[0];
#pragma unroll
    for (int u = 1; u < VU; ++u) a = lane == u ? acc[u] : a;
    if (lane < VU) {
      const int o = max(-128, min(127, __float2int_rn(alpha_pv * __int2float_rn(a))));
      ctx[b * ld_ctx + h * D + d0 + lane] = static_cast<int8_t>(o);
    }
  }
}

__global__ void advance_position_kernel(int* pos, int by) { *pos += by; }

}  // namespace

int decode_attention_s8(const int8_t* qkv, int64_t ld_qkv, int8_t* keys, int8_t* values_t, int64_t batch,
                        int64_t local_heads, int64_t head_dim, int64_t cap, const int* pos, float alpha_qk,
                        float alpha_pv, int8_t* ctx, int64_t ld_ctx, cudaStream_t stream) {
  if (batch < 0 || local_heads <= 0 || cap <= 0 || cap % 16 != 0 || (head_dim != 128 && head_dim != 64)) {
    set_error("decode_attention_s8: head_dim must be 64 or 128 and the cache capacity a positive multiple of 16");
    return TI_E_INVALID;
  }
  if (batch == 0) return TI_OK;
  if (!qkv || !keys || !values_t || !pos || !ctx) {
    set_error("decode_attention_s8: null pointer");
    return TI_E_INVALID;
  }
  const int64_t el = local_heads * head_dim;
  if (ld_qkv < 3 * el || ld_qkv % 16 != 0 || ld_ctx < el ||
      ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(keys) |
        reinterpret_cast<uintptr_t>(values_t)) & 15) != 0) {
    set_error("decode_attention_s8: rows must be 16-byte aligned and hold q, k and v side by side");
    return TI_E_INVALID;
  }
  const size_t smem = static_cast<size_t>(cap) * 5;
  if (smem > 200 * 1024 || batch * local_heads > 0x7FFFFFFF) {
    set_error("decode_attention_s8: cache capacity %lld too large", (long long)cap);
    return TI_E_INVALID;
  }
  int* status = status_word_ptr();
  if (!status) {
    set_error("decode_attention_s8: cannot resolve the device status word");
    return TI_E_CUDA;
  }
  const unsigned grid = static_cast<unsigned>(batch * local_heads);
  cudaError_t e;
  if (head_dim == 128) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(decode_attention_s8_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem));
    decode_attention_s8_kernel<128><<<grid, DEC_THREADS, smem, stream>>>(
        qkv, ld_qkv, keys, values_t, static_cast<int>(cap), static_cast<int>(local_heads), pos, alpha_qk,
        alpha_pv, ctx, ld_ctx, status);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(decode_attention_s8_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem));
    decode_attention_s8_kernel<64><<<grid, DEC_THREADS, smem, stream>>>(
        qkv, ld_qkv, keys, values_t, static_cast<int>(cap), static_cast<int>(local_heads), pos, alpha_qk,
        alpha_pv, ctx, ld_ctx, status);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("decode_attention_s8 launch failed: %s", cudaGetErrorString(e));
    return TI_E_CUDA;
  }
  return TI_OK;
}

int advance_position(int* pos, int by, cudaStream_t stream) {
  if (!pos) {
    set_error("advance_position: null pointer");
    return TI_E_INVALID;
  }
  advance_position_kernel<<<1, 1, 0, stream>>>(pos, by);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("advance_position launch failed: %s", cudaGetErrorString(e));
    return TI_E_CUDA;
  }
  return TI_OK;
}

}  // namespace ti
