// Bandwidth-bound row kernels of the W8A8 path:
//   layernorm_q         q = int8(clamp(rne(LN(x) * gamma + beta), -128, 127))
//                       (reference: torch_int/nn/fused.py:13-18, four ATen launches)
//   dq_add_layernorm_q  r = residual + scale * int32_in (+ bias); q as above from r
//                       (reference: torch_int/kernels/fused.cu:17-23, five ATen launches)
//   softmax_q           p = int8(rne(127 * softmax(max(s + mask, FLT_LOWEST))))
//                       (reference: torch_int/models/opt.py:139-178)
// One CTA owns one row.  The row is read once with 128-bit loads, kept in
// registers for the two reductions (warp shuffles + one shared-memory step) and
// written once, so HBM traffic equals the algorithmic bytes.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "gemm_i8.h"
#include "grid_dependency.cuh"
#include "norm_quant.h"

namespace ti {
namespace {

constexpr int kMaxVpt = 16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reduction; every thread gets the result.  `scratch` holds one
// float per warp and may be reused right after the call returns.
template <int THREADS, bool kMax>
__device__ __forceinline__ float block_reduce(float v, float* scratch) {
  constexpr int W = THREADS / 32;
  v = kMax ? warp_max(v) : warp_sum(v);
  if constexpr (W == 1) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // scratch may still be read from the previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < W ? scratch[lane] : (kMax ? -FLT_MAX : 0.f);
  return kMax ? warp_max(r) : warp_sum(r);
}

__device__ __forceinline__ int quant_s8(float y) {
  // clamp to [-128,127] then round half to even == RNE then saturate
  int v = __float2int_rn(y);
  return max(-128, min(127, v));
}

__device__ __forceinline__ uint32_t pack_s8x4(float a, float b, float c, float d) {
  return (static_cast<uint32_t>(quant_s8(a)) & 0xFFu) | ((static_cast<uint32_t>(quant_s8(b)) & 0xFFu) << 8) |
         ((static_cast<uint32_t>(quant_s8(c)) & 0xFFu) << 16) |
         ((static_cast<uint32_t>(quant_s8(d)) & 0xFFu) << 24);
}

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__half>(const __half* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __half2 a = *reinterpret_cast<const __half2*>(&u.x);
  const __half2 b = *reinterpret_cast<const __half2*>(&u.y);
  const float2 fa = __half22float2(a), fb = __half22float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store4<__half>(__half* p, float4 v) {
  const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&a);
  u.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// With a 16-bit residual stream the reference rounds every intermediate tensor
// to fp16 (the LayerNorm output is an fp16 tensor before clamp/round).
template <typename T>
__device__ __forceinline__ float round_to_storage(float v) {
  return v;
}
template <>
__device__ __forceinline__ float round_to_storage<__half>(float v) {
  return __half2float(__float2half_rn(v));
}

// Shared tail: LayerNorm statistics over the register-resident row `x`,
// affine transform, quantisation, 4-byte stores.
template <typename T, int THREADS, int VPT>
__device__ __forceinline__ void layernorm_quant_row(float4 (&x)[VPT], int h4, const float* gamma,
                                                    const float* beta, float eps, int H,
                                                    int8_t* qrow, float* scratch) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < h4) s += (x[j].x + x[j].y) + (x[j].z + x[j].w);
  }
  const float mean = block_reduce<THREADS, false>(s, scratch) / static_cast<float>(H);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < h4) {
      const float a = x[j].x - mean, b = x[j].y - mean, c = x[j].z - mean, d = x[j].w - mean;
      ss += (a * a + b * b) + (c * c + d * d);
    }
  }
  const float var = block_reduce<THREADS, false>(ss, scratch) / static_cast<float>(H);
  const float rstd = __fdiv_rn(1.f, __fsqrt_rn(var + eps));
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < h4) {
      const float4 g = *reinterpret_cast<const float4*>(gamma + 4 * i);
      const float4 b = *reinterpret_cast<const float4*>(beta + 4 * i);
      const float y0 = round_to_storage<T>(__fmaf_rn((x[j].x - mean) * rstd, g.x, b.x));
      const float y1 = round_to_storage<T>(__fmaf_rn((x[j].y - mean) * rstd, g.y, b.y));
      const float y2 = round_to_storage<T>(__fmaf_rn((x[j].z - mean) * rstd, g.z, b.z));
      const float y3 = round_to_storage<T>(__fmaf_rn((x[j].w - mean) * rstd, g.w, b.w));
      *reinterpret_cast<uint32_t*>(qrow + 4 * i) = pack_s8x4(y0, y1, y2, y3);
    }
  }
}

// Start of a row kernel inside a chain of dependent launches (decode steps).  The small-M GEMM that follows
// may be scheduled at once and fetch its weights while this kernel runs.  dep != 0: this kernel was itself
// launched as a programmatic dependent of the GEMM before it, so its launch latency overlaps that GEMM's last
// CTAs; it pulls its per-layer parameters (which no kernel writes) toward L2 before it waits for the GEMM.
// Measured on the OPT-30B decode step: 8.02-8.08 ms with dep = 0, 7.84-7.89 ms with dep = 1 (7.96 ms when the
// next GEMM is let go only after the wait).
template <int THREADS>
__device__ __forceinline__ void row_kernel_prologue(int dep, int H, const float* gamma, const float* beta,
                                                    const float* bias) {
  grid_dep_launch();
  if (dep != 0) {
    for (int line = threadIdx.x; line * 32 < H; line += THREADS) {  // 128-byte lines of H floats
      asm volatile("prefetch.global.L2 [%0];" ::"l"(gamma + line * 32));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(beta + line * 32));
      if (bias != nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(bias + line * 32));
    }
  }
  grid_dep_wait();  // this kernel reads the output of the one before it
}

// T: storage type of x.  LN: float = the LayerNorm output stays fp32 (the reference's LayerNormQ with
// fp32 parameters casts x to fp32 first, nn/fused.py:14); __half = it is rounded to fp16 before
// quantising (parameters cast to fp16 as well).
template <typename T, typename LN, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
layernorm_q_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                   const float* __restrict__ beta, float eps, int8_t* __restrict__ q, int H,
                   long long ldx, long long ldq, int dep) {
  __shared__ float scratch[32];
  row_kernel_prologue<THREADS>(dep, H, gamma, beta, nullptr);
  const long long row = blockIdx.x;
  const int h4 = H >> 2;
  const T* xr = x + row * ldx;
  float4 v[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < h4) v[j] = load4<T>(xr + 4 * i);
  }
  layernorm_quant_row<LN, THREADS, VPT>(v, h4, gamma, beta, eps, H, q + row * ldq, scratch);
}

template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
dq_add_layernorm_q_kernel(const int32_t* __restrict__ in, float scale, const T* __restrict__ res,
                          const float* __restrict__ in_bias, const float* __restrict__ gamma,
                          const float* __restrict__ beta, float eps, T* __restrict__ res_out,
                          int8_t* __restrict__ q, int H, int dep) {
  __shared__ float scratch[32];
  row_kernel_prologue<THREADS>(dep, H, gamma, beta, in_bias);
  const long long row = blockIdx.x;
  const int h4 = H >> 2;
  const int32_t* ir = in + row * H;
  const T* rr = res + row * H;
  T* ro = res_out + row * H;
  float4 v[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < h4) {
      const int4 a = *reinterpret_cast<const int4*>(ir + 4 * i);
      const float4 r = load4<T>(rr + 4 * i);
      float4 f = make_float4(round_to_storage<T>(__int2float_rn(a.x)), round_to_storage<T>(__int2float_rn(a.y)),
                             round_to_storage<T>(__int2float_rn(a.z)), round_to_storage<T>(__int2float_rn(a.w)));
      float4 o;
      if (in_bias != nullptr) {
        // The model's residual update with the linear layer folded in: the int32 input is the
        // accumulator of an fp32-output linear (W8A8BFP32OFP32Linear), so d = fma(scale, float(acc),
        // bias) in fp32 exactly as that linear computes it, d is cast to the residual's dtype and
        // added there (models/opt.py:281,289: residual.add_(hidden_states.to(residual.dtype))).
        const float4 bb = *reinterpret_cast<const float4*>(in_bias + 4 * i);
        o.x = r.x + round_to_storage<T>(__fmaf_rn(scale, __int2float_rn(a.x), bb.x));
        o.y = r.y + round_to_storage<T>(__fmaf_rn(scale, __int2float_rn(a.y), bb.y));
        o.z = r.z + round_to_storage<T>(__fmaf_rn(scale, __int2float_rn(a.z), bb.z));
        o.w = r.w + round_to_storage<T>(__fmaf_rn(scale, __int2float_rn(a.w), bb.w));
      } else {
        o.x = __fmaf_rn(scale, f.x, r.x);
        o.y = __fmaf_rn(scale, f.y, r.y);
        o.z = __fmaf_rn(scale, f.z, r.z);
        o.w = __fmaf_rn(scale, f.w, r.w);
      }
      o.x = round_to_storage<T>(o.x);
      o.y = round_to_storage<T>(o.y);
      o.z = round_to_storage<T>(o.z);
      o.w = round_to_storage<T>(o.w);
      store4<T>(ro + 4 * i, o);
      v[j] = o;
    }
  }
  // with a bias this is the model path: the next LayerNormQ has fp32 parameters and normalises in fp32
  if (in_bias != nullptr)
    layernorm_quant_row<float, THREADS, VPT>(v, h4, gamma, beta, eps, H, q + row * static_cast<long long>(H),
                                             scratch);
  else
    layernorm_quant_row<T, THREADS, VPT>(v, h4, gamma, beta, eps, H, q + row * static_cast<long long>(H),
                                         scratch);
}

// Scalar, multi-pass fallback for row lengths the register-resident kernels do
// not cover (H not a multiple of 4, or H > 256 * 4 * kMaxVpt).  Rows are read
// three times; the second and third reads hit L1/L2.
template <typename T, typename LN, bool kDq>
__global__ void __launch_bounds__(256)
layernorm_q_generic_kernel(const T* __restrict__ x, const int32_t* __restrict__ in, float scale,
                           const float* __restrict__ in_bias, const float* __restrict__ gamma,
                           const float* __restrict__ beta, float eps, T* __restrict__ res_out,
                           int8_t* __restrict__ q, int H, long long ldx, long long ldq) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * ldx;
  auto value = [&](int i) -> float {
    float r = static_cast<float>(xr[i]);
    if constexpr (kDq) {
      if (in_bias != nullptr)  // model path: fp32 linear output cast to the residual's dtype, then added
        r = r + round_to_storage<T>(__fmaf_rn(scale, __int2float_rn(in[row * H + i]), in_bias[i]));
      else
        r = __fmaf_rn(scale, round_to_storage<T>(__int2float_rn(in[row * H + i])), r);
      r = round_to_storage<T>(r);
    }
    return r;
  };
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += 256) {
    const float v = value(i);
    if constexpr (kDq) res_out[row * H + i] = static_cast<T>(v);
    s += v;
  }
  const float mean = block_reduce<256, false>(s, scratch) / static_cast<float>(H);
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += 256) {
    const float d = value(i) - mean;
    ss += d * d;
  }
  const float var = block_reduce<256, false>(ss, scratch) / static_cast<float>(H);
  const float rstd = __fdiv_rn(1.f, __fsqrt_rn(var + eps));
  for (int i = threadIdx.x; i < H; i += 256) {
    float y = __fmaf_rn((value(i) - mean) * rstd, gamma[i], beta[i]);
    // the model path (a bias is given) normalises in fp32 like LayerNormQ with fp32 parameters
    y = (kDq && in_bias != nullptr) ? y : round_to_storage<LN>(y);
    q[row * ldq + i] = static_cast<int8_t>(quant_s8(y));
  }
}

// Row softmax of fp32 scores -> int8 probabilities in [0,127].
//   s = score + mask (additive, optional);  s = max(s, -FLT_MAX);  p = softmax(s)
//   out = int8(rne(127 * p))
// `causal` >= 0 generates the additive mask instead of reading one: column j of
// row t (t counted inside its [T,S] matrix) is kept iff j <= t + causal, every
// other column gets -FLT_MAX, which is what the reference's mask tensor holds.
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
softmax_q_kernel(const float* __restrict__ scores, const float* __restrict__ mask,
                 int8_t* __restrict__ out, int T, int S, int heads, long long lds, long long ldo,
                 int causal) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;        // over batch*heads*T
  const int t = static_cast<int>(row % T);
  const long long bh = row / T;
  const float* sr = scores + row * lds;
  const float* mr = mask ? mask + ((bh / heads) * T + t) * static_cast<long long>(S) : nullptr;
  const int s4 = S >> 2;
  float4 v[VPT];
  float mx = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < s4) {
      float4 a = *reinterpret_cast<const float4*>(sr + 4 * i);
      if (mr) {
        const float4 m = *reinterpret_cast<const float4*>(mr + 4 * i);
        a.x += m.x; a.y += m.y; a.z += m.z; a.w += m.w;
      } else if (causal >= 0) {
        const int lim = t + causal;
        if (4 * i + 0 > lim) a.x += -FLT_MAX;
        if (4 * i + 1 > lim) a.y += -FLT_MAX;
        if (4 * i + 2 > lim) a.z += -FLT_MAX;
        if (4 * i + 3 > lim) a.w += -FLT_MAX;
      }
      a.x = fmaxf(a.x, -FLT_MAX); a.y = fmaxf(a.y, -FLT_MAX);
      a.z = fmaxf(a.z, -FLT_MAX); a.w = fmaxf(a.w, -FLT_MAX);
      v[j] = a;
      mx = fmaxf(mx, fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)));
    }
  }
  mx = block_reduce<THREADS, true>(mx, scratch);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < s4) {
      v[j].x = expf(v[j].x - mx); v[j].y = expf(v[j].y - mx);
      v[j].z = expf(v[j].z - mx); v[j].w = expf(v[j].w - mx);
      sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
  }
  sum = block_reduce<THREADS, false>(sum, scratch);
  int8_t* orow = out + row * ldo;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < s4) {
      // softmax = exp / sum (a true division, as torch does), then * 127, RNE.
      const float p0 = __fdiv_rn(v[j].x, sum) * 127.f, p1 = __fdiv_rn(v[j].y, sum) * 127.f;
      const float p2 = __fdiv_rn(v[j].z, sum) * 127.f, p3 = __fdiv_rn(v[j].w, sum) * 127.f;
      *reinterpret_cast<uint32_t*>(orow + 4 * i) = pack_s8x4(p0, p1, p2, p3);
    }
  }
}

// Warp-per-row form of softmax_q for rows of up to 32 * 4 * VPT floats: eight
// rows per CTA, no block-wide barrier, VPT independent 16-byte loads in flight
// per lane.  With a generated causal mask, chunks that lie entirely behind the
// diagonal are not read at all: their probability is exactly zero (the
// reference adds FLT_LOWEST to them, exp() of which underflows to 0).
template <int VPT>
__global__ void __launch_bounds__(256)
softmax_q_warp_kernel(const float* __restrict__ scores, const float* __restrict__ mask,
                      int8_t* __restrict__ out, long long rows, int T, int S, int heads,
                      long long lds, long long ldo, int causal) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int t = static_cast<int>(row % T);
  const long long bh = row / T;
  const float* sr = scores + row * lds;
  const float* mr = mask ? mask + ((bh / heads) * T + t) * static_cast<long long>(S) : nullptr;
  const int s4 = S >> 2;
  const int lim = (mr == nullptr && causal >= 0) ? t + causal : 0x7fffffff;  // last visible column
  float4 v[VPT];
  float mx = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = lane + j * 32;
    if (i < s4 && 4 * i <= lim) {
      float4 a = *reinterpret_cast<const float4*>(sr + 4 * i);
      if (mr) {
        const float4 m = *reinterpret_cast<const float4*>(mr + 4 * i);
        a.x += m.x; a.y += m.y; a.z += m.z; a.w += m.w;
      } else {
        if (4 * i + 1 > lim) a.y += -FLT_MAX;
        if (4 * i + 2 > lim) a.z += -FLT_MAX;
        if (4 * i + 3 > lim) a.w += -FLT_MAX;
      }
      a.x = fmaxf(a.x, -FLT_MAX); a.y = fmaxf(a.y, -FLT_MAX);
      a.z = fmaxf(a.z, -FLT_MAX); a.w = fmaxf(a.w, -FLT_MAX);
      v[j] = a;
      mx = fmaxf(mx, fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)));
    }
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = lane + j * 32;
    if (i < s4 && 4 * i <= lim) {
      v[j].x = expf(v[j].x - mx); v[j].y = expf(v[j].y - mx);
      v[j].z = expf(v[j].z - mx); v[j].w = expf(v[j].w - mx);
      sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
  }
  sum = warp_sum(sum);
  int8_t* orow = out + row * ldo;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = lane + j * 32;
    if (i < s4) {
      uint32_t packed = 0;
      if (4 * i <= lim) {
        const float p0 = __fdiv_rn(v[j].x, sum) * 127.f, p1 = __fdiv_rn(v[j].y, sum) * 127.f;
        const float p2 = __fdiv_rn(v[j].z, sum) * 127.f, p3 = __fdiv_rn(v[j].w, sum) * 127.f;
        packed = pack_s8x4(p0, p1, p2, p3);
      }
      *reinterpret_cast<uint32_t*>(orow + 4 * i) = packed;
    }
  }
}

// Streaming form of the warp-per-row softmax for long rows (more than 32*4*8 floats): the row is
// read three times - maximum, sum of exponentials, probabilities - instead of being kept in
// registers; the second and third reads hit L1/L2 (a row is at most 64 KB), DRAM traffic stays
// one read and one write, and the low register count keeps many warps resident.  Per-lane
// accumulation order and all arithmetic are those of softmax_q_warp_kernel, so both forms give
// identical results.
__global__ void __launch_bounds__(256)
softmax_q_warp_stream_kernel(const float* __restrict__ scores, const float* __restrict__ mask,
                             int8_t* __restrict__ out, long long rows, int T, int S, int heads,
                             long long lds, long long ldo, int causal) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int t = static_cast<int>(row % T);
  const long long bh = row / T;
  const float* sr = scores + row * lds;
  const float* mr = mask ? mask + ((bh / heads) * T + t) * static_cast<long long>(S) : nullptr;
  const int s4 = S >> 2;
  const int lim = (mr == nullptr && causal >= 0) ? t + causal : 0x7fffffff;
  const int n4 = min(s4, lim / 4 + 1);  // chunks that hold at least one visible column
  auto load = [&](int i) -> float4 {
    float4 a = *reinterpret_cast<const float4*>(sr + 4 * i);
    if (mr) {
      const float4 m = *reinterpret_cast<const float4*>(mr + 4 * i);
      a.x += m.x; a.y += m.y; a.z += m.z; a.w += m.w;
    } else {
      if (4 * i + 1 > lim) a.y += -FLT_MAX;
      if (4 * i + 2 > lim) a.z += -FLT_MAX;
      if (4 * i + 3 > lim) a.w += -FLT_MAX;
    }
    a.x = fmaxf(a.x, -FLT_MAX); a.y = fmaxf(a.y, -FLT_MAX);
    a.z = fmaxf(a.z, -FLT_MAX); a.w = fmaxf(a.w, -FLT_MAX);
    return a;
  };
  float mx = -FLT_MAX;
#pragma unroll 4
  for (int i = lane; i < n4; i += 32) {
    const float4 a = load(i);
    mx = fmaxf(mx, fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)));
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll 4
  for (int i = lane; i < n4; i += 32) {
    const float4 a = load(i);
    sum += (expf(a.x - mx) + expf(a.y - mx)) + (expf(a.z - mx) + expf(a.w - mx));
  }
  sum = warp_sum(sum);
  int8_t* orow = out + row * ldo;
#pragma unroll 4
  for (int i = lane; i < s4; i += 32) {
    uint32_t packed = 0;
    if (i < n4) {
      const float4 a = load(i);
      packed = pack_s8x4(__fdiv_rn(expf(a.x - mx), sum) * 127.f, __fdiv_rn(expf(a.y - mx), sum) * 127.f,
                         __fdiv_rn(expf(a.z - mx), sum) * 127.f, __fdiv_rn(expf(a.w - mx), sum) * 127.f);
    }
    *reinterpret_cast<uint32_t*>(orow + 4 * i) = packed;
  }
}

// int8 [B, T, H, D] -> [B, H, D, ld_out] at column offset col0 (the transposed,
// K-major value layout P.V needs).  64 x 64 byte tiles through shared memory,
// 4-byte accesses on both sides.
__global__ void __launch_bounds__(256)
transpose_values_kernel(const int8_t* __restrict__ v, int8_t* __restrict__ vt, int T, int H, int D,
                        long long ld_in, long long ld_out, int col0) {
  __shared__ int8_t tile[64][64 + 4];
  const int t0 = blockIdx.x * 64, d0 = blockIdx.y * 64;
  const int bh = blockIdx.z, b = bh / H, h = bh % H;
  const int8_t* src = v + static_cast<long long>(b) * T * ld_in + h * D;  // row t at + t*ld_in
  // load: 64 rows (t) x 64 bytes (d); thread -> (row = tid/16 + 16*i, 4-byte column = tid%16)
  const int c4 = threadIdx.x & 15, r = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + r + 16 * i;
    uint32_t w = 0;
    if (t < T && d0 + 4 * c4 < D)
      w = *reinterpret_cast<const uint32_t*>(src + static_cast<long long>(t) * ld_in + d0 + 4 * c4);
    *reinterpret_cast<uint32_t*>(&tile[r + 16 * i][4 * c4]) = w;
  }
  __syncthreads();
  // store: 64 rows (d) x 64 bytes (t)
  int8_t* dst = vt + (static_cast<long long>(bh) * D) * ld_out + col0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = r + 16 * i;
    const int tt = 4 * c4;
    if (d0 + d < D) {
      int8_t* p = dst + static_cast<long long>(d0 + d) * ld_out + t0 + tt;
      const int8_t e0 = tile[tt][d], e1 = tile[tt + 1][d], e2 = tile[tt + 2][d], e3 = tile[tt + 3][d];
      if (t0 + tt + 3 < T && ((reinterpret_cast<uintptr_t>(p) & 3) == 0)) {
        *reinterpret_cast<uint32_t*>(p) = (static_cast<uint32_t>(static_cast<uint8_t>(e0))) |
                                          (static_cast<uint32_t>(static_cast<uint8_t>(e1)) << 8) |
                                          (static_cast<uint32_t>(static_cast<uint8_t>(e2)) << 16) |
                                          (static_cast<uint32_t>(static_cast<uint8_t>(e3)) << 24);
      } else {
        if (t0 + tt < T) p[0] = e0;
        if (t0 + tt + 1 < T) p[1] = e1;
        if (t0 + tt + 2 < T) p[2] = e2;
        if (t0 + tt + 3 < T) p[3] = e3;
      }
    }
  }
}

// ---------------------------------------------------------------- tensor parallel
struct PeerPtrs {
  void* p[8];
};

// Synchronisation folded into the reduce kernel (n == 0: none, the caller brackets the kernel with
// tp_barrier launches instead).  Every rank owns a pad of 16 32-bit words per channel in
// peer-accessible memory: word [r] = "rank r's partial sums have arrived in my stage", word [8 + r] =
// "rank r's reduce kernel is complete".  Both carry an epoch that grows by one per exchange.
struct ExchangeSync {
  void* pads[8];   // pads[t] = rank t's pad
  int rank, n;
  uint32_t epoch;
  int* counter;    // CTAs of this launch that have finished; zero between launches
  int* status;     // the library's status word
  unsigned long long limit_ns;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits until *p has reached `epoch` (wrap-around safe).  Bounded: after limit_ns the status word is
// set to 105 and the wait ends; once the status word is non-zero no wait of this process blocks.
__device__ __forceinline__ void wait_epoch_sys(const uint32_t* p, uint32_t epoch, int* status,
                                               unsigned long long limit_ns) {
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  unsigned long long t0 = 0;
  for (unsigned it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    if (static_cast<int>(v - epoch) >= 0) return;
    if ((it & 63) == 63) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        atomicCAS(status, 0, 105);
        return;
      }
    }
  }
}

// Second half of a row-parallel linear under tensor parallelism, for the rows this
// rank owns: `stage` holds one int32 partial-sum slab per rank ([n_partials][rows][H],
// written by the ranks' GEMM epilogues through peer stores).  Per row:
//   acc = sum of the partials (exact integer addition: any order gives the same bits)
//   r   = residual + fma(scale, float(acc), bias)        (the fp32-output linear + residual add)
//   q   = int8(rne(clamp(LayerNorm(r) * gamma + beta)))
// r stays on this rank (the residual stream is sharded by rows); q is written to the
// same row of every rank's activation buffer (q_dst, peer stores): the all-gather.
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
tp_reduce_layernorm_q_kernel(const int32_t* __restrict__ stage, int n_partials, long long partial_stride,
                             float scale, const float* __restrict__ in_bias,
                             const float* __restrict__ res, const float* __restrict__ gamma,
                             const float* __restrict__ beta, float eps, float* __restrict__ res_out,
                             PeerPtrs q_dst, int n_dst, long long q_row_offset, int H, const ExchangeSync sync) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const int h4 = H >> 2;
  if (sync.n > 0) {
    // Arrival: the copies that brought my partial sums into the peers' stages precede this kernel in
    // stream order, so any CTA may announce them; a few CTAs spread over the grid do (the stores are
    // idempotent).  Then every CTA waits until all ranks' partial sums of its rows are in place.
    if (threadIdx.x < sync.n) {
      if ((blockIdx.x & 63) == 0) {
        __threadfence_system();
        st_release_sys(static_cast<uint32_t*>(sync.pads[threadIdx.x]) + sync.rank, sync.epoch);
      }
      wait_epoch_sys(static_cast<const uint32_t*>(sync.pads[sync.rank]) + threadIdx.x, sync.epoch, sync.status,
                     sync.limit_ns);
    }
    __syncthreads();
  }
  float4 v[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < h4) {
      const int32_t* ir = stage + row * H + 4 * i;
      int4 a = __ldcg(reinterpret_cast<const int4*>(ir));
      for (int s = 1; s < n_partials; ++s) {
        const int4 b = __ldcg(reinterpret_cast<const int4*>(ir + s * partial_stride));
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      }
      const float4 r = *reinterpret_cast<const float4*>(res + row * H + 4 * i);
      const float4 bb = *reinterpret_cast<const float4*>(in_bias + 4 * i);
      float4 o;
      o.x = r.x + __fmaf_rn(scale, __int2float_rn(a.x), bb.x);
      o.y = r.y + __fmaf_rn(scale, __int2float_rn(a.y), bb.y);
      o.z = r.z + __fmaf_rn(scale, __int2float_rn(a.z), bb.z);
      o.w = r.w + __fmaf_rn(scale, __int2float_rn(a.w), bb.w);
      *reinterpret_cast<float4*>(res_out + row * H + 4 * i) = o;
      v[j] = o;
    }
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < h4) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  }
  const float mean = block_reduce<THREADS, false>(s, scratch) / static_cast<float>(H);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < h4) {
      const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
      ss += (a * a + b * b) + (c * c + d * d);
    }
  }
  const float var = block_reduce<THREADS, false>(ss, scratch) / static_cast<float>(H);
  const float rstd = __fdiv_rn(1.f, __fsqrt_rn(var + eps));
  const long long qoff = (q_row_offset + row) * H;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < h4) {
      const float4 g = *reinterpret_cast<const float4*>(gamma + 4 * i);
      const float4 b = *reinterpret_cast<const float4*>(beta + 4 * i);
      const uint32_t packed = pack_s8x4(__fmaf_rn((v[j].x - mean) * rstd, g.x, b.x),
                                        __fmaf_rn((v[j].y - mean) * rstd, g.y, b.y),
                                        __fmaf_rn((v[j].z - mean) * rstd, g.z, b.z),
                                        __fmaf_rn((v[j].w - mean) * rstd, g.w, b.w));
      for (int d = 0; d < n_dst; ++d)
        *reinterpret_cast<uint32_t*>(static_cast<int8_t*>(q_dst.p[d]) + qoff + 4 * i) = packed;
    }
  }
  if (sync.n > 0) {
    // Completion: the CTA that finishes last on this rank tells every rank so, then waits until every
    // rank has said the same.  When this kernel ends, all ranks' int8 rows are in this rank's
    // activation buffer and no rank reads its stage any more (the next exchange may overwrite it).
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const int done = atomicAdd(sync.counter, 1);
      if (done == static_cast<int>(gridDim.x) - 1) {
        *sync.counter = 0;
        __threadfence_system();
        for (int t = 0; t < sync.n; ++t)
          st_release_sys(static_cast<uint32_t*>(sync.pads[t]) + 8 + sync.rank, sync.epoch);
        for (int t = 0; t < sync.n; ++t)
          wait_epoch_sys(static_cast<const uint32_t*>(sync.pads[sync.rank]) + 8 + t, sync.epoch, sync.status,
                         sync.limit_ns);
        __threadfence_system();
      }
    }
  }
}

// Barrier over the ranks of a tensor-parallel group, enqueued on a stream.  Every rank
// owns a pad of one 32-bit word per rank in peer-accessible memory.  Thread t signals
// rank t (stores `epoch` into word [rank] of t's pad, system-scope release, after a
// system fence that orders the peer stores of earlier kernels of this stream before it)
// and then waits until rank t's signal for this epoch has arrived in its own pad.  The
// wait is bounded: after `limit_ns` it records an error in *status and returns.
__global__ void tp_barrier_kernel(PeerPtrs pads, int rank, int n, uint32_t epoch, int* status,
                                  unsigned long long limit_ns) {
  const int t = threadIdx.x;
  if (t < n) {
    __threadfence_system();
    uint32_t* theirs = static_cast<uint32_t*>(pads.p[t]) + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    // Once any wait of this process has given up, later barriers still signal (so healthy peers are
    // not held up by us) but no longer wait: a broken exchange then costs one time limit in total,
    // not one per barrier, and the host finds the error in the status word afterwards.
    if (*reinterpret_cast<volatile int*>(status) != 0) return;
    const uint32_t* mine = static_cast<const uint32_t*>(pads.p[rank]) + t;
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int>(v - epoch) >= 0) break;
      if ((it & 63) == 63) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > limit_ns) {
          atomicCAS(status, 0, 105);
          break;
        }
      }
    }
    __threadfence_system();
  }
}

template <typename F>
int check_launch(const char* name, F&& f) {
  f();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s launch failed: %s", name, cudaGetErrorString(e));
    return TI_E_CUDA;
  }
  return TI_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

#define TI_VPT_SWITCH(vpt, ...)                                       \
  switch (vpt) {                                                      \
    case 1: { constexpr int VPT = 1; __VA_ARGS__; break; }            \
    case 2: { constexpr int VPT = 2; __VA_ARGS__; break; }            \
    case 3: { constexpr int VPT = 3; __VA_ARGS__; break; }            \
    case 4: { constexpr int VPT = 4; __VA_ARGS__; break; }            \
    case 5: { constexpr int VPT = 5; __VA_ARGS__; break; }            \
    case 6: { constexpr int VPT = 6; __VA_ARGS__; break; }            \
    case 7: { constexpr int VPT = 7; __VA_ARGS__; break; }            \
    case 8: { constexpr int VPT = 8; __VA_ARGS__; break; }            \
    case 9: case 10: { constexpr int VPT = 10; __VA_ARGS__; break; }  \
    case 11: case 12: { constexpr int VPT = 12; __VA_ARGS__; break; } \
    case 13: case 14: { constexpr int VPT = 14; __VA_ARGS__; break; } \
    default: { constexpr int VPT = 16; __VA_ARGS__; break; }          \
  }

// 1: a row kernel on at most kRowDepMaxRows rows (decode steps) is launched as a programmatic dependent of the
// kernel before it (see row_kernel_prologue).
int g_row_dep_mode = 1;
constexpr int64_t kRowDepMaxRows = 32;

template <typename... KArgs, typename... Args>
void launch_row_kernel(void (*kernel)(KArgs...), unsigned grid, unsigned threads, cudaStream_t stream, bool dependent,
                       Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T, typename LN>
int layernorm_q_typed(const T* x, const float* gamma, const float* beta, float eps, int8_t* q,
                      int64_t rows, int64_t H, cudaStream_t stream) {
  const int h4 = static_cast<int>(H / 4);
  const bool fast = H % 4 == 0 && h4 <= 256 * kMaxVpt && aligned16(x) && aligned16(gamma) &&
                    aligned16(beta) && (reinterpret_cast<uintptr_t>(q) & 3) == 0;
  const unsigned grid = static_cast<unsigned>(rows);
  if (!fast)
    return check_launch("layernorm_q_generic", [&] {
      layernorm_q_generic_kernel<T, LN, false><<<grid, 256, 0, stream>>>(
          x, nullptr, 0.f, nullptr, gamma, beta, eps, nullptr, q, static_cast<int>(H), H, H);
    });
  const int dep = rows <= kRowDepMaxRows ? g_row_dep_mode : 0;
  if (h4 <= 128)
    return check_launch("layernorm_q", [&] {
      launch_row_kernel(layernorm_q_kernel<T, LN, 128, 1>, grid, 128, stream, dep != 0, x, gamma, beta, eps, q,
                        static_cast<int>(H), H, H, dep);
    });
  const int vpt = (h4 + 255) / 256;
  int rc = TI_OK;
  TI_VPT_SWITCH(vpt, rc = check_launch("layernorm_q", [&] {
                  launch_row_kernel(layernorm_q_kernel<T, LN, 256, VPT>, grid, 256, stream, dep != 0, x, gamma, beta,
                                    eps, q, static_cast<int>(H), H, H, dep);
                }));
  return rc;
}

template <typename T>
int dq_add_layernorm_q_typed(const int32_t* in, float scale, const T* res, const float* in_bias,
                             const float* gamma, const float* beta, float eps, T* res_out,
                             int8_t* q, int64_t rows, int64_t H, cudaStream_t stream) {
  const int h4 = static_cast<int>(H / 4);
  const bool fast = H % 4 == 0 && h4 <= 256 * kMaxVpt && aligned16(in) && aligned16(res) &&
                    aligned16(res_out) && aligned16(gamma) && aligned16(beta) &&
                    (in_bias == nullptr || aligned16(in_bias)) &&
                    (reinterpret_cast<uintptr_t>(q) & 3) == 0;
  const unsigned grid = static_cast<unsigned>(rows);
  if (!fast)
    return check_launch("dq_add_layernorm_q_generic", [&] {
      layernorm_q_generic_kernel<T, T, true><<<grid, 256, 0, stream>>>(
          res, in, scale, in_bias, gamma, beta, eps, res_out, q, static_cast<int>(H), H, H);
    });
  const int dep = rows <= kRowDepMaxRows ? g_row_dep_mode : 0;
  if (h4 <= 128)
    return check_launch("dq_add_layernorm_q", [&] {
      launch_row_kernel(dq_add_layernorm_q_kernel<T, 128, 1>, grid, 128, stream, dep != 0, in, scale, res, in_bias,
                        gamma, beta, eps, res_out, q, static_cast<int>(H), dep);
    });
  const int vpt = (h4 + 255) / 256;
  int rc = TI_OK;
  TI_VPT_SWITCH(vpt, rc = check_launch("dq_add_layernorm_q", [&] {
                  launch_row_kernel(dq_add_layernorm_q_kernel<T, 256, VPT>, grid, 256, stream, dep != 0, in, scale, res,
                                    in_bias, gamma, beta, eps, res_out, q, static_cast<int>(H), dep);
                }));
  return rc;
}

}  // namespace

void set_row_dependent_launch(int on) { g_row_dep_mode = on ? 1 : 0; }

int layernorm_q(const void* x, int x_is_half, const float* gamma, const float* beta, float eps,
                int8_t* q, int64_t rows, int64_t H, cudaStream_t stream) {
  if (rows < 0 || H <= 0) {
    set_error("layernorm_q: bad shape rows=%lld H=%lld", (long long)rows, (long long)H);
    return TI_E_INVALID;
  }
  if (rows == 0) return TI_OK;
  if (!x || !gamma || !beta || !q) {
    set_error("layernorm_q: null pointer");
    return TI_E_INVALID;
  }
  if (rows > 0x7FFFFFFF) {
    set_error("layernorm_q: too many rows");
    return TI_E_INVALID;
  }
  if (x_is_half == 2)  // fp16 input, fp32 LayerNorm (LayerNormQ with fp32 parameters)
    return layernorm_q_typed<__half, float>(static_cast<const __half*>(x), gamma, beta, eps, q, rows, H, stream);
  if (x_is_half)
    return layernorm_q_typed<__half, __half>(static_cast<const __half*>(x), gamma, beta, eps, q, rows, H, stream);
  return layernorm_q_typed<float, float>(static_cast<const float*>(x), gamma, beta, eps, q, rows, H, stream);
}

int dq_add_layernorm_q(const int32_t* in, float scale, const void* res, int res_is_half,
                       const float* in_bias, const float* gamma, const float* beta, float eps,
                       void* res_out, int8_t* q, int64_t rows, int64_t H, cudaStream_t stream) {
  if (rows < 0 || H <= 0) {
    set_error("dq_add_layernorm_q: bad shape rows=%lld H=%lld", (long long)rows, (long long)H);
    return TI_E_INVALID;
  }
  if (rows == 0) return TI_OK;
  if (!in || !res || !gamma || !beta || !res_out || !q) {
    set_error("dq_add_layernorm_q: null pointer");
    return TI_E_INVALID;
  }
  if (rows > 0x7FFFFFFF) {
    set_error("dq_add_layernorm_q: too many rows");
    return TI_E_INVALID;
  }
  if (res_is_half)
    return dq_add_layernorm_q_typed<__half>(in, scale, static_cast<const __half*>(res), in_bias, gamma,
                                            beta, eps, static_cast<__half*>(res_out), q, rows, H, stream);
  return dq_add_layernorm_q_typed<float>(in, scale, static_cast<const float*>(res), in_bias, gamma,
                                         beta, eps, static_cast<float*>(res_out), q, rows, H, stream);
}

int softmax_q(const float* scores, const float* mask, int8_t* out, int64_t batch_heads, int64_t heads,
              int64_t T, int64_t S, int64_t lds, int64_t ldo, int causal, cudaStream_t stream) {
  if (batch_heads < 0 || T < 0 || S <= 0 || heads <= 0) {
    set_error("softmax_q: bad shape");
    return TI_E_INVALID;
  }
  const int64_t rows = batch_heads * T;
  if (rows == 0) return TI_OK;
  if (!scores || !out) {
    set_error("softmax_q: null pointer");
    return TI_E_INVALID;
  }
  if (S % 4 != 0 || lds % 4 != 0 || ldo % 4 != 0 || !aligned16(scores) || (mask && !aligned16(mask)) ||
      (reinterpret_cast<uintptr_t>(out) & 3) != 0) {
    set_error("softmax_q: S and the row strides must be multiples of 4 and pointers 16-byte aligned");
    return TI_E_INVALID;
  }
  const int s4 = static_cast<int>(S / 4);
  if (s4 > 256 * kMaxVpt || rows > 0x7FFFFFFF) {
    set_error("softmax_q: S=%lld exceeds the supported maximum of %d", (long long)S, 256 * kMaxVpt * 4);
    return TI_E_INVALID;
  }
  if (s4 <= 32 * 16) {
    const unsigned wgrid = static_cast<unsigned>((rows + 7) / 8);
    const int wv = (s4 + 31) / 32;
    int rc = TI_OK;
#define TI_SOFTMAX_WARP(V)                                                                          \
  rc = check_launch("softmax_q_warp", [&] {                                                         \
    softmax_q_warp_kernel<V><<<wgrid, 256, 0, stream>>>(scores, mask, out, rows, static_cast<int>(T), \
                                                        static_cast<int>(S), static_cast<int>(heads), \
                                                        lds, ldo, causal);                          \
  })
    if (wv <= 1) TI_SOFTMAX_WARP(1);
    else if (wv <= 2) TI_SOFTMAX_WARP(2);
    else if (wv <= 4) TI_SOFTMAX_WARP(4);
    else if (wv <= 8) TI_SOFTMAX_WARP(8);
    else
      rc = check_launch("softmax_q_warp_stream", [&] {
        softmax_q_warp_stream_kernel<<<wgrid, 256, 0, stream>>>(scores, mask, out, rows, static_cast<int>(T),
                                                                static_cast<int>(S), static_cast<int>(heads),
                                                                lds, ldo, causal);
      });
#undef TI_SOFTMAX_WARP
    return rc;
  }
  const unsigned grid = static_cast<unsigned>(rows);
  if (s4 <= 128)
    return check_launch("softmax_q", [&] {
      softmax_q_kernel<128, 1><<<grid, 128, 0, stream>>>(scores, mask, out, static_cast<int>(T),
                                                         static_cast<int>(S), static_cast<int>(heads),
                                                         lds, ldo, causal);
    });
  const int vpt = (s4 + 255) / 256;
  int rc = TI_OK;
  TI_VPT_SWITCH(vpt, rc = check_launch("softmax_q", [&] {
                  softmax_q_kernel<256, VPT><<<grid, 256, 0, stream>>>(
                      scores, mask, out, static_cast<int>(T), static_cast<int>(S),
                      static_cast<int>(heads), lds, ldo, causal);
                }));
  return rc;
}

int tp_reduce_layernorm_q(const int32_t* stage, int n_partials, int64_t partial_stride, float scale,
                          const float* in_bias, const float* res, const float* gamma, const float* beta,
                          float eps, float* res_out, void* const* q_dst, int n_dst, int64_t q_row_offset,
                          int64_t rows, int64_t H, const TpSync* ts, cudaStream_t stream) {
  if (rows < 0 || H <= 0 || n_partials < 1 || n_partials > 8 || n_dst < 1 || n_dst > 8) {
    set_error("tp_reduce_layernorm_q: bad shape");
    return TI_E_INVALID;
  }
  ExchangeSync sync = {};
  if (ts != nullptr) {
    if (ts->n < 1 || ts->n > 8 || ts->rank < 0 || ts->rank >= ts->n || !ts->pads || !ts->counter || !ts->status ||
        rows == 0) {
      set_error("tp_reduce_layernorm_q: bad synchronisation arguments (1..8 ranks, rows > 0)");
      return TI_E_INVALID;
    }
    int64_t limit_ms = ts->limit_ms <= 0 ? 2000 : ts->limit_ms;
    if (limit_ms > 60000) limit_ms = 60000;
    for (int i = 0; i < ts->n; ++i) {
      if (!ts->pads[i] || (reinterpret_cast<uintptr_t>(ts->pads[i]) & 3)) {
        set_error("tp_reduce_layernorm_q: bad pad pointer %d", i);
        return TI_E_INVALID;
      }
      sync.pads[i] = ts->pads[i];
    }
    sync.rank = ts->rank;
    sync.n = ts->n;
    sync.epoch = ts->epoch;
    sync.counter = ts->counter;
    sync.status = ts->status;
    sync.limit_ns = static_cast<unsigned long long>(limit_ms) * 1000000ull;
  }
  if (rows == 0) return TI_OK;
  const int h4 = static_cast<int>(H / 4);
  if (H % 4 != 0 || h4 > 256 * kMaxVpt || rows > 0x7FFFFFFF || partial_stride % 4 != 0 || !stage || !in_bias ||
      !res || !gamma || !beta || !res_out || !q_dst || !aligned16(stage) || !aligned16(in_bias) || !aligned16(res) ||
      !aligned16(gamma) || !aligned16(beta) || !aligned16(res_out)) {
    set_error("tp_reduce_layernorm_q: H must be a multiple of 4 and at most %d, pointers 16-byte aligned",
              256 * kMaxVpt * 4);
    return TI_E_INVALID;
  }
  PeerPtrs dst;
  for (int i = 0; i < 8; ++i) {
    dst.p[i] = i < n_dst ? q_dst[i] : nullptr;
    if (i < n_dst && (!q_dst[i] || (reinterpret_cast<uintptr_t>(q_dst[i]) & 3))) {
      set_error("tp_reduce_layernorm_q: bad destination pointer %d", i);
      return TI_E_INVALID;
    }
  }
  const unsigned grid = static_cast<unsigned>(rows);
  if (h4 <= 128)
    return check_launch("tp_reduce_layernorm_q", [&] {
      tp_reduce_layernorm_q_kernel<128, 1><<<grid, 128, 0, stream>>>(
          stage, n_partials, partial_stride, scale, in_bias, res, gamma, beta, eps, res_out, dst, n_dst,
          q_row_offset, static_cast<int>(H), sync);
    });
  const int vpt = (h4 + 255) / 256;
  int rc = TI_OK;
  TI_VPT_SWITCH(vpt, rc = check_launch("tp_reduce_layernorm_q", [&] {
                  tp_reduce_layernorm_q_kernel<256, VPT><<<grid, 256, 0, stream>>>(
                      stage, n_partials, partial_stride, scale, in_bias, res, gamma, beta, eps, res_out, dst,
                      n_dst, q_row_offset, static_cast<int>(H), sync);
                }));
  return rc;
}

int tp_barrier(void* const* pads, int rank, int n, uint32_t epoch, int* status_word, int64_t limit_ms,
               cudaStream_t stream) {
  if (limit_ms <= 0) limit_ms = 2000;
  if (limit_ms > 60000) limit_ms = 60000;  // never more than a minute: a wait must not look like a hang
  if (n < 1 || n > 8 || rank < 0 || rank >= n || !pads || !status_word) {
    set_error("tp_barrier: bad arguments");
    return TI_E_INVALID;
  }
  PeerPtrs p;
  for (int i = 0; i < 8; ++i) {
    p.p[i] = i < n ? pads[i] : nullptr;
    if (i < n && !pads[i]) {
      set_error("tp_barrier: null pad pointer");
      return TI_E_INVALID;
    }
  }
  return check_launch("tp_barrier", [&] {
    tp_barrier_kernel<<<1, 32, 0, stream>>>(p, rank, n, epoch, status_word,
                                            static_cast<unsigned long long>(limit_ms) * 1000000ull);
  });
}

int transpose_values(const int8_t* v, int8_t* vt, int64_t B, int64_t T, int64_t H, int64_t D,
                     int64_t ld_in, int64_t ld_out, int64_t col0, cudaStream_t stream) {
  if (B < 0 || T < 0 || H <= 0 || D <= 0 || ld_out < col0 + T || col0 < 0 || ld_in < H * D || ld_in % 4 != 0) {
    set_error("transpose_values: bad shape");
    return TI_E_INVALID;
  }
  if (B == 0 || T == 0) return TI_OK;
  if (!v || !vt) {
    set_error("transpose_values: null pointer");
    return TI_E_INVALID;
  }
  if (D % 4 != 0 || (reinterpret_cast<uintptr_t>(v) & 3) != 0 || B * H > 65535) {
    set_error("transpose_values: head_dim must be a multiple of 4, the input 4-byte aligned and "
              "batch*heads <= 65535");
    return TI_E_INVALID;
  }
  dim3 grid(static_cast<unsigned>((T + 63) / 64), static_cast<unsigned>((D + 63) / 64),
            static_cast<unsigned>(B * H));
  return check_launch("transpose_values", [&] {
    transpose_values_kernel<<<grid, 256, 0, stream>>>(v, vt, static_cast<int>(T), static_cast<int>(H),
                                                      static_cast<int>(D), ld_in, ld_out,
                                                      static_cast<int>(col0));
  });
}

}  // namespace ti
