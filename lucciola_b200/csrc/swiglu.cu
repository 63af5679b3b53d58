// SwiGLU: out = silu(gate) * up with silu(x) = x / (1 + exp(-x)), computed in
// 32-bit and rounded once (src/kernels/swiglu.cu:8,30-36 of lucciola).  gate
// and up are two column ranges of one matrix row (the fused gate|up product)
// or two separate matrices; `in_stride` is the distance between their rows.
// `act` chooses the activation of the gate: 0 silu, 1 relu (out = max(gate, 0) * up), 2 the tanh form of gelu,
// 3 a clamped swish with a shifted linear part: g' = min(gate, limit), u' = clamp(up, -limit, limit),
// out = g' * sigmoid(1.702 g') * (u' + 1).
#include "common.cuh"

namespace lb {

__device__ __forceinline__ float gated_act(int act, float limit, float g, float u) {
  if (act == 1) return fmaxf(g, 0.f) * u;
  if (act == 2) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  if (act == 3) {
    g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
  }
  return g / (1.f + expf(-g)) * u;
}

template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gate,
                              const T* __restrict__ up, long long in_stride, int inter,
                              long long total, int act, float limit) {
  pdl_trigger();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / inter;
    const int c = (int)(idx - t * inter);
    const float g = to_f32(gate[t * in_stride + c]);
    const float u = to_f32(up[t * in_stride + c]);
    out[idx] = from_f32<T>(gated_act(act, limit, g, u));
  }
}

// Eight bfloat16 values a thread (16-byte accesses).
__global__ void swiglu_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gate,
                                     const bf16* __restrict__ up, long long in_stride, int inter,
                                     long long total8, int act, float limit) {
  pdl_trigger();
  pdl_wait();
  const int per_row = inter >> 3;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total8;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / per_row;
    const int c = (int)(idx - t * per_row) << 3;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gate + t * in_stride + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(up + t * in_stride + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 g = __bfloat1622float2(g2[i]);
      const float2 u = __bfloat1622float2(u2[i]);
      o2[i] = act == 0 ? __floats2bfloat162_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y)
                       : __floats2bfloat162_rn(gated_act(act, limit, g.x, u.x), gated_act(act, limit, g.y, u.y));
    }
    *reinterpret_cast<uint4*>(out + t * inter + c) = o4;
  }
}

}  // namespace lb

LB_EXPORT int lb_swiglu(int dtype, void* out, const void* gate, const void* up, long long in_stride,
                        int num_tokens, int inter, int act, float limit, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype), "swiglu: bad dtype %d", dtype);
  LB_CHECK_ARG(num_tokens >= 0 && inter > 0 && in_stride >= inter, "swiglu: bad sizes");
  LB_CHECK_ARG(act >= 0 && act <= 3, "swiglu: activation %d is none of silu (0), relu (1), gelu_tanh (2), clamped swish (3)", act);
  if (num_tokens == 0) return 0;
  const long long total = (long long)num_tokens * inter;
  const bool vec = dtype == LB_BF16 && inter % 8 == 0 && in_stride % 8 == 0 &&
                   ((uintptr_t)gate % 16 == 0) && ((uintptr_t)up % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (vec) {
    const long long total8 = total >> 3;
    const int blocks = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
    lb::launch(lb::swiglu_bf16x8_kernel, dim3(blocks), dim3(256), 0, stream, (lb::bf16*)out, (const lb::bf16*)gate,
               (const lb::bf16*)up, in_stride, inter, total8, act, limit);
  } else {
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    LB_DISPATCH_DTYPE(dtype, T, {
      lb::launch(lb::swiglu_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)out, (const T*)gate, (const T*)up,
                 in_stride, inter, total, act, limit);
    })
  }
  LB_CHECK_LAUNCH("swiglu");
  return 0;
}

// Activations of a feed-forward without a gate, out = act(x), computed in 32-bit and rounded once.  `act`:
// 0 silu, 1 relu, 2 the tanh form of gelu, 5 the square of relu, 4 xIELU with its two positive numbers a_p, a_n (p0, p1):
//   x > 0: a_p x^2 + x / 2        x <= 0: a_n (exp(x) - 1 - x) + x / 2
// (the design's learned numbers p, q enter as a_p = softplus(p), a_n = 1/2 + softplus(q), formed once on the host).
namespace lb {

__device__ __forceinline__ float plain_act(int act, float p0, float p1, float x) {
  if (act == 4) return x > 0.f ? fmaf(p0 * x, x, 0.5f * x) : fmaf(p1, expm1f(x) - x, 0.5f * x);
  if (act == 5) { const float r = fmaxf(x, 0.f); return r * r; }
  return gated_act(act, 0.f, x, 1.f);
}

template <typename T>
__global__ void activation_kernel(T* __restrict__ out, const T* __restrict__ x, long long in_stride, int n, long long total,
                                  int act, float p0, float p1) {
  pdl_trigger();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / n;
    const int c = (int)(idx - t * n);
    out[idx] = from_f32<T>(plain_act(act, p0, p1, to_f32(x[t * in_stride + c])));
  }
}

// bfloat16 rows whose sizes and addresses allow it: eight entries a thread as one 16-byte word in and one out
__global__ void activation_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ x, long long in_stride, int n8,
                                         long long total8, int act, float p0, float p1) {
  pdl_trigger();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / n8;
    const int c = (int)(idx - t * n8) * 8;
    const uint4 in = *reinterpret_cast<const uint4*>(x + t * in_stride + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&in);
    uint4 res;
    __nv_bfloat162* r = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      r[j] = __floats2bfloat162_rn(plain_act(act, p0, p1, f.x), plain_act(act, p0, p1, f.y));
    }
    *reinterpret_cast<uint4*>(out + t * (long long)n8 * 8 + c) = res;
  }
}

}  // namespace lb

LB_EXPORT int lb_activation(int dtype, void* out, const void* x, long long in_stride, int num_tokens, int n, int act, float p0,
                            float p1, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype), "activation: bad dtype %d", dtype);
  LB_CHECK_ARG(out && x && num_tokens >= 0 && n > 0 && in_stride >= n, "activation: bad sizes");
  LB_CHECK_ARG(act == 0 || act == 1 || act == 2 || act == 4 || act == 5,
               "activation: %d is none of silu (0), relu (1), gelu_tanh (2), xielu (4), relu squared (5)", act);
  if (num_tokens == 0) return 0;
  const long long total = (long long)num_tokens * n;
  if (dtype == LB_BF16 && n % 8 == 0 && in_stride % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    const long long total8 = total >> 3;
    const int blocks8 = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
    lb::launch(lb::activation_bf16x8_kernel, dim3(blocks8), dim3(256), 0, stream, (lb::bf16*)out, (const lb::bf16*)x, in_stride, n / 8,
               total8, act, p0, p1);
    LB_CHECK_LAUNCH("activation");
    return 0;
  }
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  LB_DISPATCH_DTYPE(dtype, T, {
    lb::launch(lb::activation_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)out, (const T*)x, in_stride, n, total, act, p0, p1);
  })
  LB_CHECK_LAUNCH("activation");
  return 0;
}

// out[t, :n] = x[t, :n] (32-bit rows that may be a column range of a wider matrix) rounded to out's type, out rows
// contiguous: what a product with 32-bit output left, as the input of a second product.
namespace lb {
template <typename TO>
__global__ void round_cols_kernel(TO* __restrict__ out, const float* __restrict__ x, long long x_ld, int n, long long total) {
  pdl_trigger();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / n;
    out[idx] = from_f32<TO>(x[t * x_ld + (idx - t * n)]);
  }
}
}  // namespace lb

LB_EXPORT int lb_round_cols(void* out, int out_dtype, const float* x, long long x_ld, int num_rows, int n, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && out && x && num_rows >= 0 && n > 0 && x_ld >= n, "round_cols: bad arguments");
  if (num_rows == 0) return 0;
  const long long total = (long long)num_rows * n;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  LB_DISPATCH_DTYPE(out_dtype, TO, {
    lb::launch(lb::round_cols_kernel<TO>, dim3(blocks), dim3(256), 0, stream, (TO*)out, x, x_ld, n, total);
  })
  LB_CHECK_LAUNCH("round_cols");
  return 0;
}
