// A short causal convolution over time on each channel of 32-bit rows, with an optional bias and silu:
//
//   out_t = act( b + sum_{j < taps} w[j, :] * x_(t - taps + 1 + j) )        (zeros before the sequence's start)
//
// for the tokens of a step, which are portions of several sequences.  Unlike causal_taps.cu the input is not added
// to the result, and input and output are 32-bit rows that may be column ranges of wider matrices (a product's
// 32-bit output goes in, what a recurrence reads comes out).  What lies before a portion comes from the sequence's
// state: the last taps - 1 inputs, oldest first, [slots + 1, taps - 1, channels] in 32-bit, zero for a new sequence.
// lb_short_conv reads the state; lb_short_conv_state, launched after it, replaces the state by the last taps - 1
// inputs of (state ++ portion).  The weight comes transposed, [taps, channels], oldest tap first.  A token's sum
// visits the taps in one order whatever the portion, so a result does not depend on how a sequence is cut.
#include "common.cuh"

namespace lb {

__device__ __forceinline__ float silu_exact(float x) { return x / (1.f + expf(-x)); }

__global__ void short_conv_kernel(float* __restrict__ out, long long out_ld, const float* __restrict__ x, long long x_ld,
                                  const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state,
                                  const int* __restrict__ token_seq, const int* __restrict__ cu_tokens,
                                  const int* __restrict__ slots, int channels, int taps, int act) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  const int idx = t - cu_tokens[s];                       // place of the token in its portion
  const float* st = state + (size_t)slots[s] * (taps - 1) * channels;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {                      // the input taps - 1 - j tokens back
      const int back = taps - 1 - j;
      const float v = idx - back >= 0 ? x[(size_t)(t - back) * x_ld + c] : st[(size_t)(taps - 1 + idx - back) * channels + c];
      acc = fmaf(w[(size_t)j * channels + c], v, acc);
    }
    if (bias) acc += bias[c];
    out[(size_t)t * out_ld + c] = act ? silu_exact(acc) : acc;
  }
}

// The same with four channels a thread (16-byte words), for rows whose sizes and addresses allow it.  Two tokens a CTA
// would read each input once more from L2 instead of twice; the taps' order within a token's sum is the same.
__global__ void short_conv_x4_kernel(float* __restrict__ out, long long out_ld, const float* __restrict__ x, long long x_ld,
                                     const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state,
                                     const int* __restrict__ token_seq, const int* __restrict__ cu_tokens,
                                     const int* __restrict__ slots, int channels, int taps, int act) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  const int idx = t - cu_tokens[s];
  const float* st = state + (size_t)slots[s] * (taps - 1) * channels;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < channels; c += gridDim.y * blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      const float4 v = *reinterpret_cast<const float4*>(idx - back >= 0 ? x + (size_t)(t - back) * x_ld + c
                                                                         : st + (size_t)(taps - 1 + idx - back) * channels + c);
      const float4 f = *reinterpret_cast<const float4*>(w + (size_t)j * channels + c);
      acc.x = fmaf(f.x, v.x, acc.x); acc.y = fmaf(f.y, v.y, acc.y); acc.z = fmaf(f.z, v.z, acc.z); acc.w = fmaf(f.w, v.w, acc.w);
    }
    if (bias) {
      const float4 b = *reinterpret_cast<const float4*>(bias + c);
      acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
    }
    if (act) { acc.x = silu_exact(acc.x); acc.y = silu_exact(acc.y); acc.z = silu_exact(acc.z); acc.w = silu_exact(acc.w); }
    *reinterpret_cast<float4*>(out + (size_t)t * out_ld + c) = acc;
  }
}

__global__ void short_conv_state_kernel(float* __restrict__ state, const float* __restrict__ x, long long x_ld,
                                        const int* __restrict__ cu_tokens, const int* __restrict__ slots, int channels, int taps) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x;
  const int first = cu_tokens[s], n = cu_tokens[s + 1] - first;
  float* st = state + (size_t)slots[s] * (taps - 1) * channels;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    // entry i of the new state is element n - (taps - 1) + i of the portion, or, where that lies before the
    // portion, entry i + n of the old state; i ascends, so an old entry is read before it is overwritten
    for (int i = 0; i < taps - 1; ++i) {
      const int m = n - (taps - 1) + i;
      st[(size_t)i * channels + c] = m >= 0 ? x[(size_t)(first + m) * x_ld + c] : st[(size_t)(i + n) * channels + c];
    }
  }
}

}  // namespace lb

LB_EXPORT int lb_short_conv(float* out, long long out_ld, const float* x, long long x_ld, const float* w, const float* bias,
                            const float* state, const int* token_seq, const int* cu_tokens, const int* slots, int num_tokens,
                            int channels, int taps, int act, cudaStream_t stream) {
  LB_CHECK_ARG(num_tokens >= 0 && channels > 0 && taps >= 1 && taps <= 16, "short_conv: bad sizes T=%d channels=%d taps=%d",
               num_tokens, channels, taps);
  LB_CHECK_ARG(out && x && w && token_seq && cu_tokens && slots && (taps == 1 || state), "short_conv: null argument");
  LB_CHECK_ARG(out != x, "short_conv: the output must not be the input (a token reads the inputs before it)");
  if (num_tokens == 0) return 0;
  auto a16 = [](const void* q) { return (uintptr_t)q % 16 == 0; };
  if (channels % 4 == 0 && out_ld % 4 == 0 && x_ld % 4 == 0 && a16(out) && a16(x) && a16(w) && a16(bias) && a16(state)) {
    const int threads4 = channels >= 1024 ? 256 : 64;
    int by4 = (channels / 4 + threads4 - 1) / threads4;
    if (by4 > 64) by4 = 64;
    lb::launch(lb::short_conv_x4_kernel, dim3(num_tokens, by4), dim3(threads4), 0, stream, out, out_ld, x, x_ld, w, bias, state,
               token_seq, cu_tokens, slots, channels, taps, act);
    LB_CHECK_LAUNCH("short_conv");
    return 0;
  }
  const int threads = channels >= 256 ? 256 : 64;
  int by = (channels + threads - 1) / threads;
  if (by > 64) by = 64;
  lb::launch(lb::short_conv_kernel, dim3(num_tokens, by), dim3(threads), 0, stream, out, out_ld, x, x_ld, w, bias, state, token_seq,
             cu_tokens, slots, channels, taps, act);
  LB_CHECK_LAUNCH("short_conv");
  return 0;
}

LB_EXPORT int lb_short_conv_state(float* state, const float* x, long long x_ld, const int* cu_tokens, const int* slots,
                                  int num_seqs, int channels, int taps, cudaStream_t stream) {
  LB_CHECK_ARG(num_seqs >= 0 && channels > 0 && taps >= 2 && taps <= 16, "short_conv_state: bad sizes");
  LB_CHECK_ARG(state && x && cu_tokens && slots, "short_conv_state: null argument");
  if (num_seqs == 0) return 0;
  const int threads = channels >= 256 ? 256 : 64;
  int by = (channels + threads - 1) / threads;
  if (by > 64) by = 64;
  lb::launch(lb::short_conv_state_kernel, dim3(num_seqs, by), dim3(threads), 0, stream, state, x, x_ld, cu_tokens, slots, channels, taps);
  LB_CHECK_LAUNCH("short_conv_state");
  return 0;
}
