// Embedding gather: out[t, :] = table[ids[t], :], written in the type of the
// residual stream (32-bit).  Reference behaviour: src/kernels/embedding.cu:22-38
// of lucciola copies the row unchanged, without scaling; an id outside the
// table reads row 0 there.  Here ids are validated on the host before a step;
// the clamp below only keeps a bad id from reading outside the table.
//
// With a table of learned position vectors the row pos_table[positions[t], :] is added in 32-bit,
// unscaled, for models that encode positions at the input instead of inside attention.
//
// `scale` multiplies the table's row (in 32-bit, before anything is added); `out2`, if given, receives a second copy
// of the result, for models that add the embedding's output to the stream again later.
//
// With a table of frequencies (sin_freq, 64-bit, [ceil(hidden / 2)]) a sinusoidal position vector is added
// instead: entry 2i gets sin(p * sin_freq[i]), entry 2i + 1 the cosine of the same angle.  The angle is formed
// and brought into (-pi, pi] in 64-bit, so that a position in the hundreds of thousands costs no digits; sine and
// cosine of the remainder are 32-bit.
#include "common.cuh"

namespace lb {

template <typename TW>
__global__ void embedding_kernel(float* __restrict__ out, const int* __restrict__ ids,
                                 const TW* __restrict__ table, int hidden, int vocab,
                                 const TW* __restrict__ pos_table, const int* __restrict__ positions, int max_positions,
                                 float scale, float* __restrict__ out2) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const TW* row = table + (size_t)id * hidden;
  float* dst = out + (size_t)t * hidden;
  if (scale != 1.f || out2) {                 // a scaled table row, optionally written twice (one copy stays as it is)
    float* dst2 = out2 ? out2 + (size_t)t * hidden : nullptr;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = to_f32(row[i]) * scale;
      if (pos_table) {
        int p = positions[t];
        if (p < 0 || p >= max_positions) p = 0;
        v += to_f32(pos_table[(size_t)p * hidden + i]);
      }
      dst[i] = v;
      if (dst2) dst2[i] = v;
    }
    return;
  }
  if (pos_table) {
    int p = positions[t];
    if (p < 0 || p >= max_positions) p = 0;
    const TW* prow = pos_table + (size_t)p * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(row[i]) + to_f32(prow[i]);
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(row[i]);
  }
}

template <typename TW>
__global__ void embedding_sinusoid_kernel(float* __restrict__ out, const int* __restrict__ ids, const TW* __restrict__ table,
                                          int hidden, int vocab, const double* __restrict__ sin_freq,
                                          const int* __restrict__ positions) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const TW* row = table + (size_t)id * hidden;
  float* dst = out + (size_t)t * hidden;
  const double pos = (double)positions[t];
  const double two_pi = 6.283185307179586476925286766559;
  for (int i = threadIdx.x; 2 * i < hidden; i += blockDim.x) {
    const double a = pos * sin_freq[i];
    const float r = (float)(a - two_pi * rint(a / two_pi));
    float s, c;
    sincosf(r, &s, &c);
    dst[2 * i] = to_f32(row[2 * i]) + s;
    if (2 * i + 1 < hidden) dst[2 * i + 1] = to_f32(row[2 * i + 1]) + c;
  }
}

}  // namespace lb

// pos_table (same type as table, [max_positions, hidden]) and positions are optional, together; sin_freq
// (with positions, without pos_table) asks for sinusoidal position vectors instead.
LB_EXPORT int lb_embedding(float* out, const int* ids, const void* table, int table_dtype,
                           int num_tokens, int hidden, int vocab, const void* pos_table, const int* positions,
                           int max_positions, const double* sin_freq, float scale, float* out2, cudaStream_t stream) {
  LB_CHECK_ARG(sin_freq == nullptr || (scale == 1.f && out2 == nullptr), "embedding: sinusoidal positions take no scale and no second copy");
  LB_CHECK_ARG(sin_freq == nullptr || (pos_table == nullptr && positions != nullptr),
               "embedding: sinusoidal positions need the positions and exclude a table of position vectors");
  LB_CHECK_ARG(sin_freq != nullptr || ((pos_table == nullptr) == (positions == nullptr) && (pos_table == nullptr || max_positions > 0)),
               "embedding: a position table needs positions and its number of rows");
  LB_CHECK_ARG(lb::valid_dtype(table_dtype), "embedding: bad table dtype %d", table_dtype);
  LB_CHECK_ARG(num_tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes T=%d H=%d V=%d",
               num_tokens, hidden, vocab);
  if (num_tokens == 0) return 0;
  int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
  if (sin_freq) {
    LB_DISPATCH_DTYPE(table_dtype, TW, {
      lb::launch(lb::embedding_sinusoid_kernel<TW>, dim3(num_tokens), dim3(threads), 0, stream, out, ids, (const TW*)table, hidden,
                 vocab, sin_freq, positions);
    })
    LB_CHECK_LAUNCH("embedding");
    return 0;
  }
  LB_DISPATCH_DTYPE(table_dtype, TW, {
    lb::launch(lb::embedding_kernel<TW>, dim3(num_tokens), dim3(threads), 0, stream, out, ids, (const TW*)table, hidden, vocab,
               (const TW*)pos_table, positions, max_positions, scale, out2);
  })
  LB_CHECK_LAUNCH("embedding");
  return 0;
}
