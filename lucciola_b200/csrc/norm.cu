// Residual add fused with RMSNorm.
//
//   v      = residual[src] + delta[src]          (delta optional)
//   residual[src] = v                            (only when rows == nullptr)
//   out[i] = v * rsqrt(mean(v^2) + eps) * weight
//
// with src = rows ? rows[i] : i.  The residual stream and the norm weight are
// 32-bit; the statistics, the normalisation and the product with the weight
// are computed in 32-bit and rounded once, as src/kernels/rmsnorm.cu:57-97 of
// lucciola does (weight multiplied inside the single rounding, no 1+w).  The
// reference runs add (src/kernels/add.cu:11-14), a copy and the norm as three
// launches; this is one pass over the row.
#include "common.cuh"

namespace lb {

template <typename TD, typename TO, int VEC>
__global__ void add_rmsnorm_kernel(TO* __restrict__ out, float* __restrict__ residual,
                                   const TD* __restrict__ delta, const float* __restrict__ weight,
                                   const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int src = rows ? rows[i] : i;
  float* r = residual + (size_t)src * hidden;
  const TD* d = delta ? delta + (size_t)src * hidden : nullptr;
  TO* o = out + (size_t)i * hidden;
  const bool update = (rows == nullptr) && (delta != nullptr);

  float ss = 0.f;
  if (VEC == 4) {
    const int n4 = hidden >> 2;
    for (int j = threadIdx.x; j < n4; j += blockDim.x) {
      float4 v = reinterpret_cast<const float4*>(r)[j];
      if (d) {
        v.x += to_f32(d[4 * j + 0]); v.y += to_f32(d[4 * j + 1]);
        v.z += to_f32(d[4 * j + 2]); v.w += to_f32(d[4 * j + 3]);
        if (update) reinterpret_cast<float4*>(r)[j] = v;
      }
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
      float v = r[j];
      if (d) { v += to_f32(d[j]); if (update) r[j] = v; }
      ss += v * v;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  // Second pass: the row is in L1/L2.  When the residual was not updated the
  // sum has to be formed again.
  const bool readd = d && !update;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
    float v = r[j];
    if (readd) v += to_f32(d[j]);
    o[j] = from_f32<TO>(v * inv * weight[j]);
  }
}

// Four consecutive elements as one access.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}

// The same for rows that fit the CTA's registers (hidden = PER * threads, PER a multiple of 4): one pass.  Every
// load of a thread is issued before any is used, the norm weights even before the kernel ahead has finished (they do
// not depend on it); the row is read once, kept in registers across the sum, and written with 8- or 16-byte stores.
template <typename TD, typename TO, int PER>
__global__ void add_rmsnorm_row_kernel(TO* __restrict__ out, float* __restrict__ residual, const TD* __restrict__ delta,
                                       const float* __restrict__ weight, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  const int tid = threadIdx.x, nt = blockDim.x;
  float4 w[PER / 4], v[PER / 4];
#pragma unroll
  for (int q = 0; q < PER / 4; ++q) w[q] = load4(weight + 4 * (q * nt + tid));
  pdl_wait();
  const int i = blockIdx.x;
  const int src = rows ? rows[i] : i;
  float* r = residual + (size_t)src * hidden;
  const bool update = (rows == nullptr) && (delta != nullptr);
#pragma unroll
  for (int q = 0; q < PER / 4; ++q) v[q] = load4(r + 4 * (q * nt + tid));
  if (delta) {
    const TD* d = delta + (size_t)src * hidden;
    float4 dv[PER / 4];
#pragma unroll
    for (int q = 0; q < PER / 4; ++q) dv[q] = load4(d + 4 * (q * nt + tid));
#pragma unroll
    for (int q = 0; q < PER / 4; ++q) { v[q].x += dv[q].x; v[q].y += dv[q].y; v[q].z += dv[q].z; v[q].w += dv[q].w; }
  }
  float ss = 0.f;
#pragma unroll
  for (int q = 0; q < PER / 4; ++q) {
    if (update) store4(r + 4 * (q * nt + tid), v[q]);
    ss += v[q].x * v[q].x + v[q].y * v[q].y + v[q].z * v[q].z + v[q].w * v[q].w;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TO* o = out + (size_t)i * hidden;
#pragma unroll
  for (int q = 0; q < PER / 4; ++q)
    store4(o + 4 * (q * nt + tid), make_float4(v[q].x * inv * w[q].x, v[q].y * inv * w[q].y, v[q].z * inv * w[q].z, v[q].w * inv * w[q].w));
}

// Short rows without a delta (the heads of a mixer's output, one row a head): a warp a row, eight rows a CTA.
template <typename TO>
__global__ void rmsnorm_short_rows_kernel(TO* __restrict__ out, const float* __restrict__ x, const float* __restrict__ weight,
                                          int num_rows, int hidden, float eps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= num_rows) return;
  const float* r = x + (size_t)row * hidden;
  float ss = 0.f;
  for (int j = lane; j < hidden; j += 32) { const float v = r[j]; ss += v * v; }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TO* o = out + (size_t)row * hidden;
  for (int j = lane; j < hidden; j += 32) o[j] = from_f32<TO>(r[j] * inv * weight[j]);
}

// RMSNorm in groups: the row is cut into `groups` equal consecutive parts and each part is divided by its own
// sqrt(mean(part^2) + eps); the whole is multiplied by the weight.  Up to two deltas are added to the residual
// stream first (in 32-bit, a then b), for blocks whose sublayers run side by side and leave their outputs unsummed.
// A group is walked by `wpg` warps; the partial sums of a group's warps are added in warp order, so a row's result
// does not depend on the batch.  The row is read from global memory for the sums and again (from cache) for the output.
template <typename TD, typename TO, int EPL>
__global__ void add_group_rmsnorm_kernel(TO* __restrict__ out, float* __restrict__ residual, const TD* __restrict__ delta_a,
                                         const TD* __restrict__ delta_b, const float* __restrict__ weight,
                                         const int* __restrict__ rows, int hidden, int groups, int wpg, float eps) {
  // EPL > 0: a lane has at most EPL elements of a group and keeps them in registers between the sum and the output
  // (all loads issued before any is used); EPL == 0: any size, the row is read again (from cache) for the output.
  __shared__ float part[32];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int src = rows ? rows[i] : i;
  float* r = residual + (size_t)src * hidden;
  const TD* da = delta_a ? delta_a + (size_t)src * hidden : nullptr;
  const TD* db = delta_b ? delta_b + (size_t)src * hidden : nullptr;
  TO* o = out + (size_t)i * hidden;
  const bool update = (rows == nullptr) && (da != nullptr || db != nullptr);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gsize = hidden / groups;
  const int per_round = nwarps / wpg;                 // groups worked on at a time
  const int seg = warp % wpg;
  constexpr int NV = EPL > 0 ? EPL : 1;
  for (int g0 = 0; g0 < groups; g0 += per_round) {
    const int g = g0 + warp / wpg;
    float ss = 0.f;
    float v[NV];
    if (g < groups) {
      if (EPL > 0) {
        float x[NV], ya[NV], yb[NV];
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          const int j = seg * 32 + lane + k * wpg * 32, c = g * gsize + j;
          const bool in = j < gsize;
          x[k] = in ? r[c] : 0.f;
          ya[k] = (in && da) ? to_f32(da[c]) : 0.f;
          yb[k] = (in && db) ? to_f32(db[c]) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          const int j = seg * 32 + lane + k * wpg * 32, c = g * gsize + j;
          float t = x[k];
          if (da) t += ya[k];
          if (db) t += yb[k];
          v[k] = t;
          if (update && j < gsize) r[c] = t;
          ss += t * t;
        }
      } else {
        for (int j = seg * 32 + lane; j < gsize; j += wpg * 32) {
          const int c = g * gsize + j;
          float t = r[c];
          if (da) t += to_f32(da[c]);
          if (db) t += to_f32(db[c]);
          if (update) r[c] = t;
          ss += t * t;
        }
      }
    }
    ss = warp_sum(ss);
    __syncthreads();                                  // `part` may still be read by the groups handled just before
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    if (g < groups) {
      float tot = 0.f;
      for (int k = 0; k < wpg; ++k) tot += part[(warp / wpg) * wpg + k];
      const float inv = 1.f / sqrtf(tot / (float)gsize + eps);
      if (EPL > 0) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          const int j = seg * 32 + lane + k * wpg * 32, c = g * gsize + j;
          if (j < gsize) o[c] = from_f32<TO>(v[k] * inv * weight[c]);
        }
      } else {
        for (int j = seg * 32 + lane; j < gsize; j += wpg * 32) {
          const int c = g * gsize + j;
          float t = r[c];                             // own earlier write, or the untouched row
          if (!update) {
            if (da) t += to_f32(da[c]);
            if (db) t += to_f32(db[c]);
          }
          o[c] = from_f32<TO>(t * inv * weight[c]);
        }
      }
    }
  }
}

}  // namespace lb

// out = group RMSNorm of (residual [+ delta_a] [+ delta_b]); the sum is written back to the residual stream when
// rows == nullptr.  hidden must be a multiple of groups.
LB_EXPORT int lb_add_group_rmsnorm(void* out, int out_dtype, float* residual, const void* delta_a, const void* delta_b,
                                   int delta_dtype, const float* weight, const int* rows, int num_rows, int hidden,
                                   int groups, float eps, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && lb::valid_dtype(delta_dtype), "add_group_rmsnorm: bad dtype");
  LB_CHECK_ARG(num_rows >= 0 && hidden > 0 && groups > 0 && hidden % groups == 0,
               "add_group_rmsnorm: bad sizes rows=%d hidden=%d groups=%d", num_rows, hidden, groups);
  if (num_rows == 0) return 0;
  // about 128 elements a warp, 1 to 16 warps; a group gets a whole number of warps, or a warp whole groups in turn
  int want = (hidden + 127) / 128;
  if (want > 16) want = 16;
  if (want < 1) want = 1;
  int wpg = want / groups;
  if (wpg < 1) wpg = 1;
  int per_round = want / wpg;
  if (per_round > groups) per_round = groups;
  if (per_round < 1) per_round = 1;
  const int warps = wpg * per_round;
  const int per_lane = (hidden / groups + wpg * 32 - 1) / (wpg * 32);      // elements of a group a lane has
  LB_DISPATCH_DTYPE(delta_dtype, TD, {
    LB_DISPATCH_DTYPE(out_dtype, TO, {
      // few rows (decoding): the variant that keeps a lane's elements in registers and issues all loads at once; many
      // rows keep the SMs busy without that and run faster in the looping variant.  Both add the same terms in the same
      // order, so the choice never shows in a result.
      if (per_lane <= 8 && num_rows <= 256)
        lb::launch(lb::add_group_rmsnorm_kernel<TD, TO, 8>, dim3(num_rows), dim3(warps * 32), 0, stream, (TO*)out, residual,
                   (const TD*)delta_a, (const TD*)delta_b, weight, rows, hidden, groups, wpg, eps);
      else
        lb::launch(lb::add_group_rmsnorm_kernel<TD, TO, 0>, dim3(num_rows), dim3(warps * 32), 0, stream, (TO*)out, residual,
                   (const TD*)delta_a, (const TD*)delta_b, weight, rows, hidden, groups, wpg, eps);
    })
  })
  LB_CHECK_LAUNCH("add_group_rmsnorm");
  return 0;
}

// x *= factor, 32-bit (the scale of a model's logits).
namespace lb {
__global__ void scale_kernel(float* __restrict__ x, long long n, float factor) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] *= factor;
}
}  // namespace lb

// residual += delta in 32-bit, for a block that must hand on one delta where it has two.
namespace lb {
template <typename TD>
__global__ void add_into_kernel(float* __restrict__ residual, const TD* __restrict__ delta, long long n) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    residual[i] += to_f32(delta[i]);
}
}  // namespace lb

LB_EXPORT int lb_add_into(float* residual, const void* delta, int delta_dtype, long long n, cudaStream_t stream) {
  LB_CHECK_ARG(residual && delta && n >= 0 && lb::valid_dtype(delta_dtype), "add_into: bad arguments");
  if (n == 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  LB_DISPATCH_DTYPE(delta_dtype, TD, {
    lb::launch(lb::add_into_kernel<TD>, dim3((unsigned)blocks), dim3(256), 0, stream, residual, (const TD*)delta, n);
  })
  LB_CHECK_LAUNCH("add_into");
  return 0;
}

LB_EXPORT int lb_scale(float* x, long long n, float factor, cudaStream_t stream) {
  LB_CHECK_ARG(x && n >= 0, "scale: bad arguments");
  if (n == 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  lb::launch(lb::scale_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, n, factor);
  LB_CHECK_LAUNCH("scale");
  return 0;
}

LB_EXPORT int lb_add_rmsnorm(void* out, int out_dtype, float* residual, const void* delta,
                             int delta_dtype, const float* weight, const int* rows, int num_rows,
                             int hidden, float eps, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && lb::valid_dtype(delta_dtype), "add_rmsnorm: bad dtype");
  LB_CHECK_ARG(num_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", num_rows, hidden);
  if (num_rows == 0) return 0;
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const bool vec4 = (hidden % 4 == 0);
  // rows of 4, 8 or 16 elements a thread (a whole number of warps, 64 to 1024 threads), 16-byte aligned operands:
  // the one-pass kernel.  8 elements a thread where that works (4096 -> 512 threads, 5120 -> 640), else 4, else 16.
  int per = 0;
  for (int cand : {8, 4, 16}) {
    if (hidden % cand == 0 && (hidden / cand) % 32 == 0 && hidden / cand >= 64 && hidden / cand <= 1024) { per = cand; threads = hidden / cand; break; }
  }
  const bool aligned = ((uintptr_t)out % 16 == 0) && ((uintptr_t)residual % 16 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)weight % 16 == 0);
  if (delta == nullptr && rows == nullptr && hidden <= 512) {
    // short rows: a warp a row, whatever their number (a row's sum must not depend on the batch)
    LB_DISPATCH_DTYPE(out_dtype, TO, {
      lb::launch(lb::rmsnorm_short_rows_kernel<TO>, dim3((num_rows + 7) / 8), dim3(256), 0, stream, (TO*)out, (const float*)residual,
                 weight, num_rows, hidden, eps);
    })
    LB_CHECK_LAUNCH("add_rmsnorm");
    return 0;
  }
  LB_DISPATCH_DTYPE(delta_dtype, TD, {
    LB_DISPATCH_DTYPE(out_dtype, TO, {
      if (aligned && (per == 4 || per == 8 || per == 16)) {
        if (per == 4)
          lb::launch(lb::add_rmsnorm_row_kernel<TD, TO, 4>, dim3(num_rows), dim3(threads), 0, stream,
                     (TO*)out, residual, (const TD*)delta, weight, rows, hidden, eps);
        else if (per == 8)
          lb::launch(lb::add_rmsnorm_row_kernel<TD, TO, 8>, dim3(num_rows), dim3(threads), 0, stream,
                     (TO*)out, residual, (const TD*)delta, weight, rows, hidden, eps);
        else
          lb::launch(lb::add_rmsnorm_row_kernel<TD, TO, 16>, dim3(num_rows), dim3(threads), 0, stream,
                     (TO*)out, residual, (const TD*)delta, weight, rows, hidden, eps);
      } else if (vec4)
        lb::launch(lb::add_rmsnorm_kernel<TD, TO, 4>, dim3(num_rows), dim3(threads), 0, stream,
                   (TO*)out, residual, (const TD*)delta, weight, rows, hidden, eps);
      else
        lb::launch(lb::add_rmsnorm_kernel<TD, TO, 1>, dim3(num_rows), dim3(threads), 0, stream,
                   (TO*)out, residual, (const TD*)delta, weight, rows, hidden, eps);
    })
  })
  LB_CHECK_LAUNCH("add_rmsnorm");
  return 0;
}

// Two norms of one stream, and the sum of two normed rows: what a block needs whose two sublayers read the same
// residual stream through a norm each, and a mixer that adds two outputs after norming each over the model width.
//
// lb_add_rmsnorm_pair: residual += delta_a + delta_b (each optional, 32-bit sum, in place); then, with
// f = 1 / sqrt(mean(residual^2) + eps), out_a = residual * f * w_a and (optional) out_b = residual * f * w_b: the
// two norms share the row's root mean square and differ in their weights only.
// lb_rmsnorm_mix2: out = sa * a / rms(a) * w_a + sb * b / rms(b) * w_b, 32-bit rows in and out.
// One CTA a row, sums in an order that the row's size fixes.
namespace lb {

template <typename TD, typename TO>
__global__ void add_rmsnorm_pair_kernel(TO* __restrict__ out_a, TO* __restrict__ out_b, float* __restrict__ residual,
                                        const TD* __restrict__ delta_a, const TD* __restrict__ delta_b,
                                        const float* __restrict__ w_a, const float* __restrict__ w_b, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = residual[base + i];
    if (delta_a) v += to_f32(delta_a[base + i]);
    if (delta_b) v += to_f32(delta_b[base + i]);
    if (delta_a || delta_b) residual[base + i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = residual[base + i] * inv;
    out_a[base + i] = from_f32<TO>(v * w_a[i]);
    if (out_b) out_b[base + i] = from_f32<TO>(v * w_b[i]);
  }
}

__global__ void rmsnorm_mix2_kernel(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                    const float* __restrict__ w_a, const float* __restrict__ w_b, float sa, float sb, int hidden,
                                    float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * hidden;
  float ssa = 0.f, ssb = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float x = a[base + i], y = b[base + i];
    ssa += x * x;
    ssb += y * y;
  }
  ssa = block_sum(ssa, scratch);
  ssb = block_sum(ssb, scratch);
  const float fa = sa / sqrtf(ssa / (float)hidden + eps), fb = sb / sqrtf(ssb / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    out[base + i] = a[base + i] * fa * w_a[i] + b[base + i] * fb * w_b[i];
}

}  // namespace lb

LB_EXPORT int lb_add_rmsnorm_pair(void* out_a, void* out_b, int out_dtype, float* residual, const void* delta_a,
                                  const void* delta_b, int delta_dtype, const float* w_a, const float* w_b, int num_rows,
                                  int hidden, float eps, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && lb::valid_dtype(delta_dtype), "add_rmsnorm_pair: bad dtype");
  LB_CHECK_ARG(out_a && residual && w_a && (!out_b || w_b) && num_rows >= 0 && hidden > 0, "add_rmsnorm_pair: bad arguments");
  if (num_rows == 0) return 0;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  LB_DISPATCH_DTYPE(delta_dtype, TD, {
    LB_DISPATCH_DTYPE(out_dtype, TO, {
      lb::launch(lb::add_rmsnorm_pair_kernel<TD, TO>, dim3(num_rows), dim3(threads), 0, stream, (TO*)out_a, (TO*)out_b, residual,
                 (const TD*)delta_a, (const TD*)delta_b, w_a, w_b, hidden, eps);
    })
  })
  LB_CHECK_LAUNCH("add_rmsnorm_pair");
  return 0;
}

LB_EXPORT int lb_rmsnorm_mix2(float* out, const float* a, const float* b, const float* w_a, const float* w_b, float sa, float sb,
                              int num_rows, int hidden, float eps, cudaStream_t stream) {
  LB_CHECK_ARG(out && a && b && w_a && w_b && num_rows >= 0 && hidden > 0, "rmsnorm_mix2: bad arguments");
  if (num_rows == 0) return 0;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  lb::launch(lb::rmsnorm_mix2_kernel, dim3(num_rows), dim3(threads), 0, stream, out, a, b, w_a, w_b, sa, sb, hidden, eps);
  LB_CHECK_LAUNCH("rmsnorm_mix2");
  return 0;
}
