// Linear attention with a fixed decay per head ("lightning attention"): per sequence and head, with a state
// S [dim, vdim] in 32-bit,
//
//   q_t = silu(a_t)   k_t = silu(b_t)   v_t = silu(c_t)        a, b, c: this token's columns of the input projection
//   (or, with act = 0, q, k, v as the columns hold them: a mixer that rotates q and k first, for one)
//   S_t = decay_h * S_(t-1) + k_t v_t^T
//   o_t = S_t^T q_t
//
// for the tokens of a step, which are portions of several sequences; a sequence's state is read from its slot
// before its first token of the step and written back after its last.  Everything here is 32-bit, and the
// state is carried token by token: no chunk is multiplied out, so nothing is divided by a power of the decay.
//
// One CTA takes (32 value columns, one head, one sequence).  Warp w keeps rows w*DS .. w*DS+DS-1 of the state
// in registers, one value column a lane.  The tokens are walked in chunks: all threads turn a chunk's inputs into
// q, k and v in shared memory, then every warp walks the chunk's tokens in order and leaves its share of o_t,
// and the shares are added in warp order.  The order of every sum is fixed by (dim, DS) alone, so a token's
// result does not depend on how the sequence was cut into steps or on what else is in the batch.
//
// Also here: what follows the recurrence in a mixer of this kind (the heads' outputs normed together, gated
// elementwise) and the gate of one number a head that a softmax attention beside it may have.
#include "common.cuh"

namespace lb {

struct DecayRecurrenceParams {
  const float* pre; long long ld;       // [T, ld]: q pre-activations at q_col, k at k_col, v at v_col
  int q_col, k_col, v_col;
  const float* decay;                   // [heads]
  float* state;                         // [slots + 1, heads, dim, vdim]
  float* out;                           // [T, heads * vdim]
  const int* cu_tokens; const int* slots;
  int heads, dim, vdim;
  int act;                              // 1: q, k, v pass silu; 0: they are taken as they come
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

template <int DS, int TC, int MAX_THREADS>
__global__ void __launch_bounds__(MAX_THREADS) decay_recurrence_kernel(DecayRecurrenceParams p) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int dimp = nwarps * DS;
  float* ks = smem;                                   // [TC][dimp]
  float* qs = ks + TC * dimp;                         // [TC][dimp]
  float* vs = qs + TC * dimp;                         // [TC][32]
  float* part = vs + TC * 32;                         // [TC][nwarps][32]
  const int e = blockIdx.x * 32 + lane, h = blockIdx.y, seq = blockIdx.z;
  const bool e_ok = e < p.vdim;
  const float decay = p.decay[h];
  const int first = p.cu_tokens[seq], n = p.cu_tokens[seq + 1] - first;
  float* st = p.state + (((size_t)p.slots[seq] * p.heads + h) * p.dim) * p.vdim;
  float s[DS];
  pdl_wait();
#pragma unroll
  for (int i = 0; i < DS; ++i) {
    const int d = warp * DS + i;
    s[i] = (d < p.dim && e_ok) ? st[(size_t)d * p.vdim + e] : 0.f;
  }
  for (int c0 = 0; c0 < n; c0 += TC) {
    const int cn = min(TC, n - c0);
    for (int idx = threadIdx.x; idx < cn * dimp; idx += blockDim.x) {
      const int tt = idx / dimp, d = idx - tt * dimp;
      float k = 0.f, q = 0.f;                         // rows beyond dim: nothing enters, nothing is read
      if (d < p.dim) {
        const float* row = p.pre + (size_t)(first + c0 + tt) * p.ld + h * p.dim + d;
        q = p.act ? silu_f(row[p.q_col]) : row[p.q_col];
        k = p.act ? silu_f(row[p.k_col]) : row[p.k_col];
      }
      ks[idx] = k; qs[idx] = q;
    }
    for (int idx = threadIdx.x; idx < cn * 32; idx += blockDim.x) {
      const int tt = idx >> 5, ee = blockIdx.x * 32 + (idx & 31);
      float v = 0.f;
      if (ee < p.vdim) {
        v = p.pre[(size_t)(first + c0 + tt) * p.ld + p.v_col + h * p.vdim + ee];
        if (p.act) v = silu_f(v);
      }
      vs[idx] = v;
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float v = vs[tt * 32 + lane];
      const float* kr = ks + tt * dimp + warp * DS;
      const float* qr = qs + tt * dimp + warp * DS;
      float acc = 0.f;                                // rows in order
#pragma unroll
      for (int i4 = 0; i4 < DS; i4 += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + i4);
        const float4 q4 = *reinterpret_cast<const float4*>(qr + i4);
        s[i4 + 0] = fmaf(decay, s[i4 + 0], k4.x * v); acc = fmaf(s[i4 + 0], q4.x, acc);
        s[i4 + 1] = fmaf(decay, s[i4 + 1], k4.y * v); acc = fmaf(s[i4 + 1], q4.y, acc);
        s[i4 + 2] = fmaf(decay, s[i4 + 2], k4.z * v); acc = fmaf(s[i4 + 2], q4.z, acc);
        s[i4 + 3] = fmaf(decay, s[i4 + 3], k4.w * v); acc = fmaf(s[i4 + 3], q4.w, acc);
      }
      part[(tt * nwarps + warp) * 32 + lane] = acc;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < cn * 32; idx += blockDim.x) {
      const int tt = idx >> 5, l = idx & 31, ee = blockIdx.x * 32 + l;
      if (ee >= p.vdim) continue;
      float o = 0.f;
      for (int w = 0; w < nwarps; ++w) o += part[(tt * nwarps + w) * 32 + l];
      p.out[(size_t)(first + c0 + tt) * (p.heads * p.vdim) + h * p.vdim + ee] = o;
    }
    // the next chunk's staging writes ks, qs and vs, which nobody reads any more; `part` is written again only
    // behind the barrier that follows that staging
  }
#pragma unroll
  for (int i = 0; i < DS; ++i) {
    const int d = warp * DS + i;
    if (d < p.dim && e_ok) st[(size_t)d * p.vdim + e] = s[i];
  }
}

template <int DS, int TC, int MAX_THREADS = 256>
static cudaError_t launch_decay_recurrence(const DecayRecurrenceParams& p, int num_seqs, cudaStream_t stream) {
  const int nwarps = (p.dim + DS - 1) / DS;
  const size_t smem = (size_t)TC * (2 * nwarps * DS + 32 + nwarps * 32) * sizeof(float);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    const cudaError_t e = cudaFuncSetAttribute(decay_recurrence_kernel<DS, TC, MAX_THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    allowed = smem;
  }
  return launch(decay_recurrence_kernel<DS, TC, MAX_THREADS>, dim3((p.vdim + 31) / 32, p.heads, num_seqs), dim3(nwarps * 32), smem, stream, p);
}


// The same recurrence with a chunk's OUTPUTS formed side by side instead of token after token, for steps that bring many
// tokens a sequence.  With S0 the state before a chunk of C tokens and t, j counting inside the chunk,
//
//   o_t = decay^(t+1) * S0^T q_t  +  sum_{j <= t} decay^(t-j) (q_t . k_j) v_j
//
// The first term is C independent sums over the rows of S0 (no token waits for the one before), the second needs the
// C x C scores of the chunk, which every thread of the CTA shares.  The state itself still moves token by token,
// S <- decay S + k_j v_j^T, the very operations of the kernel above; only the order in which an output's terms are
// added differs (32-bit throughout; silu by the fast exponential and reciprocal, 2 ulp).  The raw inputs of the next
// chunk are requested before the work on the current one and turned into q, k, v after it.
//
// Both terms are sums over the rows of the state (the scores are sums over the same rows of q and k), so the rows may
// be shared out: with `row_split` R a CTA takes dim / R rows and writes its share of every output to plane r of `out`
// ([R, T, heads * vdim]); whoever reads `out` adds the planes in order.  A prompt of one sequence then fills R times
// as many SMs.
constexpr int DC_C = 16;

struct DecayChunkParams {
  DecayRecurrenceParams b;
  int row_split, rows_a_cta;              // rows_a_cta: a multiple of 4
  long long plane;                        // elements between two planes of out
};

__device__ __forceinline__ float silu_fast(float x) { return x * __frcp_rn(1.f + __expf(-x)); }

template <int DS, int NV>      // NV: values of v a thread holds for the next chunk, ceil(C * 32 / threads) rounded up to 2, 4, 8 or 16
__global__ void __launch_bounds__(256) decay_chunk_kernel(DecayChunkParams pc) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  const DecayRecurrenceParams& p = pc.b;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5, nt = blockDim.x;
  const int dimp = nwarps * DS, ldq = dimp + 4;       // rows padded by 4 floats: the scores read 16 rows at one column
  constexpr int PER = 2 * DC_C * DS / 32;             // raw q and k values a thread holds for the next chunk (2 C dimp / threads)
  constexpr int TSTEP = 32 / DS;                      // tokens between two of a thread's values: threads / dimp
  float* qs = smem;                                   // [C][ldq]
  float* ks = qs + DC_C * ldq;                        // [C][ldq]
  float* vs = ks + DC_C * ldq;                        // [C][32]
  float* part = vs + DC_C * 32;                       // [C][nwarps][32]
  float* wts = part + DC_C * nwarps * 32;             // [C][C + 1]
  const int ct = blockIdx.x / pc.row_split, rs = blockIdx.x - ct * pc.row_split;
  const int e0 = ct * 32, e = e0 + lane, h = blockIdx.y, seq = blockIdx.z;
  const int row0 = rs * pc.rows_a_cta, row_end = min(p.dim, row0 + pc.rows_a_cta);     // this CTA's rows of the state
  const bool e_ok = e < p.vdim;
  const float decay = p.decay[h];
  float pw[DC_C + 1];                                 // powers of the decay
  pw[0] = 1.f;
#pragma unroll
  for (int i = 1; i <= DC_C; ++i) pw[i] = pw[i - 1] * decay;
  const int first = p.cu_tokens[seq], n = p.cu_tokens[seq + 1] - first;
  float* st = p.state + (((size_t)p.slots[seq] * p.heads + h) * p.dim) * p.vdim;
  float* out = p.out + (size_t)rs * pc.plane;
  float s[DS];
  float raw[PER], rawv[NV];
  // a thread's u-th raw value is q (u < PER / 2) or k at (token u' * TSTEP + tq, row td) of the chunk, u' = u mod PER / 2
  const int tq = threadIdx.x / dimp, td = threadIdx.x - tq * dimp;
  const bool td_ok = row0 + td < row_end;
  const float* q_src = p.pre + p.q_col + h * p.dim + row0 + td;
  const float* k_src = p.pre + p.k_col + h * p.dim + row0 + td;
  pdl_wait();
  auto request = [&](int c0) {                        // the raw inputs of the chunk that starts at token c0
    const int cn = min(DC_C, n - c0);
#pragma unroll
    for (int u = 0; u < PER / 2; ++u) {
      const int tt = u * TSTEP + tq;
      const bool ok = tt < cn && td_ok;
      const size_t off = (size_t)(first + c0 + tt) * p.ld;
      raw[u] = ok ? q_src[off] : -INFINITY;
      raw[PER / 2 + u] = ok ? k_src[off] : -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      const int idx = u * nt + threadIdx.x, tt = idx >> 5, ee = e0 + (idx & 31);
      rawv[u] = (idx < DC_C * 32 && tt < cn && ee < p.vdim) ? p.pre[(size_t)(first + c0 + tt) * p.ld + p.v_col + h * p.vdim + ee] : -INFINITY;
    }
  };
  auto stage = [&]() {                                // silu of what was requested, into shared memory (nothing requested: 0)
#pragma unroll
    for (int u = 0; u < PER / 2; ++u) {
      const int tt = u * TSTEP + tq;
      qs[tt * ldq + td] = raw[u] == -INFINITY ? 0.f : (p.act ? silu_fast(raw[u]) : raw[u]);
      ks[tt * ldq + td] = raw[PER / 2 + u] == -INFINITY ? 0.f : (p.act ? silu_fast(raw[PER / 2 + u]) : raw[PER / 2 + u]);
    }
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      const int idx = u * nt + threadIdx.x;
      if (idx < DC_C * 32) vs[idx] = rawv[u] == -INFINITY ? 0.f : (p.act ? silu_fast(rawv[u]) : rawv[u]);
    }
  };
#pragma unroll
  for (int i = 0; i < DS; ++i) {
    const int d = row0 + warp * DS + i;
    s[i] = (d < row_end && e_ok) ? st[(size_t)d * p.vdim + e] : 0.f;
  }
  if (n > 0) { request(0); stage(); }
  __syncthreads();
  for (int c0 = 0; c0 < n; c0 += DC_C) {
    const int cn = min(DC_C, n - c0);
    if (c0 + DC_C < n) request(c0 + DC_C);
    // the part of every output that comes from the state before the chunk: C sums side by side
    {
      float acc[DC_C];
#pragma unroll
      for (int t = 0; t < DC_C; ++t) acc[t] = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < DS; i4 += 4) {
#pragma unroll
        for (int t = 0; t < DC_C; ++t) {
          const float4 q4 = *reinterpret_cast<const float4*>(qs + t * ldq + warp * DS + i4);
          acc[t] = fmaf(s[i4 + 0], q4.x, acc[t]); acc[t] = fmaf(s[i4 + 1], q4.y, acc[t]);
          acc[t] = fmaf(s[i4 + 2], q4.z, acc[t]); acc[t] = fmaf(s[i4 + 3], q4.w, acc[t]);
        }
      }
#pragma unroll
      for (int t = 0; t < DC_C; ++t) part[(t * nwarps + warp) * 32 + lane] = acc[t] * pw[t + 1];
    }
    // the state moves on, token by token
    for (int j = 0; j < cn; ++j) {
      const float v = vs[j * 32 + lane];
      const float* kr = ks + j * ldq + warp * DS;
#pragma unroll
      for (int i4 = 0; i4 < DS; i4 += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + i4);
        s[i4 + 0] = fmaf(decay, s[i4 + 0], k4.x * v); s[i4 + 1] = fmaf(decay, s[i4 + 1], k4.y * v);
        s[i4 + 2] = fmaf(decay, s[i4 + 2], k4.z * v); s[i4 + 3] = fmaf(decay, s[i4 + 3], k4.w * v);
      }
    }
    // the chunk's own scores, weighted by the decay over the distance: wts[t][j] = decay^(t-j) (q_t . k_j) for j <= t
    for (int idx = threadIdx.x; idx < DC_C * DC_C; idx += nt) {
      const int t = idx / DC_C, j = idx - t * DC_C;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      if (j <= t && t < cn) {
        const float* qr = qs + t * ldq;
        const float* kr = ks + j * ldq;
        for (int i = 0; i < dimp; i += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qr + i);
          const float4 k4 = *reinterpret_cast<const float4*>(kr + i);
          a0 = fmaf(q4.x, k4.x, a0); a1 = fmaf(q4.y, k4.y, a1); a2 = fmaf(q4.z, k4.z, a2); a3 = fmaf(q4.w, k4.w, a3);
        }
      }
      float w = 1.f;                                   // decay^(t-j) by the same products as the table
      for (int r = 0; r < t - j; ++r) w *= decay;
      wts[t * (DC_C + 1) + j] = ((a0 + a1) + (a2 + a3)) * w;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < cn * 32; idx += nt) {
      const int t = idx >> 5, l = idx & 31, ee = e0 + l;
      if (ee >= p.vdim) continue;
      float o = 0.f;
      for (int w = 0; w < nwarps; ++w) o += part[(t * nwarps + w) * 32 + l];
      for (int j = 0; j <= t; ++j) o = fmaf(wts[t * (DC_C + 1) + j], vs[j * 32 + l], o);
      out[(size_t)(first + c0 + t) * (p.heads * p.vdim) + h * p.vdim + ee] = o;
    }
    __syncthreads();
    if (c0 + DC_C < n) stage();
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < DS; ++i) {
    const int d = row0 + warp * DS + i;
    if (d < row_end && e_ok) st[(size_t)d * p.vdim + e] = s[i];
  }
}

template <int DS, int NV>
static cudaError_t launch_decay_chunk_nv(const DecayChunkParams& pc, int num_seqs, int nwarps, cudaStream_t stream) {
  const int dimp = nwarps * DS;
  const size_t smem = (size_t)(2 * DC_C * (dimp + 4) + DC_C * 32 + DC_C * nwarps * 32 + DC_C * (DC_C + 1)) * sizeof(float);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    const cudaError_t e = cudaFuncSetAttribute(decay_chunk_kernel<DS, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    allowed = smem;
  }
  return launch(decay_chunk_kernel<DS, NV>, dim3(((pc.b.vdim + 31) / 32) * pc.row_split, pc.b.heads, num_seqs), dim3(nwarps * 32), smem, stream, pc);
}

template <int DS>
static cudaError_t launch_decay_chunk(const DecayChunkParams& pc, int num_seqs, cudaStream_t stream) {
  const int nwarps = (pc.rows_a_cta + DS - 1) / DS;
  const int nv = (DC_C * 32 + nwarps * 32 - 1) / (nwarps * 32);
  if (nv <= 2) return launch_decay_chunk_nv<DS, 2>(pc, num_seqs, nwarps, stream);
  if (nv <= 4) return launch_decay_chunk_nv<DS, 4>(pc, num_seqs, nwarps, stream);
  if (nv <= 8) return launch_decay_chunk_nv<DS, 8>(pc, num_seqs, nwarps, stream);
  return launch_decay_chunk_nv<DS, 16>(pc, num_seqs, nwarps, stream);
}

// out[t, :] = x[t, :] * rsqrt(mean(x[t]^2) + eps) * weight * sigmoid(gate[t, :]) * scale: the heads' outputs normed
// together and gated elementwise.  out may be a column range of a wider matrix (row stride out_ld).  x may come in
// `planes` planes (`plane` elements apart) whose sum is meant; they are added in order.
template <typename TO>
__global__ void rmsnorm_gated_kernel(TO* __restrict__ out, long long out_ld, const float* __restrict__ x,
                                     const float* __restrict__ weight, const float* __restrict__ gate, long long gate_ld,
                                     float scale, float eps, int n, int planes, long long plane) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const float* r = x + (size_t)blockIdx.x * n;
  const float* g = gate + (size_t)blockIdx.x * gate_ld;
  auto value = [&](int j) {
    float v = r[j];
    for (int q = 1; q < planes; ++q) v += r[(size_t)q * plane + j];
    return v;
  };
  float ss = 0.f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) { const float v = value(j); ss += v * v; }
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)n + eps);
  TO* o = out + (size_t)blockIdx.x * out_ld;
  for (int j = threadIdx.x; j < n; j += blockDim.x)
    o[j] = from_f32<TO>(value(j) * inv * weight[j] * (1.f / (1.f + expf(-g[j]))) * scale);
}

// out[t, h, :] = x[t, h, :] * sigmoid(gate[t, h]) * scale: one number a head
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, long long out_ld, const T* __restrict__ x, const float* __restrict__ gate,
                                 long long gate_ld, float scale, int heads, int vdim) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, n = heads * vdim;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float g = gate[(size_t)t * gate_ld + j / vdim];
    out[(size_t)t * out_ld + j] = from_f32<T>(to_f32(x[(size_t)t * n + j]) * (1.f / (1.f + expf(-g))) * scale);
  }
}

}  // namespace lb

// max_tokens_a_seq: the most tokens any sequence brings, if the host knows it (0: unknown); in the token-by-token kernel
// it only chooses the chunk's size, which never shows in a result.
// row_split >= 1 asks for the kernel that forms a chunk's outputs side by side (steps of more than 4 tokens a sequence):
// the same state within 32-bit rounding of the activations, outputs equal within rounding (their terms are added in
// another order), several times faster.  `out` then has row_split planes of `plane` elements, each CTA's share of the
// outputs going to the plane of its rows (see lb_decay_row_split); the reader adds them.  0 keeps every step in the
// token-by-token kernel, whose outputs do not depend on how a sequence was cut into steps.
LB_EXPORT int lb_decay_row_split(int num_seqs, int heads, int dim, int vdim, int max_tokens_a_seq) {
  if ((max_tokens_a_seq > 0 && max_tokens_a_seq <= 4) || dim > 1024) return 0;          // the token-by-token kernel
  const long long base = (long long)num_seqs * heads * ((vdim + 31) / 32);
  int r = 1;
  while (r < 8 && base * r < 148 && dim / (2 * r) >= 32) r *= 2;     // fill the SMs, with 32 rows a CTA at least
  while (dim / r > 256) r *= 2;                                      // at most 256 rows a CTA
  return r;
}

LB_EXPORT int lb_decay_recurrence(const float* pre, long long ld, int q_col, int k_col, int v_col, const float* decay,
                                  float* state, float* out, const int* cu_tokens, const int* slots, int num_seqs,
                                  int heads, int dim, int vdim, int max_tokens_a_seq, int row_split, long long plane,
                                  int act, cudaStream_t stream) {
  LB_CHECK_ARG(pre && decay && state && out && cu_tokens && slots, "decay_recurrence: null argument");
  LB_CHECK_ARG(num_seqs >= 0 && heads > 0 && heads <= 65535 && dim > 0 && dim <= 1024 && vdim > 0 && num_seqs <= 65535,
               "decay_recurrence: bad sizes seqs=%d heads=%d dim=%d vdim=%d (dim at most 1024)", num_seqs, heads, dim, vdim);
  if (num_seqs == 0) return 0;
  lb::DecayRecurrenceParams p;
  p.pre = pre; p.ld = ld; p.q_col = q_col; p.k_col = k_col; p.v_col = v_col; p.decay = decay;
  p.state = state; p.out = out; p.cu_tokens = cu_tokens; p.slots = slots; p.heads = heads; p.dim = dim; p.vdim = vdim;
  p.act = act ? 1 : 0;
  const bool few = max_tokens_a_seq > 0 && max_tokens_a_seq <= 4;
  cudaError_t e;
  if (row_split >= 1) {
    lb::DecayChunkParams pc;
    pc.b = p; pc.row_split = row_split; pc.plane = plane;
    pc.rows_a_cta = ((dim + row_split - 1) / row_split + 3) / 4 * 4;
    LB_CHECK_ARG(pc.rows_a_cta <= 256 && row_split <= 64, "decay_recurrence: %d rows cannot be shared out %d ways", dim, row_split);
    const int rows = pc.rows_a_cta;
    if (rows <= 32) e = lb::launch_decay_chunk<4>(pc, num_seqs, stream);
    else if (rows <= 64) e = lb::launch_decay_chunk<8>(pc, num_seqs, stream);
    else if (rows <= 128) e = lb::launch_decay_chunk<16>(pc, num_seqs, stream);
    else e = lb::launch_decay_chunk<32>(pc, num_seqs, stream);
    if (e != cudaSuccess) { lb::set_error("decay_recurrence: %s", cudaGetErrorString(e)); return 2; }
    LB_CHECK_LAUNCH("decay_recurrence");
    return 0;
  }
  // rows of the state a warp keeps: as few as give at most 8 warps; heads of more than 256 rows: 32 rows a warp
  if (dim > 256) e = lb::launch_decay_recurrence<32, 4, 1024>(p, num_seqs, stream);
  else if (few) {
    if (dim <= 32) e = lb::launch_decay_recurrence<4, 4>(p, num_seqs, stream);
    else if (dim <= 64) e = lb::launch_decay_recurrence<8, 4>(p, num_seqs, stream);
    else if (dim <= 128) e = lb::launch_decay_recurrence<16, 4>(p, num_seqs, stream);
    else e = lb::launch_decay_recurrence<32, 4>(p, num_seqs, stream);
  } else if (dim <= 32) e = lb::launch_decay_recurrence<4, 16>(p, num_seqs, stream);
  else if (dim <= 64) e = lb::launch_decay_recurrence<8, 16>(p, num_seqs, stream);
  else if (dim <= 128) e = lb::launch_decay_recurrence<16, 16>(p, num_seqs, stream);
  else e = lb::launch_decay_recurrence<32, 16>(p, num_seqs, stream);
  if (e != cudaSuccess) { lb::set_error("decay_recurrence: %s", cudaGetErrorString(e)); return 2; }
  LB_CHECK_LAUNCH("decay_recurrence");
  return 0;
}

LB_EXPORT int lb_rmsnorm_gated(void* out, int out_dtype, long long out_ld, const float* x, const float* weight,
                               const float* gate, long long gate_ld, float scale, float eps, int num_rows, int n,
                               int planes, long long plane, cudaStream_t stream) {
  LB_CHECK_ARG(planes >= 1, "rmsnorm_gated: at least one plane");
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && out && x && weight && gate, "rmsnorm_gated: bad arguments");
  LB_CHECK_ARG(num_rows >= 0 && n > 0 && out_ld >= n && gate_ld >= n, "rmsnorm_gated: bad sizes rows=%d n=%d", num_rows, n);
  if (num_rows == 0) return 0;
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  LB_DISPATCH_DTYPE(out_dtype, TO, {
    lb::launch(lb::rmsnorm_gated_kernel<TO>, dim3(num_rows), dim3(threads), 0, stream, (TO*)out, out_ld, x, weight, gate, gate_ld,
               scale, eps, n, planes, plane);
  })
  LB_CHECK_LAUNCH("rmsnorm_gated");
  return 0;
}

LB_EXPORT int lb_head_gate(void* out, int dtype, long long out_ld, const void* x, const float* gate, long long gate_ld,
                           float scale, int num_rows, int heads, int vdim, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype) && out && x && gate, "head_gate: bad arguments");
  LB_CHECK_ARG(num_rows >= 0 && heads > 0 && vdim > 0 && out_ld >= (long long)heads * vdim && gate_ld >= heads,
               "head_gate: bad sizes rows=%d heads=%d vdim=%d", num_rows, heads, vdim);
  if (num_rows == 0) return 0;
  const int n = heads * vdim;
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  LB_DISPATCH_DTYPE(dtype, T, {
    lb::launch(lb::head_gate_kernel<T>, dim3(num_rows), dim3(threads), 0, stream, (T*)out, out_ld, (const T*)x, gate, gate_ld, scale,
               heads, vdim);
  })
  LB_CHECK_LAUNCH("head_gate");
  return 0;
}
