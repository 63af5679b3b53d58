// Linear recurrences whose decay and write strength depend on the token: the gated delta rule and the selective
// state space of Mamba-2, one kernel.  Per head, with a 32-bit state S [dim, vdim] that a sequence carries from
// token to token (zero for a new sequence):
//
//   delta rule    g = exp(-exp(A_h) softplus(a_t + dt_h))     w = sigmoid(b_t)
//                 S <- g S;   u = w (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//   state space   w = softplus(a_t + dt_h)     g = exp(-exp(A_h) w)
//                 S <- g S + k_t (w v_t)^T;    o_t = S^T q_t + D_h v_t          (k = B, q = C, v = x)
//
// The two differ in one term: the delta rule takes what the state already predicts for k_t off the value before it
// writes.  q and k come in `groups` heads of `dim` that heads / groups heads share; with unit_norm they are made unit
// vectors first, x / sqrt(sum x^2 + unit_eps), and q is multiplied by q_scale.  All inputs are 32-bit rows that may
// be column ranges of wider matrices; a, b are one number a head and token.
//
// A CTA takes (32 value columns, a head, a sequence) and walks the sequence's tokens of this step in order.  A
// column of the state belongs to four neighbouring lanes, which hold its rows r = sub + 4 i in registers and add
// their partial dot products by two shuffles; the columns never talk to one another.  The tokens' q, k, v, g, w are
// staged through shared memory 16 tokens at a time (the unit norm and the decay are formed there, a warp a token).
// Every sum visits its terms in an order that the sizes fix, so a result does not depend on how a sequence is cut
// into steps or on what else the step holds.
#include "common.cuh"

namespace lb {

constexpr int SR_TOKENS = 16;    // tokens staged at a time
constexpr int SR_COLS = 32;      // value columns of a CTA
constexpr int SR_SUB = 4;        // lanes that share a column

struct StateRecurrenceParams {
  const float* q; const float* k; const float* v; const float* a; const float* b;
  long long q_ld, k_ld, v_ld, a_ld, b_ld;
  const float* A_log; const float* dt_bias; const float* D;
  float* state; float* out; long long out_ld;
  const int* cu_tokens; const int* slots;
  int heads, groups, dim, vdim, unit_norm;
  float q_scale, unit_eps;
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <bool DELTA, int RPL>
__global__ void __launch_bounds__(SR_COLS * SR_SUB) state_recurrence_kernel(StateRecurrenceParams p) {
  constexpr int DP = RPL * SR_SUB;                 // rows, padded
  __shared__ float q_s[SR_TOKENS][DP];
  __shared__ float k_s[SR_TOKENS][DP];
  __shared__ float v_s[SR_TOKENS][SR_COLS];
  __shared__ float g_s[SR_TOKENS], w_s[SR_TOKENS];
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = tid % SR_SUB, col_local = tid / SR_SUB;
  const int h = blockIdx.y, seq = blockIdx.z;
  const int col = blockIdx.x * SR_COLS + col_local;
  const bool col_ok = col < p.vdim;
  const int grp = h / (p.heads / p.groups);
  const float A = expf(p.A_log[h]), dtb = p.dt_bias[h];
  const float Dh = p.D ? p.D[h] : 0.f;
  pdl_wait();
  const int first = p.cu_tokens[seq], n = p.cu_tokens[seq + 1] - first;
  float* S = p.state + ((size_t)p.slots[seq] * p.heads + h) * p.dim * p.vdim;

  float s[RPL];
#pragma unroll
  for (int i = 0; i < RPL; ++i) {
    const int r = sub + SR_SUB * i;
    s[i] = (col_ok && r < p.dim) ? S[(size_t)r * p.vdim + col] : 0.f;
  }

  for (int t0 = 0; t0 < n; t0 += SR_TOKENS) {
    const int nt = min(SR_TOKENS, n - t0);
    __syncthreads();                               // the chunk before has been read
    for (int i = tid; i < nt * DP; i += blockDim.x) {
      const int tt = i / DP, r = i % DP;
      const size_t row = (size_t)(first + t0 + tt);
      q_s[tt][r] = r < p.dim ? p.q[row * p.q_ld + (size_t)grp * p.dim + r] : 0.f;
      k_s[tt][r] = r < p.dim ? p.k[row * p.k_ld + (size_t)grp * p.dim + r] : 0.f;
    }
    for (int i = tid; i < nt * SR_COLS; i += blockDim.x) {
      const int tt = i / SR_COLS, c = blockIdx.x * SR_COLS + i % SR_COLS;
      v_s[tt][i % SR_COLS] = c < p.vdim ? p.v[(size_t)(first + t0 + tt) * p.v_ld + (size_t)h * p.vdim + c] : 0.f;
    }
    if (tid < nt) {
      const size_t row = (size_t)(first + t0 + tid);
      const float sp = softplus_f(p.a[row * p.a_ld + h] + dtb);
      g_s[tid] = expf(-A * sp);
      w_s[tid] = DELTA ? 1.f / (1.f + expf(-p.b[row * p.b_ld + h])) : sp;
    }
    __syncthreads();
    if (p.unit_norm) {
      for (int tt = warp; tt < nt; tt += (SR_COLS * SR_SUB) / 32) {
        float sq = 0.f, sk = 0.f;
        for (int r = lane; r < p.dim; r += 32) { sq += q_s[tt][r] * q_s[tt][r]; sk += k_s[tt][r] * k_s[tt][r]; }
        sq = warp_sum(sq); sk = warp_sum(sk);
        const float fq = p.q_scale / sqrtf(sq + p.unit_eps), fk = 1.f / sqrtf(sk + p.unit_eps);
        for (int r = lane; r < p.dim; r += 32) { q_s[tt][r] *= fq; k_s[tt][r] *= fk; }
      }
      __syncthreads();
    }
    for (int tt = 0; tt < nt; ++tt) {
      const float g = g_s[tt], w = w_s[tt], vj = v_s[tt][col_local];
      const float* kk = k_s[tt];
      const float* qq = q_s[tt];
      float u;
      if (DELTA) {
        float d0 = 0.f, d1 = 0.f;
#pragma unroll
        for (int i = 0; i < RPL; i += 2) {
          d0 = fmaf(s[i], kk[sub + SR_SUB * i], d0);
          d1 = fmaf(s[i + 1], kk[sub + SR_SUB * (i + 1)], d1);
        }
        float d = d0 + d1;
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        u = w * (vj - g * d);
      } else {
        u = w * vj;
      }
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int i = 0; i < RPL; i += 2) {
        s[i] = fmaf(g, s[i], kk[sub + SR_SUB * i] * u);
        s[i + 1] = fmaf(g, s[i + 1], kk[sub + SR_SUB * (i + 1)] * u);
        o0 = fmaf(s[i], qq[sub + SR_SUB * i], o0);
        o1 = fmaf(s[i + 1], qq[sub + SR_SUB * (i + 1)], o1);
      }
      float o = o0 + o1;
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (sub == 0 && col_ok) p.out[(size_t)(first + t0 + tt) * p.out_ld + (size_t)h * p.vdim + col] = o + Dh * vj;
    }
  }
#pragma unroll
  for (int i = 0; i < RPL; ++i) {
    const int r = sub + SR_SUB * i;
    if (col_ok && r < p.dim) S[(size_t)r * p.vdim + col] = s[i];
  }
}

// Norm in equal groups of a row with a gate, after a recurrence:
//   gate_first = 0:  out = y / rms_group(y) * w * act(gate)           (the gated delta rule: a group is a head)
//   gate_first = 1:  z = y * act(gate);  out = z / rms_group(z) * w     (Mamba-2: the gate comes before the norm)
// w has `wn` entries and is read at column % wn (wn = the group's size: one weight shared by the groups).
// act: 0 silu, 1 sigmoid.  A warp a group, the groups of a row in turn.
template <typename TO>
__global__ void gated_group_norm_kernel(TO* __restrict__ out, long long out_ld, const float* __restrict__ y, long long y_ld,
                                        const float* __restrict__ gate, long long gate_ld, const float* __restrict__ w, int wn,
                                        int n, int groups, int gate_first, int act, float eps, float scale) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gs = n / groups;
  const float* yr = y + (size_t)t * y_ld;
  const float* gr = gate + (size_t)t * gate_ld;
  for (int g = warp; g < groups; g += nwarps) {
    float ss = 0.f;
    for (int c = lane; c < gs; c += 32) {
      float x = yr[g * gs + c];
      if (gate_first) {
        const float z = gr[g * gs + c];
        x *= act == 0 ? z / (1.f + expf(-z)) : 1.f / (1.f + expf(-z));
      }
      ss += x * x;
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)gs + eps);
    for (int c = lane; c < gs; c += 32) {
      const int col = g * gs + c;
      const float z = gr[col];
      const float a = act == 0 ? z / (1.f + expf(-z)) : 1.f / (1.f + expf(-z));
      const float x = yr[col];
      const float r = gate_first ? (x * a) * inv * w[col % wn] : x * inv * w[col % wn] * a;
      out[(size_t)t * out_ld + col] = from_f32<TO>(r * scale);
    }
  }
}

}  // namespace lb

LB_EXPORT int lb_state_recurrence(int delta, const float* q, long long q_ld, const float* k, long long k_ld, const float* v,
                                  long long v_ld, const float* a, long long a_ld, const float* b, long long b_ld,
                                  const float* A_log, const float* dt_bias, const float* D, float* state, float* out,
                                  long long out_ld, const int* cu_tokens, const int* slots, int num_seqs, int heads, int groups,
                                  int dim, int vdim, int unit_norm, float q_scale, float unit_eps, cudaStream_t stream) {
  LB_CHECK_ARG(q && k && v && a && A_log && dt_bias && state && out && cu_tokens && slots && (!delta || b),
               "state_recurrence: null argument");
  LB_CHECK_ARG(heads > 0 && groups > 0 && heads % groups == 0, "state_recurrence: %d heads are not a multiple of %d groups", heads, groups);
  LB_CHECK_ARG(dim > 0 && dim <= 256 && vdim > 0, "state_recurrence: state rows %d not in 1..256", dim);
  LB_CHECK_ARG(heads <= 65535 && num_seqs <= 65535, "state_recurrence: too many heads or sequences");
  if (num_seqs == 0) return 0;
  lb::StateRecurrenceParams p;
  p.q = q; p.k = k; p.v = v; p.a = a; p.b = b; p.q_ld = q_ld; p.k_ld = k_ld; p.v_ld = v_ld; p.a_ld = a_ld; p.b_ld = b_ld;
  p.A_log = A_log; p.dt_bias = dt_bias; p.D = D; p.state = state; p.out = out; p.out_ld = out_ld;
  p.cu_tokens = cu_tokens; p.slots = slots; p.heads = heads; p.groups = groups; p.dim = dim; p.vdim = vdim;
  p.unit_norm = unit_norm; p.q_scale = q_scale; p.unit_eps = unit_eps;
  dim3 grid((vdim + lb::SR_COLS - 1) / lb::SR_COLS, heads, num_seqs), block(lb::SR_COLS * lb::SR_SUB);
#define LB_SR(RPL)                                                                                        \
  do {                                                                                                    \
    if (delta) lb::launch(lb::state_recurrence_kernel<true, RPL>, grid, block, 0, stream, p);             \
    else lb::launch(lb::state_recurrence_kernel<false, RPL>, grid, block, 0, stream, p);                  \
  } while (0)
  if (dim <= 32) LB_SR(8);
  else if (dim <= 64) LB_SR(16);
  else if (dim <= 128) LB_SR(32);
  else LB_SR(64);
#undef LB_SR
  LB_CHECK_LAUNCH("state_recurrence");
  return 0;
}

LB_EXPORT int lb_gated_group_norm(void* out, int out_dtype, long long out_ld, const float* y, long long y_ld, const float* gate,
                                  long long gate_ld, const float* w, int wn, int num_rows, int n, int groups, int gate_first,
                                  int act, float eps, float scale, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype), "gated_group_norm: bad dtype");
  LB_CHECK_ARG(out && y && gate && w && num_rows >= 0 && n > 0 && groups > 0 && n % groups == 0 && wn > 0 && (act == 0 || act == 1),
               "gated_group_norm: bad arguments rows=%d n=%d groups=%d", num_rows, n, groups);
  if (num_rows == 0) return 0;
  int warps = groups < 8 ? groups : 8;
  LB_DISPATCH_DTYPE(out_dtype, TO, {
    lb::launch(lb::gated_group_norm_kernel<TO>, dim3(num_rows), dim3(warps * 32), 0, stream, (TO*)out, out_ld, y, y_ld, gate, gate_ld,
               w, wn, n, groups, gate_first, act, eps, scale);
  })
  LB_CHECK_LAUNCH("gated_group_norm");
  return 0;
}
