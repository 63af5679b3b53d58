// Linear recurrences whose decay and write strength depend on the token: the gated delta rule and the selective
// state space of Mamba-2, one kernel.  Per head, with a 32-bit state S [dim, vdim] that a sequence carries from
// token to token (zero for a new sequence):
//
//   delta rule    g = exp(-exp(A_h) softplus(a_t + dt_h))     w = sigmoid(b_t)
//                 S <- g S;   u = w (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//                 (rows_decay: g is a vector, one decay for every row r of the state, S <- diag(g) S; `a` holds the decays, made by
//                  lb_channel_decay from a_t[h, r] and dt[h, r])
//   state space   w = softplus(a_t + dt_h)     g = exp(-exp(A_h) w)
//                 S <- g S + k_t (w v_t)^T;    o_t = S^T q_t + D_h v_t          (k = B, q = C, v = x)
//
// The two differ in one term: the delta rule takes what the state already predicts for k_t off the value before it
// writes.  q and k come in `groups` heads of `dim` that heads / groups heads share; with unit_norm they are made unit
// vectors first, x / sqrt(sum x^2 + unit_eps), and q is multiplied by q_scale.  All inputs are 32-bit rows that may
// be column ranges of wider matrices; a, b are one number a head and token.
//
// A CTA of 128 threads takes (COLS value columns, a head, a sequence) and walks the sequence's tokens of this step in
// order.  A column of the state belongs to SUB neighbouring lanes (4, 8 or 16 by the state's rows; COLS = 128 / SUB),
// each of which holds RPL consecutive rows in registers and adds its partial dot products to its neighbours' by
// shuffles; the columns never talk to one another.  The tokens' q, k, v and the two numbers a head are fetched 16
// tokens at a time by cp.async into one of two buffers, the chunk after the one at work, so the walk never waits for
// global memory; the unit norm and the decays are formed in shared memory when a chunk has landed (a warp a token).
// Only S^T k lies on the path from one token to the next: the lanes' partial read-outs S^T q go to shared memory
// unreduced and are added, SUB at a time, when the chunk is through, which also makes the stores of `out` whole
// lines.  The state enters and leaves through a shared tile, in whole lines as well.  Every sum visits its terms in
// an order that the sizes fix, so a result does not depend on how a sequence is cut into steps or on what else the
// step holds.
#include "common.cuh"

namespace lb {

constexpr int SR_TOKENS = 16;    // tokens staged at a time; 1 in steps of single tokens, whose CTAs then need a fifth of the shared memory
constexpr int SR_THREADS = 128;

struct StateRecurrenceParams {
  const float* q; const float* k; const float* v; const float* a; const float* b;
  long long q_ld, k_ld, v_ld, a_ld, b_ld;
  const float* A_log; const float* dt_bias; const float* D;
  float* state; float* out; long long out_ld;
  const int* cu_tokens; const int* slots;
  int heads, groups, dim, vdim, unit_norm;
  float q_scale, unit_eps;
  int vec;                       // q, k, v rows start on 16-byte boundaries and hold whole 16-byte pieces
  int svec;                      // so do the state's rows
  int avec;                      // with a decay for every state row: so do the rows of `a`
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

__device__ __forceinline__ void sr_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void sr_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// floats of shared memory: q and k (two buffers of 16 rows of (RPL + 4) * SUB), v, a, b (two buffers), g, w, and the
// tile that holds the lanes' partial read-outs of a chunk or, at both ends, the CTA's part of the state
// (with a decay for every state row, two more buffers of 16 rows behind the tile)
__host__ __device__ constexpr int sr_smem_floats(int rpl, int sub, int tokens, bool rows_decay = false) {
  const int cols = SR_THREADS / sub, row = (rpl + 4) * sub;
  const int tile = tokens * SR_THREADS > rpl * sub * cols ? tokens * SR_THREADS : rpl * sub * cols;
  return 4 * tokens * row + 2 * tokens * cols + 6 * (tokens < 4 ? 4 : tokens) + tile + (rows_decay ? 2 * tokens * row : 0);
}

// VG: the decay is a vector, one number for every row of the state (key channel) and token, S <- diag(g) S.  `a` then
// holds the decays themselves, heads * dim numbers a token, as lb_channel_decay leaves them: formed once for all the
// CTAs that share a head, and off the path from one token to the next.
template <bool DELTA, int RPL, int SUB, int TOK, bool VG = false>
__global__ void __launch_bounds__(SR_THREADS) state_recurrence_kernel(StateRecurrenceParams p) {
  constexpr int T = TOK, COLS = SR_THREADS / SUB, ROW = (RPL + 4) * SUB, DP = RPL * SUB;
  constexpr int TURN = 32 / SUB < 4 ? 4 : 32 / SUB;   // columns by which a lane's rows are turned in the state's tile: whole 16-byte words
  extern __shared__ __align__(16) float sr_smem[];
  float* q_s = sr_smem;                           // [2][T][ROW]: row r of a token at r + 4 * (r / RPL)
  float* k_s = q_s + 2 * T * ROW;
  float* v_s = k_s + 2 * T * ROW;                 // [2][T][COLS]
  constexpr int TS = T < 4 ? 4 : T;               // the small arrays in whole 16-byte words, so that the tile behind them is aligned
  float* a_s = v_s + 2 * T * COLS;                // [2][TS] as the product left them
  float* b_s = a_s + 2 * TS;
  float* g_s = b_s + 2 * TS;                      // [TS] decay
  float* w_s = g_s + TS;                          // [TS] write strength
  float* o_s = w_s + TS;                          // [T][COLS][SUB] partial read-outs; the state's tile [DP][COLS] at both ends
  constexpr int TILE = T * SR_THREADS > DP * COLS ? T * SR_THREADS : DP * COLS;
  float* gv_s = o_s + TILE;                       // VG: [2][T][ROW], laid out as k_s: the decays of the state's rows
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = tid % SUB, col_local = tid / SUB;
  const int h = blockIdx.y, seq = blockIdx.z;
  const int col0 = blockIdx.x * COLS;
  const int grp = h / (p.heads / p.groups);
  const float A = VG ? 0.f : expf(p.A_log[h]), dtb = VG ? 0.f : p.dt_bias[h];
  const float Dh = p.D ? p.D[h] : 0.f;
  if (p.dim < DP || col0 + COLS > p.vdim) {        // rows past dim and columns past vdim stay zero; nothing else of the buffers is read unwritten
    for (int i = tid; i < 4 * T * ROW + 2 * T * COLS; i += SR_THREADS) sr_smem[i] = 0.f;
    if (VG) for (int i = tid; i < 2 * T * ROW; i += SR_THREADS) gv_s[i] = 0.f;
  }
  pdl_wait();
  const int first = p.cu_tokens[seq], n = p.cu_tokens[seq + 1] - first;
  float* S = p.state + ((size_t)p.slots[seq] * p.heads + h) * p.dim * p.vdim;
  const int shift = (TURN * sub) % COLS;     // a lane's column of the state's tile, turned so that a warp's lanes spread over the banks

  // the state: whole lines into the tile, then each lane's rows into registers
  if (p.svec) {                                    // 16-byte words: the turn is a multiple of four columns
    for (int i = tid; i < DP * (COLS / 4); i += SR_THREADS) {
      const int r = i / (COLS / 4), c = (i % (COLS / 4)) * 4, col = col0 + c;
      const float4 x = (r < p.dim && col < p.vdim) ? *reinterpret_cast<const float4*>(S + (size_t)r * p.vdim + col) : make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(o_s + r * COLS + (c + TURN * (r / RPL)) % COLS) = x;
    }
  } else {
    for (int i = tid; i < DP * COLS; i += SR_THREADS) {
      const int r = i / COLS, c = i % COLS, col = col0 + c;
      o_s[r * COLS + (c + TURN * (r / RPL)) % COLS] = (r < p.dim && col < p.vdim) ? S[(size_t)r * p.vdim + col] : 0.f;
    }
  }
  __syncthreads();
  float s[RPL];
#pragma unroll
  for (int i = 0; i < RPL; ++i) s[i] = o_s[(sub * RPL + i) * COLS + (col_local + shift) % COLS];

  auto fetch = [&](int c) {                        // chunk c into buffer c & 1
    const int buf = c & 1, t0 = c * T, nt = min(T, n - t0);
    float* qb = q_s + buf * T * ROW;
    float* kb = k_s + buf * T * ROW;
    float* vb = v_s + buf * T * COLS;
    const size_t row0 = (size_t)(first + t0);
    if (p.vec) {
      const int per = p.dim / 4;
      for (int i = tid; i < nt * per; i += SR_THREADS) {
        const int tt = i / per, r = (i % per) * 4, dst = tt * ROW + r + 4 * (r / RPL);
        sr_cp16(qb + dst, p.q + (row0 + tt) * p.q_ld + (size_t)grp * p.dim + r);
        sr_cp16(kb + dst, p.k + (row0 + tt) * p.k_ld + (size_t)grp * p.dim + r);
      }
      for (int i = tid; i < nt * (COLS / 4); i += SR_THREADS) {
        const int tt = i / (COLS / 4), c4 = (i % (COLS / 4)) * 4;
        if (col0 + c4 < p.vdim) sr_cp16(vb + tt * COLS + c4, p.v + (row0 + tt) * p.v_ld + (size_t)h * p.vdim + col0 + c4);
      }
    } else {
      for (int i = tid; i < nt * p.dim; i += SR_THREADS) {
        const int tt = i / p.dim, r = i % p.dim, dst = tt * ROW + r + 4 * (r / RPL);
        sr_cp4(qb + dst, p.q + (row0 + tt) * p.q_ld + (size_t)grp * p.dim + r);
        sr_cp4(kb + dst, p.k + (row0 + tt) * p.k_ld + (size_t)grp * p.dim + r);
      }
      for (int i = tid; i < nt * COLS; i += SR_THREADS) {
        const int tt = i / COLS, c = i % COLS;
        if (col0 + c < p.vdim) sr_cp4(vb + tt * COLS + c, p.v + (row0 + tt) * p.v_ld + (size_t)h * p.vdim + col0 + c);
      }
    }
    if (VG) {
      float* gb = gv_s + buf * T * ROW;
      if (p.avec) {
        const int per = p.dim / 4;
        for (int i = tid; i < nt * per; i += SR_THREADS) {
          const int tt = i / per, r = (i % per) * 4;
          sr_cp16(gb + tt * ROW + r + 4 * (r / RPL), p.a + (row0 + tt) * p.a_ld + (size_t)h * p.dim + r);
        }
      } else {
        for (int i = tid; i < nt * p.dim; i += SR_THREADS) {
          const int tt = i / p.dim, r = i % p.dim;
          sr_cp4(gb + tt * ROW + r + 4 * (r / RPL), p.a + (row0 + tt) * p.a_ld + (size_t)h * p.dim + r);
        }
      }
    }
    if (tid < nt) {
      if (!VG) sr_cp4(a_s + buf * TS + tid, p.a + (row0 + tid) * p.a_ld + h);
      if (DELTA) sr_cp4(b_s + buf * TS + tid, p.b + (row0 + tid) * p.b_ld + h);
    }
  };

  const int chunks = (n + T - 1) / T;
  __syncthreads();                                 // the tile is read; the zeros are in place
  if (chunks > 0) fetch(0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int c = 0; c < chunks; ++c) {
    const int buf = c & 1, t0 = c * T, nt = min(T, n - t0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                               // chunk c has landed for all; chunk c - 1 is through, its read-outs are added
    if (c + 1 < chunks) fetch(c + 1);              // into the buffer chunk c - 1 has left
    asm volatile("cp.async.commit_group;" ::: "memory");
    float* qb = q_s + buf * T * ROW;
    float* kb = k_s + buf * T * ROW;
    const float* vb = v_s + buf * T * COLS;
    float* gb = gv_s + buf * T * ROW;
    if (VG) {
      if (tid < nt) w_s[tid] = 1.f / (1.f + expf(-b_s[buf * TS + tid]));
    } else if (tid < nt) {
      const float sp = softplus_f(a_s[buf * TS + tid] + dtb);
      g_s[tid] = expf(-A * sp);
      w_s[tid] = DELTA ? 1.f / (1.f + expf(-b_s[buf * TS + tid])) : sp;
    }
    if (p.unit_norm) {
      for (int tt = warp; tt < nt; tt += SR_THREADS / 32) {
        float* qr = qb + tt * ROW;
        float* kr = kb + tt * ROW;
        float sq = 0.f, sk = 0.f;
        for (int r = lane; r < p.dim; r += 32) { const int at = r + 4 * (r / RPL); sq += qr[at] * qr[at]; sk += kr[at] * kr[at]; }
        sq = warp_sum(sq); sk = warp_sum(sk);
        const float fq = p.q_scale / sqrtf(sq + p.unit_eps), fk = 1.f / sqrtf(sk + p.unit_eps);
        for (int r = lane; r < p.dim; r += 32) { const int at = r + 4 * (r / RPL); qr[at] *= fq; kr[at] *= fk; }
      }
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float g = VG ? 1.f : g_s[tt], w = w_s[tt], vj = vb[tt * COLS + col_local];
      float kk[RPL], qq[RPL];
#pragma unroll
      for (int i = 0; i < RPL; i += 4) {
        *reinterpret_cast<float4*>(kk + i) = *reinterpret_cast<const float4*>(kb + tt * ROW + sub * (RPL + 4) + i);
        *reinterpret_cast<float4*>(qq + i) = *reinterpret_cast<const float4*>(qb + tt * ROW + sub * (RPL + 4) + i);
      }
      if (VG) {                                    // every row decays by its own factor first; the rest is the rule with g = 1
#pragma unroll
        for (int i = 0; i < RPL; i += 4) {
          const float4 g4 = *reinterpret_cast<const float4*>(gb + tt * ROW + sub * (RPL + 4) + i);
          s[i] *= g4.x; s[i + 1] *= g4.y; s[i + 2] *= g4.z; s[i + 3] *= g4.w;
        }
      }
      float u;
      if (DELTA) {
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
        for (int i = 0; i < RPL; i += 4) {
          d0 = fmaf(s[i], kk[i], d0); d1 = fmaf(s[i + 1], kk[i + 1], d1);
          d2 = fmaf(s[i + 2], kk[i + 2], d2); d3 = fmaf(s[i + 3], kk[i + 3], d3);
        }
        float d = (d0 + d1) + (d2 + d3);
#pragma unroll
        for (int m = 1; m < SUB; m <<= 1) d += __shfl_xor_sync(0xffffffffu, d, m);
        u = w * (vj - g * d);
      } else {
        u = w * vj;
      }
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < RPL; i += 4) {
        s[i] = fmaf(g, s[i], kk[i] * u); s[i + 1] = fmaf(g, s[i + 1], kk[i + 1] * u);
        s[i + 2] = fmaf(g, s[i + 2], kk[i + 2] * u); s[i + 3] = fmaf(g, s[i + 3], kk[i + 3] * u);
        o0 = fmaf(s[i], qq[i], o0); o1 = fmaf(s[i + 1], qq[i + 1], o1);
        o2 = fmaf(s[i + 2], qq[i + 2], o2); o3 = fmaf(s[i + 3], qq[i + 3], o3);
      }
      o_s[tt * SR_THREADS + tid] = (o0 + o1) + (o2 + o3);          // [tt][col_local][sub]
    }
    __syncthreads();
    for (int i = tid; i < nt * COLS; i += SR_THREADS) {
      const int tt = i / COLS, cc = i % COLS, col = col0 + cc;
      const float* part = o_s + tt * SR_THREADS + cc * SUB;
      float o = (part[0] + part[1]) + (part[2] + part[3]);
      if (SUB >= 8) o += (part[4] + part[5]) + (part[6] + part[7]);
      if (SUB == 16) o += ((part[8] + part[9]) + (part[10] + part[11])) + ((part[12] + part[13]) + (part[14] + part[15]));
      if (col < p.vdim) p.out[(size_t)(first + t0 + tt) * p.out_ld + (size_t)h * p.vdim + col] = o + Dh * vb[tt * COLS + cc];
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                                 // the last read-outs are added: the tile is free for the state
#pragma unroll
  for (int i = 0; i < RPL; ++i) o_s[(sub * RPL + i) * COLS + (col_local + shift) % COLS] = s[i];
  __syncthreads();
  if (p.svec) {
    for (int i = tid; i < DP * (COLS / 4); i += SR_THREADS) {
      const int r = i / (COLS / 4), c = (i % (COLS / 4)) * 4, col = col0 + c;
      if (r < p.dim && col < p.vdim)
        *reinterpret_cast<float4*>(S + (size_t)r * p.vdim + col) = *reinterpret_cast<const float4*>(o_s + r * COLS + (c + TURN * (r / RPL)) % COLS);
    }
  } else {
    for (int i = tid; i < DP * COLS; i += SR_THREADS) {
      const int r = i / COLS, c = i % COLS, col = col0 + c;
      if (r < p.dim && col < p.vdim) S[(size_t)r * p.vdim + col] = o_s[r * COLS + (c + TURN * (r / RPL)) % COLS];
    }
  }
}

// Decays for every key channel, in place: a[t, h * dim + r] <- exp(-exp(A_log[h]) * softplus(a[t, h * dim + r] + dt_bias[h * dim + r])).
__global__ void channel_decay_kernel(float* __restrict__ a, long long a_ld, const float* __restrict__ A_log,
                                     const float* __restrict__ dt_bias, int n, int dim, long long total) {
  pdl_trigger();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / n;
    const int c = (int)(idx - t * n);
    float* x = a + t * a_ld + c;
    *x = expf(-expf(A_log[c / dim]) * softplus_f(*x + dt_bias[c]));
  }
}

// Norm in equal groups of a row with a gate, after a recurrence:
//   gate_first = 0:  out = y / rms_group(y) * w * act(gate)           (the gated delta rule: a group is a head)
//   gate_first = 1:  z = y * act(gate);  out = z / rms_group(z) * w     (Mamba-2: the gate comes before the norm)
// w has `wn` entries and is read at column % wn (wn = the group's size: one weight shared by the groups); no w: no weight.
// y may come in `planes` planes, `plane` elements apart, whose sum is meant (a recurrence whose CTAs share out a state's rows).
// act: 0 silu, 1 sigmoid.  One to eight warps a (row, group), by the group's size, and as many groups of a row in a CTA
// (threadIdx.y) as make it 256 threads; a group's warps add their sums of squares in warp order.
template <typename TO>
__global__ void gated_group_norm_kernel(TO* __restrict__ out, long long out_ld, const float* __restrict__ y, long long y_ld,
                                        const float* __restrict__ gate, long long gate_ld, const float* __restrict__ w, int wn,
                                        int n, int groups, int gate_first, int act, float eps, float scale, int planes, long long plane) {
  __shared__ float part[8][8];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, gy = threadIdx.y, g = blockIdx.y * blockDim.y + gy;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int gs = g < groups ? n / groups : 0;      // a group past the last has no columns, but meets the others at the barrier
  const float* yr = y + (size_t)t * y_ld + (size_t)g * gs;
  const float* gr = gate + (size_t)t * gate_ld + (size_t)g * gs;
  auto value = [&](int c) {                        // y may come in planes whose sum, in order, is meant
    float v = yr[c];
    for (int q = 1; q < planes; ++q) v += yr[(size_t)q * plane + c];
    return v;
  };
  float ss = 0.f;
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float x = value(c);
    if (gate_first) {
      const float z = gr[c];
      x *= act == 0 ? z / (1.f + expf(-z)) : 1.f / (1.f + expf(-z));
    }
    ss += x * x;
  }
  ss = warp_sum(ss);
  if (lane == 0) part[gy][warp] = ss;
  __syncthreads();
  ss = 0.f;
  for (int i = 0; i < nwarps; ++i) ss += part[gy][i];
  const float inv = 1.f / sqrtf(ss / (float)(n / groups) + eps);
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    const int col = g * gs + c;
    const float z = gr[c];
    const float a = act == 0 ? z / (1.f + expf(-z)) : 1.f / (1.f + expf(-z));
    const float x = value(c);
    const float wc = w ? w[col % wn] : 1.f;
    const float r = gate_first ? (x * a) * inv * wc : x * inv * wc * a;
    out[(size_t)t * out_ld + col] = from_f32<TO>(r * scale);
  }
}

}  // namespace lb

LB_EXPORT int lb_state_recurrence(int delta, const float* q, long long q_ld, const float* k, long long k_ld, const float* v,
                                  long long v_ld, const float* a, long long a_ld, const float* b, long long b_ld,
                                  const float* A_log, const float* dt_bias, const float* D, float* state, float* out,
                                  long long out_ld, const int* cu_tokens, const int* slots, int num_seqs, int heads, int groups,
                                  int dim, int vdim, int unit_norm, float q_scale, float unit_eps, int single_tokens, int rows_decay,
                                  int wide_lanes, cudaStream_t stream) {
  LB_CHECK_ARG(!rows_decay || delta, "state_recurrence: a decay for every state row comes with the delta rule");
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
  auto aligned = [](const float* x, long long ld) { return ((uintptr_t)x % 16 == 0) && ld % 4 == 0; };
  p.vec = dim % 4 == 0 && vdim % 4 == 0 && aligned(q, q_ld) && aligned(k, k_ld) && aligned(v, v_ld);
  p.svec = vdim % 4 == 0 && (uintptr_t)state % 16 == 0;
  p.avec = rows_decay && dim % 4 == 0 && aligned(a, a_ld);
#define LB_SR1(RPL, SUB, TOK)                                                                                       \
  do {                                                                                                              \
    const size_t smem = (size_t)lb::sr_smem_floats(RPL, SUB, TOK) * sizeof(float);                                  \
    static bool cfg = false;                                                                                        \
    if (!cfg) {                                                                                                     \
      cudaFuncSetAttribute(lb::state_recurrence_kernel<true, RPL, SUB, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      cudaFuncSetAttribute(lb::state_recurrence_kernel<false, RPL, SUB, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      cfg = true;                                                                                                   \
    }                                                                                                               \
    dim3 grid((vdim + lb::SR_THREADS / SUB - 1) / (lb::SR_THREADS / SUB), heads, num_seqs), block(lb::SR_THREADS); \
    if (rows_decay) {                                                                                               \
      const size_t smem_g = (size_t)lb::sr_smem_floats(RPL, SUB, TOK, true) * sizeof(float);                        \
      static bool cfg_g = false;                                                                                    \
      if (!cfg_g) {                                                                                                 \
        cudaFuncSetAttribute(lb::state_recurrence_kernel<true, RPL, SUB, TOK, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_g); \
        cfg_g = true;                                                                                               \
      }                                                                                                             \
      lb::launch(lb::state_recurrence_kernel<true, RPL, SUB, TOK, true>, grid, block, smem_g, stream, p);           \
    } else if (delta) lb::launch(lb::state_recurrence_kernel<true, RPL, SUB, TOK>, grid, block, smem, stream, p);          \
    else lb::launch(lb::state_recurrence_kernel<false, RPL, SUB, TOK>, grid, block, smem, stream, p);               \
  } while (0)
  // a step of single tokens stages one token at a time: the same sums in the same order, a fifth of the shared memory
#define LB_SR(RPL, SUB)                                                                                             \
  do {                                                                                                              \
    if (single_tokens) LB_SR1(RPL, SUB, 1);                                                                         \
    else LB_SR1(RPL, SUB, lb::SR_TOKENS);                                                                           \
  } while (0)
  // Eight rows a lane: the fewer rows a lane walks a token, the shorter the path from one token to the next (the sums
  // over a column's lanes are a butterfly of log2(SUB) shuffles), which is what a step with few sequences waits for:
  // a prompt of 2048 tokens with 16 heads of 128 x 128 (128 CTAs) takes a third less time.  A step that fills every SM
  // several times over (many single tokens; 32 such heads) is bound by the instructions issued, of which sixteen rows a
  // lane need fewer (10 to 15 % faster); `wide_lanes` asks for that layout.  The two add a column's terms in another order.
  if (dim <= 32) LB_SR(8, 4);
  else if (dim <= 64) { if (wide_lanes) LB_SR(16, 4); else LB_SR(8, 8); }
  else if (dim <= 128) { if (wide_lanes) LB_SR(16, 8); else LB_SR(8, 16); }
  else { if (wide_lanes) LB_SR(32, 8); else LB_SR(16, 16); }
#undef LB_SR1
#undef LB_SR
  LB_CHECK_LAUNCH("state_recurrence");
  return 0;
}

LB_EXPORT int lb_channel_decay(float* a, long long a_ld, const float* A_log, const float* dt_bias, int num_rows, int heads, int dim,
                               cudaStream_t stream) {
  LB_CHECK_ARG(a && A_log && dt_bias && num_rows >= 0 && heads > 0 && dim > 0 && a_ld >= (long long)heads * dim, "channel_decay: bad arguments");
  if (num_rows == 0) return 0;
  const long long total = (long long)num_rows * heads * dim;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  lb::launch(lb::channel_decay_kernel, dim3(blocks), dim3(256), 0, stream, a, a_ld, A_log, dt_bias, heads * dim, dim, total);
  LB_CHECK_LAUNCH("channel_decay");
  return 0;
}

LB_EXPORT int lb_gated_group_norm(void* out, int out_dtype, long long out_ld, const float* y, long long y_ld, const float* gate,
                                  long long gate_ld, const float* w, int wn, int num_rows, int n, int groups, int gate_first,
                                  int act, float eps, float scale, int planes, long long plane, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && planes >= 1, "gated_group_norm: bad dtype or plane count");
  LB_CHECK_ARG(out && y && gate && num_rows >= 0 && n > 0 && groups > 0 && n % groups == 0 && (!w || wn > 0) && (act == 0 || act == 1),
               "gated_group_norm: bad arguments rows=%d n=%d groups=%d", num_rows, n, groups);
  if (num_rows == 0) return 0;
  LB_CHECK_ARG(groups <= 65535, "gated_group_norm: %d groups", groups);
  const int gs = n / groups;
  const int warps = gs >= 1024 ? 8 : gs >= 512 ? 4 : gs >= 256 ? 2 : 1;     // by the group's size alone
  int per_cta = 8 / warps;                                                  // groups of a row in one CTA
  if (per_cta > groups) per_cta = groups;
  LB_CHECK_ARG((groups + per_cta - 1) / per_cta <= 65535, "gated_group_norm: %d groups", groups);
  LB_DISPATCH_DTYPE(out_dtype, TO, {
    lb::launch(lb::gated_group_norm_kernel<TO>, dim3(num_rows, (groups + per_cta - 1) / per_cta), dim3(warps * 32, per_cta), 0, stream,
               (TO*)out, out_ld, y, y_ld, gate, gate_ld, w, wn > 0 ? wn : 1, n, groups, gate_first, act, eps, scale, planes, plane);
  })
  LB_CHECK_LAUNCH("gated_group_norm");
  return 0;
}
