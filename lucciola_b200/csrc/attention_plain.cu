// Plain paged attention: one warp per (query token, query head), keys visited
// in their order in the sequence, everything in 32-bit.  It serves the 32-bit
// path of the engine and is the kernel beside which the fast bfloat16 kernels
// are tested.  It takes any head size up to 512, any head counts and group
// sizes, any page size, whole prompts, portions and single decoded tokens alike.
//
// Formulas as in lucciola: kv head = q head / (nq / nkv)
// (src/kernels/attention_paged.cu:68), score = (q . k) * scale, key j allowed
// iff j <= pos (src/kernels/flash_attention.cu:183-225), online softmax with
// m, l, o and out = o / l (src/kernels/flash_attention.cu:246-298, 311-347).
// A sliding window, which lucciola does not have, adds j > pos - window.
// Keys outside the allowed range are never read, so what a reused page still
// holds cannot reach a sum.
//
// Two more things lucciola does not have.  Values may have another size than keys (v_dim; the value pool is
// then [page][kv_head][slot][v_dim]).  And a linear distance bias: with `slopes` (one 32-bit number a query
// head) the score of key j for the query at position i is (q . k) * scale - slopes[h] * (i - j).
//
// Three more options.  A capped score: s <- softcap * tanh(s / softcap).  A sink: with `sinks` (one 32-bit number a
// query head) the softmax's denominator also holds exp(sinks[h]), which has no key and no value.  And pooled
// blocks behind the window: with pool = P > 0 the query at position i also sees entry b of a second paged cache (one
// entry for every P tokens, at "position" b of its own block table) for every b with (b + 1) P - 1 <= i - window,
// in the same softmax; the entries are the means that lb_pool_kv writes.
//
// And chunks: with chunk = C > 0 positions are cut into runs of C counted from the sequence's start, and the query at
// position i sees the keys floor(i / C) * C .. i only (beside a window, whichever starts later).
#include "common.cuh"

namespace lb {

struct PlainAttnParams {
  const void* q; void* out; const void* k_cache; const void* v_cache;
  const int* positions; const int* token_seq; const int* block_table;
  int num_q_heads, num_kv_heads, head_dim, page_size, max_pages, window;
  float scale;
  int v_dim;               // size of a value head
  const float* slopes;     // optional [num_q_heads]: distance bias
  float softcap;           // 0: scores are not capped
  const float* sinks;      // optional [num_q_heads]
  int pool;                // 0: no pooled blocks; P: one pooled entry for every P tokens
  const void* pool_k; const void* pool_v; const int* pool_table; int pool_max_pages;
  int chunk;               // 0: none; C: the query at position i sees no key before floor(i / C) * C
};

template <typename T, int DPL>
__global__ void plain_attention_kernel(PlainAttnParams p) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int t = blockIdx.y;
  const int h = blockIdx.x * nwarps + warp;
  if (h >= p.num_q_heads) return;
  const int d = p.head_dim, dv = p.v_dim;
  const float slope = p.slopes ? p.slopes[h] : 0.f;
  const int kvh = h / (p.num_q_heads / p.num_kv_heads);
  float* qs = smem + (size_t)warp * d;
  const T* q = (const T*)p.q + ((size_t)t * p.num_q_heads + h) * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_f32(q[i]);
  __syncwarp();

  const int pos = p.positions[t];
  const int* bt = p.block_table + (size_t)p.token_seq[t] * p.max_pages;
  int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  if (p.chunk > 0) lo = max(lo, pos - pos % p.chunk);
  const T* kc = (const T*)p.k_cache;
  const T* vc = (const T*)p.v_cache;

  float m = -INFINITY, l = 0.f;
  float o[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) o[i] = 0.f;

  // keys j0 .. j1 - 1 of one paged cache, 32 at a time (a lane a key), through the online softmax
  auto visit = [&](const T* kc, const T* vc, const int* bt, int j0, int j1, bool biased) {
    for (int base = j0; base < j1; base += 32) {
      const int j = base + lane;
      const bool valid = j < j1;
      long long off = -1;                        // the key's place in its pool, in heads
      float s = -INFINITY;
      if (valid) {
        const int page = bt[j / p.page_size];
        if (page >= 0) {
          off = ((long long)page * p.num_kv_heads + kvh) * p.page_size + (j % p.page_size);
          const T* k = kc + off * d;
          float acc = 0.f;
          for (int i = 0; i < d; ++i) acc += qs[i] * to_f32(k[i]);
          s = acc * p.scale;
          if (biased) s -= slope * (float)(pos - j);
          if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
        }
      }
      const float m_new = fmaxf(m, warp_max(s));
      if (m_new == -INFINITY) continue;          // no key of this pass has a page: uniform over the warp
      const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
      const float pj = (off >= 0) ? expf(s - m_new) : 0.f;
      l = l * alpha + warp_sum(pj);
#pragma unroll
      for (int i = 0; i < DPL; ++i) o[i] *= alpha;
      const int n = min(32, j1 - base);
      for (int jj = 0; jj < n; ++jj) {
        const float pv = __shfl_sync(0xffffffffu, pj, jj);
        const long long voff = __shfl_sync(0xffffffffu, off, jj);
        if (voff < 0) continue;  // uniform over the warp
        const T* v = vc + voff * dv;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          const int dim = lane + 32 * i;
          if (dim < dv) o[i] += pv * to_f32(v[dim]);
        }
      }
      m = m_new;
    }
  };
  visit(kc, vc, bt, lo, pos + 1, true);
  if (p.pool > 0 && p.window > 0) {
    const int nb = (pos - p.window + 1) / p.pool;          // blocks that end at or before pos - window (negative: none)
    if (nb > 0)
      visit((const T*)p.pool_k, (const T*)p.pool_v, p.pool_table + (size_t)p.token_seq[t] * p.pool_max_pages, 0, nb, false);
  }
  if (p.sinks) {
    const float sink = p.sinks[h];
    const float m_new = fmaxf(m, sink);
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * alpha + expf(sink - m_new);
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] *= alpha;
    m = m_new;
  }
  T* out = (T*)p.out + ((size_t)t * p.num_q_heads + h) * dv;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int dim = lane + 32 * i;
    if (dim < dv) out[dim] = from_f32<T>(o[i] * inv);
  }
}

template <typename T>
int launch_plain(const PlainAttnParams& p, int num_tokens, cudaStream_t stream) {
  const int warps = 4;
  dim3 grid((p.num_q_heads + warps - 1) / warps, num_tokens);
  const size_t smem = (size_t)warps * p.head_dim * sizeof(float);
  const int dpl = (p.v_dim + 31) / 32;
  if (dpl <= 1) launch(plain_attention_kernel<T, 1>, grid, dim3(warps * 32), smem, stream, p);
  else if (dpl <= 2) launch(plain_attention_kernel<T, 2>, grid, dim3(warps * 32), smem, stream, p);
  else if (dpl <= 4) launch(plain_attention_kernel<T, 4>, grid, dim3(warps * 32), smem, stream, p);
  else if (dpl <= 8) launch(plain_attention_kernel<T, 8>, grid, dim3(warps * 32), smem, stream, p);
  else launch(plain_attention_kernel<T, 16>, grid, dim3(warps * 32), smem, stream, p);
  return 0;
}

}  // namespace lb

LB_EXPORT int lb_attention_plain(int dtype, const void* q, void* out, const void* k_cache,
                                 const void* v_cache, const int* positions, const int* token_seq,
                                 const int* block_table, int num_tokens, int num_q_heads,
                                 int num_kv_heads, int head_dim, int page_size, int max_pages,
                                 int window, float scale, int v_dim, const float* slopes, float softcap,
                                 const float* sinks, int pool, const void* pool_k, const void* pool_v, const int* pool_table,
                                 int pool_max_pages, int chunk, cudaStream_t stream) {
  LB_CHECK_ARG(chunk >= 0 && (chunk == 0 || pool == 0), "attention_plain: chunks of %d keys (and no pooled blocks with them)", chunk);
  LB_CHECK_ARG(pool == 0 || (pool > 0 && window > 0 && pool_k && pool_v && pool_table && pool_max_pages > 0),
               "attention_plain: pooled blocks need a window, the pooled cache and its block table");
  LB_CHECK_ARG(softcap >= 0.f, "attention_plain: a cap of %f", (double)softcap);
  if (v_dim <= 0) v_dim = head_dim;
  LB_CHECK_ARG(v_dim <= 512, "attention_plain: value size %d not in 1..512", v_dim);
  LB_CHECK_ARG(lb::valid_dtype(dtype), "attention_plain: bad dtype %d", dtype);
  LB_CHECK_ARG(head_dim > 0 && head_dim <= 512, "attention_plain: head_dim %d not in 1..512", head_dim);
  LB_CHECK_ARG(num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0,
               "attention_plain: %d query heads are not a multiple of %d kv heads", num_q_heads,
               num_kv_heads);
  LB_CHECK_ARG(page_size > 0 && max_pages > 0 && window >= 0, "attention_plain: bad page size or window");
  LB_CHECK_ARG(num_tokens <= 65535, "attention_plain: at most 65535 tokens a step, got %d", num_tokens);
  if (num_tokens == 0) return 0;
  lb::PlainAttnParams p;
  p.q = q; p.out = out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.positions = positions; p.token_seq = token_seq; p.block_table = block_table;
  p.num_q_heads = num_q_heads; p.num_kv_heads = num_kv_heads; p.head_dim = head_dim;
  p.page_size = page_size; p.max_pages = max_pages; p.window = window; p.scale = scale; p.v_dim = v_dim; p.slopes = slopes;
  p.softcap = softcap; p.sinks = sinks; p.pool = pool; p.pool_k = pool_k; p.pool_v = pool_v; p.pool_table = pool_table;
  p.pool_max_pages = pool_max_pages; p.chunk = chunk;
  LB_DISPATCH_DTYPE(dtype, T, { lb::launch_plain<T>(p, num_tokens, stream); })
  LB_CHECK_LAUNCH("attention_plain");
  return 0;
}
