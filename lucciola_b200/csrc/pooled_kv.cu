// Two small steps of attention whose keys are normed over the whole projection and pooled behind a window.
//
// lb_bias_rmsnorm_cols: up to three column ranges of 32-bit rows, in place: x <- x + bias, then, where a range has a
// norm weight, x <- x / sqrt(mean(x^2) + eps) * w with the mean over the whole range (all heads of a projection at
// once, not head by head).  One CTA a token and range; the sum's order depends on the range's size alone.
//
// lb_pool_kv: the mean key and the mean value of every block of P consecutive tokens that this step completes, read
// from the pages as the cache holds them and written to a second paged cache with one entry a block (entry b at
// "position" b of its own block table).  A block b is complete in this step when its last token (b + 1) P - 1 is one
// of the step's tokens; its P tokens are then all in their pages, from this step or from steps before (the cache
// keeps at least the last P tokens).  Sums are 32-bit in the tokens' order, divided by P.
#include "common.cuh"

namespace lb {

struct ColumnRanges {
  int col[3], size[3];
  const float* bias[3];
  const float* weight[3];
};

__global__ void bias_rmsnorm_cols_kernel(float* __restrict__ x, long long ld, ColumnRanges r, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int seg = blockIdx.y;
  float* row = x + (size_t)blockIdx.x * ld + r.col[seg];
  const int n = r.size[seg];
  const float* bias = r.bias[seg];
  const float* w = r.weight[seg];
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = row[i] + (bias ? bias[i] : 0.f);
    row[i] = v;
    ss += v * v;
  }
  if (w == nullptr) return;                      // uniform over the block
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = row[i] * inv * w[i];
}

template <typename T>
__global__ void pool_kv_kernel(const T* __restrict__ k_cache, const T* __restrict__ v_cache, const int* __restrict__ table,
                               int max_pages, T* __restrict__ pool_k, T* __restrict__ pool_v, const int* __restrict__ pool_table,
                               int pool_max_pages, const int* __restrict__ cu_tokens, const int* __restrict__ context_lens,
                               int num_kv_heads, int d, int dv, int page_size, int P) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y, kvh = blockIdx.z;
  const int ctx = context_lens[s];
  const int start = ctx - (cu_tokens[s + 1] - cu_tokens[s]);
  const int b = start / P + blockIdx.x;          // the first block that can end inside the step, and those behind it
  if ((long long)(b + 1) * P > ctx) return;
  const int dest = pool_table[(size_t)s * pool_max_pages + b / page_size];
  if (dest < 0) return;
  const size_t dest_off = ((size_t)dest * num_kv_heads + kvh) * page_size + (b % page_size);
  const int* bt = table + (size_t)s * max_pages;
  for (int i = threadIdx.x; i < d + dv; i += blockDim.x) {
    const bool is_k = i < d;
    const int e = is_k ? i : i - d, width = is_k ? d : dv;
    const T* src = is_k ? k_cache : v_cache;
    float sum = 0.f;
    for (int j0 = 0; j0 < P; j0 += 8) {          // eight loads in flight, then their sum in token order
      float x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int pos = b * P + j0 + u;
        const int page = j0 + u < P ? bt[pos / page_size] : -1;
        x[u] = page >= 0 ? to_f32(src[(((size_t)page * num_kv_heads + kvh) * page_size + pos % page_size) * width + e]) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) sum += x[u];
    }
    (is_k ? pool_k : pool_v)[dest_off * width + e] = from_f32<T>(sum / (float)P);
  }
}

}  // namespace lb

LB_EXPORT int lb_bias_rmsnorm_cols(float* x, long long ld, int num_rows, int ranges, const int* col, const int* size,
                                   const float* const* bias, const float* const* weight, float eps, cudaStream_t stream) {
  LB_CHECK_ARG(x && num_rows >= 0 && ranges >= 1 && ranges <= 3 && col && size && bias && weight, "bias_rmsnorm_cols: bad arguments");
  if (num_rows == 0) return 0;
  lb::ColumnRanges r;
  int widest = 0;
  for (int i = 0; i < 3; ++i) {
    r.col[i] = i < ranges ? col[i] : 0; r.size[i] = i < ranges ? size[i] : 0;
    r.bias[i] = i < ranges ? bias[i] : nullptr; r.weight[i] = i < ranges ? weight[i] : nullptr;
    LB_CHECK_ARG(r.size[i] >= 0 && r.col[i] >= 0, "bias_rmsnorm_cols: bad range");
    if (r.size[i] > widest) widest = r.size[i];
  }
  const int threads = widest >= 2048 ? 512 : (widest >= 512 ? 256 : 128);
  lb::launch(lb::bias_rmsnorm_cols_kernel, dim3(num_rows, ranges), dim3(threads), 0, stream, x, ld, r, eps);
  LB_CHECK_LAUNCH("bias_rmsnorm_cols");
  return 0;
}

LB_EXPORT int lb_pool_kv(int dtype, const void* k_cache, const void* v_cache, const int* table, int max_pages, void* pool_k,
                         void* pool_v, const int* pool_table, int pool_max_pages, const int* cu_tokens, const int* context_lens,
                         int num_seqs, int max_blocks, int num_kv_heads, int head_dim, int v_dim, int page_size, int pool,
                         cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype), "pool_kv: bad dtype %d", dtype);
  LB_CHECK_ARG(k_cache && v_cache && table && pool_k && pool_v && pool_table && cu_tokens && context_lens, "pool_kv: null argument");
  LB_CHECK_ARG(num_seqs >= 0 && num_seqs <= 65535 && num_kv_heads > 0 && num_kv_heads <= 65535 && head_dim > 0 && v_dim > 0 &&
               page_size > 0 && pool > 0 && max_blocks >= 0, "pool_kv: bad sizes");
  if (num_seqs == 0 || max_blocks == 0) return 0;
  const int threads = head_dim + v_dim >= 256 ? 256 : 64;
  LB_DISPATCH_DTYPE(dtype, T, {
    lb::launch(lb::pool_kv_kernel<T>, dim3(max_blocks, num_seqs, num_kv_heads), dim3(threads), 0, stream, (const T*)k_cache,
               (const T*)v_cache, table, max_pages, (T*)pool_k, (T*)pool_v, pool_table, pool_max_pages, cu_tokens, context_lens,
               num_kv_heads, head_dim, v_dim, page_size, pool);
  })
  LB_CHECK_LAUNCH("pool_kv");
  return 0;
}
