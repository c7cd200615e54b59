// Preparation of queries, keys and values for attention without rotation: biases, an RMS norm of the
// *whole* query projection of a token (all heads at once, one weight per channel) and of the whole key
// projection, and the write of keys and values into their pages.
//
//   q = (z_q + b_q) * rsqrt(mean_all((z_q + b_q)^2) + eps) * w_q,   k likewise,   v = z_v + b_v
//
// Statistics and sums are float32; the result is rounded once on store.  One block per token; a row of
// the input holds the query heads, then the key heads, then the value heads.
#include "common.cuh"
#include "stacked_input.cuh"

namespace tk {

struct QkvRowNormParams {
  StackedInput in;
  int q_off, k_off, v_off;
  const float* q_bias; const float* k_bias; const float* v_bias;   // or null
  const float* q_norm; const float* k_norm;                        // or null: no norm
  void* q_out;              // [n_tokens, n_q_heads * k_dim]
  void* k_cache;            // [num_pages, n_kv_heads, page_size, k_dim]
  void* v_cache;            // [num_pages, n_kv_heads, page_size, v_dim]
  const int* positions; const int* tok_req; const int* req_slot; const int* block_table;
  const int* req_q_len; const int* req_kv_len;
  int* err;
  int n_tokens, n_reqs, n_q_heads, n_kv_heads, k_dim, v_dim, page_size, max_pages, num_pages;
  float eps;
};

template <typename T>
__global__ void qkv_rownorm_kernel(QkvRowNormParams p) {
  extern __shared__ float row[];           // the biased query row, then the biased key row
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int nq = p.n_q_heads * p.k_dim, nk = p.n_kv_heads * p.k_dim, nv = p.n_kv_heads * p.v_dim;
  const size_t base = (size_t)t * p.in.row_stride;
  // where the token's keys and values go: a chain of dependent loads, started before the rows are read so
  // that it is over when the rows are
  const int pos = p.positions[t], r = p.tok_req[t];
  const bool known = pos >= 0 && r >= 0 && r < p.n_reqs;
  const int pidx = known ? pos / p.page_size : 0, slot = known ? pos - pidx * p.page_size : 0;
  const int page = (known && pidx < p.max_pages) ? p.block_table[(size_t)p.req_slot[r] * p.max_pages + pidx] : -1;
  int kv_len = 0, q_len = 0;
  if (known && p.req_kv_len != nullptr) { kv_len = p.req_kv_len[r]; q_len = p.req_q_len[r]; }
  float ssq = 0.0f, ssk = 0.0f;
  for (int c = threadIdx.x; c < nq; c += blockDim.x) {
    const float x = stacked_ld<T>(p.in, base + p.q_off + c) + (p.q_bias ? p.q_bias[c] : 0.0f);
    row[c] = x; ssq += x * x;
  }
  for (int c = threadIdx.x; c < nk; c += blockDim.x) {
    const float x = stacked_ld<T>(p.in, base + p.k_off + c) + (p.k_bias ? p.k_bias[c] : 0.0f);
    row[nq + c] = x; ssk += x * x;
  }
  ssq = block_sum(ssq, scratch);
  ssk = block_sum(ssk, scratch);
  const float rq = p.q_norm ? rsqrtf(ssq / (float)nq + p.eps) : 1.0f;
  const float rk = p.k_norm ? rsqrtf(ssk / (float)nk + p.eps) : 1.0f;
  T* q = (T*)p.q_out + (size_t)t * nq;
  for (int c = threadIdx.x; c < nq; c += blockDim.x) q[c] = from_f32<T>(row[c] * rq * (p.q_norm ? p.q_norm[c] : 1.0f));

  if (pos < 0) { if (threadIdx.x == 0) set_error(p.err, kErrPosition, t, pos, 0); return; }
  if (r < 0 || r >= p.n_reqs) { if (threadIdx.x == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
  if (page < 0 || page >= p.num_pages) { if (threadIdx.x == 0) set_error(p.err, kErrPage, t, pidx, page); return; }
  // the request's last token of this step clears the rest of a page that was begun in this step, so
  // that a live page never holds stale values behind the last position
  int zero_rows = 0;
  if (p.req_kv_len != nullptr) {
    if (pos == kv_len - 1 && pos - slot >= kv_len - q_len) zero_rows = p.page_size - 1 - slot;
  }
  for (int c = threadIdx.x; c < nk; c += blockDim.x) {
    const int h = c / p.k_dim, e = c - h * p.k_dim;
    T* dst = (T*)p.k_cache + (((size_t)page * p.n_kv_heads + h) * p.page_size + slot) * p.k_dim + e;
    dst[0] = from_f32<T>(row[nq + c] * rk * (p.k_norm ? p.k_norm[c] : 1.0f));
    for (int z = 1; z <= zero_rows; ++z) dst[(size_t)z * p.k_dim] = from_f32<T>(0.0f);
  }
  for (int c = threadIdx.x; c < nv; c += blockDim.x) {
    const int h = c / p.v_dim, e = c - h * p.v_dim;
    T* dst = (T*)p.v_cache + (((size_t)page * p.n_kv_heads + h) * p.page_size + slot) * p.v_dim + e;
    dst[0] = from_f32<T>(stacked_ld<T>(p.in, base + p.v_off + c) + (p.v_bias ? p.v_bias[c] : 0.0f));
    for (int z = 1; z <= zero_rows; ++z) dst[(size_t)z * p.v_dim] = from_f32<T>(0.0f);
  }
}

}  // namespace tk

TK_API int tk_qkv_rownorm(const void* x, const float* parts, int n_parts, long long part_stride, int row_stride,
                          int q_off, int k_off, int v_off, const float* q_bias, const float* k_bias,
                          const float* v_bias, const float* q_norm, const float* k_norm, void* q_out, void* k_cache,
                          void* v_cache, const int* positions, const int* tok_req, const int* req_slot,
                          const int* block_table, const int* req_q_len, const int* req_kv_len, int* err, int n_tokens,
                          int n_reqs, int n_q_heads, int n_kv_heads, int k_dim, int v_dim, int page_size, int max_pages,
                          int num_pages, float eps, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const size_t smem = (size_t)(n_q_heads + n_kv_heads) * k_dim * sizeof(float);
  if ((x == nullptr) == (parts == nullptr) || n_q_heads < 1 || n_kv_heads < 1 || k_dim < 1 || v_dim < 1 ||
      smem > 200 * 1024) {
    return (int)cudaErrorInvalidValue;
  }
  tk::QkvRowNormParams p;
  p.in.x = x; p.in.parts = parts; p.in.n_parts = n_parts; p.in.row_stride = row_stride; p.in.part_stride = part_stride;
  p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.q_bias = q_bias; p.k_bias = k_bias; p.v_bias = v_bias;
  p.q_norm = q_norm; p.k_norm = k_norm; p.q_out = q_out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.positions = positions; p.tok_req = tok_req; p.req_slot = req_slot; p.block_table = block_table;
  p.req_q_len = req_q_len; p.req_kv_len = req_kv_len; p.err = err;
  p.n_tokens = n_tokens; p.n_reqs = n_reqs; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.k_dim = k_dim;
  p.v_dim = v_dim; p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages; p.eps = eps;
  cudaError_t e = cudaSuccess;
  // a step of few tokens fills few SMs: more threads a row then, so that a row is one round of loads
  const int threads = n_tokens <= 64 ? 1024 : 256;
#define TK_ROWNORM(T)                                                                                                   \
  do {                                                                                                                  \
    if (smem > 48 * 1024) {                                                                                             \
      e = cudaFuncSetAttribute(tk::qkv_rownorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
      if (e != cudaSuccess) return (int)e;                                                                              \
    }                                                                                                                   \
    e = tk::launch(tk::qkv_rownorm_kernel<T>, dim3((unsigned)n_tokens), dim3(threads), smem, stream, p);                \
  } while (0)
  if (dtype == tk::kF32) { TK_ROWNORM(float); } else if (dtype == tk::kBF16) { TK_ROWNORM(__nv_bfloat16); }
  else return (int)cudaErrorInvalidValue;
#undef TK_ROWNORM
  return (int)e;
}
