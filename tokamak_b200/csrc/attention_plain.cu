// Paged attention, general form: any mix of prompt portions and single decoded
// tokens, any head_dim up to 1024, any group size, float32 or bfloat16 pages.
//
// One thread block per (token, query head).  The query at absolute position p
// sees keys [max(0, p - window + 1), p] of its own request (window <= 0: all),
// the causal rule of the reference for a chunk at start_pos > 0
// (src/tokamak/model/step_context.py:93-102) and its decode length mask
// (src/tokamak/kernels/paged_attention.py:97-123).  Scores are scaled by
// softmax_scale, the softmax is an online one with float32 running maximum,
// normaliser and accumulator (paged_attention.py:111-123,139-151).  This is the
// kernel of the float32 path and of every shape the tiled kernels refuse.
//
// Options that other designs use: values of another size than keys (v_dim), a soft cap on the
// scaled scores (score <- cap * tanh(score / cap), cap <= 0: none), and a sink per query head:
// a learned number whose exponential joins the softmax denominator once, with no key and no
// value, neither scaled nor capped.  Queries may be float32 over bfloat16 pages and are addressed by
// a token and a head stride; key and value rows have strides of their own, so that values which are the
// leading elements of the key rows (a latent cache) are read from the key pages.  Two more: a chunked
// mask (chunk > 0: a query sees only the keys of its own block of `chunk` positions, blocks counted from
// position 0 of the sequence) and a distance bias (slopes: one float per query head; the score of key j
// for the query at position p loses slope * (p - j), after scale and cap).  Or a distance bias from a table
// (dist_bias: [n_q_heads, dist_len] float32): the key at distance n = p - j gains dist_bias[h, min(n, dist_len - 1)],
// after scale and cap (a learned bias by bucketed distance, the buckets laid out distance by distance).
#include "common.cuh"

namespace tk {

constexpr int kPlainWarps = 4;

struct AttnParams {
  const void* q;            // element (t, h, e) at t * q_tok_stride + h * q_head_stride + e
  void* out;                // [n_tokens, n_q_heads, v_dim]
  const void* k_cache;      // [num_pages, n_kv_heads, page_size, k_stride]: a row's first head_dim elements
  const void* v_cache;      // [num_pages, n_kv_heads, page_size, v_stride]: a row's first v_dim elements
  const float* sinks;       // [n_q_heads] or null
  const float* slopes;      // [n_q_heads] or null
  const float* dist_bias;   // [n_q_heads, dist_len] or null
  int dist_len;
  const int* positions;     // [n_tokens]
  const int* tok_req;       // [n_tokens]
  const int* req_slot;      // [n_reqs]
  const int* block_table;   // [n_slots, max_pages]
  const int* items;         // [n_items] token indices to process, or null for all tokens
  int* err;
  int n_tokens, n_reqs, n_q_heads, n_kv_heads, head_dim;
  int page_size, max_pages, num_pages, window, v_dim, chunk;
  long long q_tok_stride, q_head_stride;
  int k_stride, v_stride;
  float scale, softcap;
};

// TQ: element type of the queries, T: of pages and output; kPerLane: elements of a head per lane.
template <typename TQ, typename T, int kPerLane>
__global__ void attention_plain_kernel(AttnParams p) {
  constexpr int kPlainMaxPerLane = kPerLane;
  pdl_trigger();
  pdl_wait();
  __shared__ float s_m[kPlainWarps];
  __shared__ float s_l[kPlainWarps];
  __shared__ float s_acc[kPlainWarps][kPlainMaxPerLane * 32];

  const int t = p.items ? p.items[blockIdx.x] : blockIdx.x;
  const int hq = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int d = p.head_dim;
  const int dv = p.v_dim;
  const int group = p.n_q_heads / p.n_kv_heads;
  const int hkv = hq / group;
  const int pos = p.positions[t];
  const int r = p.tok_req[t];
  if (pos < 0 || r < 0 || r >= p.n_reqs) {
    if (threadIdx.x == 0) set_error(p.err, pos < 0 ? kErrPosition : kErrRequest, t, pos, r);
    return;
  }
  const int* table = p.block_table + (size_t)p.req_slot[r] * p.max_pages;
  int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
  if (p.chunk > 0) lo = max(lo, pos - pos % p.chunk);
  const float slope = p.slopes != nullptr ? p.slopes[hq] : 0.0f;
  const float* dist = p.dist_bias != nullptr ? p.dist_bias + (size_t)hq * p.dist_len : nullptr;

  const TQ* qrow = (const TQ*)p.q + (size_t)t * p.q_tok_stride + (size_t)hq * p.q_head_stride;
  float qreg[kPlainMaxPerLane];
  float acc[kPlainMaxPerLane];
#pragma unroll
  for (int i = 0; i < kPlainMaxPerLane; ++i) {
    const int e = i * 32 + lane;
    qreg[i] = (e < d) ? to_f32<TQ>(qrow[e]) * p.scale : 0.0f;
    acc[i] = 0.0f;
  }
  float m = -INFINITY, l = 0.0f;
  // the sink is one more term of the denominator: the first warp starts from it
  if (p.sinks != nullptr && warp == 0) { m = p.sinks[hq]; l = 1.0f; }
  const float inv_cap = p.softcap > 0.0f ? 1.0f / p.softcap : 0.0f;

  for (int j = lo + warp; j <= pos; j += kPlainWarps) {
    const int pidx = j / p.page_size;
    const int page = (pidx < p.max_pages) ? table[pidx] : -1;   // beyond the row: reported, not read
    if (page < 0 || page >= p.num_pages) {
      if (lane == 0) set_error(p.err, kErrPage, t, pidx, page);
      break;
    }
    const size_t row = ((size_t)page * p.n_kv_heads + hkv) * p.page_size + (j % p.page_size);
    const T* krow = (const T*)p.k_cache + row * p.k_stride;
    const T* vrow = (const T*)p.v_cache + row * p.v_stride;
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < kPlainMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < d) dot += qreg[i] * to_f32<T>(krow[e]);
    }
    dot = warp_sum(dot);
    if (p.softcap > 0.0f) dot = p.softcap * tanhf(dot * inv_cap);
    dot -= slope * (float)(pos - j);
    if (dist != nullptr) dot += dist[min(pos - j, p.dist_len - 1)];
    const float m_new = fmaxf(m, dot);
    const float corr = expf(m - m_new);   // m = -inf on the first key: exp(-inf) = 0
    const float pj = expf(dot - m_new);
    l = l * corr + pj;
#pragma unroll
    for (int i = 0; i < kPlainMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < dv) acc[i] = acc[i] * corr + pj * to_f32<T>(vrow[e]);
    }
    m = m_new;
  }

  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < kPlainMaxPerLane; ++i) s_acc[warp][i * 32 + lane] = acc[i];
  __syncthreads();

  if (warp == 0) {
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPlainWarps; ++w) m_all = fmaxf(m_all, s_m[w]);
    float l_all = 0.0f;
    float f[kPlainWarps];
#pragma unroll
    for (int w = 0; w < kPlainWarps; ++w) {
      f[w] = (s_m[w] == -INFINITY) ? 0.0f : expf(s_m[w] - m_all);
      l_all += s_l[w] * f[w];
    }
    const float inv = 1.0f / l_all;   // the query always sees its own key, so l_all > 0
    T* orow = (T*)p.out + ((size_t)t * p.n_q_heads + hq) * dv;
#pragma unroll
    for (int i = 0; i < kPlainMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < dv) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kPlainWarps; ++w) o += s_acc[w][e] * f[w];
        orow[e] = from_f32<T>(o * inv);
      }
    }
  }
}

}  // namespace tk

TK_API int tk_attention_plain(const void* q, void* out, const void* k_cache, const void* v_cache,
                              const int* positions, const int* tok_req, const int* req_slot,
                              const int* block_table, const int* items, int* err, int n_tokens, int n_reqs,
                              int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                              int max_pages, int num_pages, int window, float scale, int dtype,
                              int v_dim, float softcap, const float* sinks, int q_dtype, long long q_tok_stride,
                              long long q_head_stride, int k_stride, int v_stride, int chunk, const float* slopes,
                              const float* dist_bias, int dist_len, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (v_dim <= 0) v_dim = head_dim;
  const int widest = head_dim > v_dim ? head_dim : v_dim;
  if (head_dim < 1 || widest > 1024 || n_kv_heads < 1 || n_q_heads % n_kv_heads != 0 || n_q_heads > 65535 ||
      k_stride < head_dim || v_stride < v_dim || (q_dtype != dtype && q_dtype != tk::kF32) ||
      (dist_bias != nullptr && dist_len < 1)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::AttnParams p;
  p.q = q; p.out = out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.positions = positions; p.tok_req = tok_req; p.req_slot = req_slot; p.block_table = block_table;
  p.items = items; p.err = err; p.n_tokens = n_tokens; p.n_reqs = n_reqs; p.n_q_heads = n_q_heads;
  p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.page_size = page_size;
  p.max_pages = max_pages; p.num_pages = num_pages; p.window = window; p.scale = scale;
  p.v_dim = v_dim; p.softcap = softcap; p.sinks = sinks; p.chunk = chunk; p.slopes = slopes; p.dist_bias = dist_bias; p.dist_len = dist_len;
  p.q_tok_stride = q_tok_stride; p.q_head_stride = q_head_stride; p.k_stride = k_stride; p.v_stride = v_stride;
  dim3 grid(n_tokens, n_q_heads);
  cudaError_t e = cudaSuccess;
#define TK_PLAIN_LAUNCH(TQ, K)                                                                                   \
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::attention_plain_kernel<TQ, T, K>, grid, dim3(tk::kPlainWarps * 32), \
                                             0, stream, p))
#define TK_PLAIN_SIZES(TQ)                                   \
  do {                                                       \
    if (widest <= 128) { TK_PLAIN_LAUNCH(TQ, 4); }           \
    else if (widest <= 256) { TK_PLAIN_LAUNCH(TQ, 8); }      \
    else if (widest <= 640) { TK_PLAIN_LAUNCH(TQ, 20); }     \
    else { TK_PLAIN_LAUNCH(TQ, 32); }                        \
  } while (0)
  if (q_dtype == dtype) {
    if (dtype == tk::kF32) { TK_PLAIN_SIZES(float); } else { TK_PLAIN_SIZES(__nv_bfloat16); }
  } else {
    TK_PLAIN_SIZES(float);
  }
#undef TK_PLAIN_SIZES
#undef TK_PLAIN_LAUNCH
  return (int)e;
}
