// Preparation of queries, keys and values head by head, with the options that several attention
// mixers share:
//
//   biases             z <- z + b                                   (q, k, v; each may be absent)
//   head norm          x <- x / sqrt(mean_head(x^2) + eps) * w      (q and k; w of one head's size, shared by all
//                                                                    heads, or absent: unit norm)
//   query temperature  q <- q * (1 + coef * ln(floor((p + 1) / every) + 1))   at position p
//   rotation           over the first `rotary_dim` elements of every q and k head, either of neighbouring
//                      pairs (2i, 2i + 1) or of halves (i, i + rotary_dim / 2); the pair (u, w) at angle a
//                      becomes (u cos a - w sin a, w cos a + u sin a)
//   values from keys   v = the key projection (with its bias) as it was before norm and rotation; the
//                      projection then has no value columns
//
// and the write of keys and values into their pages.  Everything is float32 and rounded once on store.
// One warp per (token, head); a row of the input is a stacked projection (activation type or float32
// partial sums) in which the queries, keys and values start at q_off, k_off and v_off.
#include "common.cuh"
#include "stacked_input.cuh"

namespace tk {

constexpr int kHeadsWarps = 4;
constexpr int kHeadsMaxDim = 512;

struct QkvHeadsParams {
  StackedInput in;
  int q_off, k_off, v_off;                  // v_off < 0: values from keys
  const float* q_bias; const float* k_bias; const float* v_bias;
  const float* q_norm; const float* k_norm; // [k_dim] or null
  int head_norm;                            // 0: no norm
  float eps;
  const float2* rope_table;                 // [n_tokens, rotary_dim / 2] (cos, sin) or null
  int rotary_dim, halves;
  float temp_coef; int temp_every;          // temp_every <= 0: no temperature
  void* q_out;                              // [n_tokens, n_q_heads, k_dim]
  void* k_cache;                            // [num_pages, n_kv_heads, page_size, k_dim]
  void* v_cache;                            // [num_pages, n_kv_heads, page_size, v_dim]
  const int* positions; const int* tok_req; const int* req_slot; const int* block_table;
  const int* req_q_len; const int* req_kv_len;
  int* err;
  int n_tokens, n_reqs, n_q_heads, n_kv_heads, k_dim, v_dim, page_size, max_pages, num_pages;
};

template <typename T>
__global__ void qkv_heads_kernel(QkvHeadsParams p) {
  __shared__ float s_head[kHeadsWarps][kHeadsMaxDim];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int own_v = p.v_off >= 0 ? p.n_kv_heads : 0;
  const int heads_total = p.n_q_heads + p.n_kv_heads + own_v;
  const int t = blockIdx.x;
  const int h = blockIdx.y * kHeadsWarps + warp;
  if (h >= heads_total) return;
  int kind, head;     // 0 = q, 1 = k, 2 = v
  if (h < p.n_q_heads) { kind = 0; head = h; }
  else if (h < p.n_q_heads + p.n_kv_heads) { kind = 1; head = h - p.n_q_heads; }
  else { kind = 2; head = h - p.n_q_heads - p.n_kv_heads; }
  const int d = kind == 2 ? p.v_dim : p.k_dim;
  const int col = (kind == 0 ? p.q_off : kind == 1 ? p.k_off : p.v_off) + head * d;
  const float* bias = kind == 0 ? p.q_bias : kind == 1 ? p.k_bias : p.v_bias;
  const size_t src = (size_t)t * p.in.row_stride + col;
  const int pos = p.positions[t];
  if (pos < 0) { if (lane == 0) set_error(p.err, kErrPosition, t, pos, 0); return; }

  T* dst = nullptr;
  T* dst_v = nullptr;          // values from keys: the same head of the value pages
  int zero_rows = 0;
  if (kind == 0) {
    dst = (T*)p.q_out + ((size_t)t * p.n_q_heads + head) * d;
  } else {
    const int r = p.tok_req[t];
    if (r < 0 || r >= p.n_reqs) { if (lane == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
    const int pidx = pos / p.page_size;
    const int slot = pos - pidx * p.page_size;
    const int page = (pidx < p.max_pages) ? p.block_table[(size_t)p.req_slot[r] * p.max_pages + pidx] : -1;
    if (page < 0 || page >= p.num_pages) { if (lane == 0) set_error(p.err, kErrPage, t, pidx, page); return; }
    const size_t row = ((size_t)page * p.n_kv_heads + head) * p.page_size + slot;
    dst = (T*)(kind == 1 ? p.k_cache : p.v_cache) + row * d;
    if (kind == 1 && p.v_off < 0) dst_v = (T*)p.v_cache + row * p.v_dim;
    // the request's last token of this step clears the rest of a page that was begun in this step, so
    // that a live page never holds stale values behind the last position
    if (p.req_kv_len != nullptr) {
      const int kv_len = p.req_kv_len[r], q_len = p.req_q_len[r];
      if (pos == kv_len - 1 && pos - slot >= kv_len - q_len) zero_rows = p.page_size - 1 - slot;
    }
  }
  for (int z = 1; z <= zero_rows; ++z) {
    for (int e = lane; e < d; e += 32) {
      dst[(size_t)z * d + e] = from_f32<T>(0.0f);
      if (dst_v != nullptr) dst_v[(size_t)z * d + e] = from_f32<T>(0.0f);
    }
  }

  float* x = s_head[warp];
  float ss = 0.0f;
  for (int e = lane; e < d; e += 32) {
    const float v = stacked_ld<T>(p.in, src + e) + (bias != nullptr ? bias[head * d + e] : 0.0f);
    x[e] = v;
    ss += v * v;
    if (kind == 2) dst[e] = from_f32<T>(v);
    if (dst_v != nullptr) dst_v[e] = from_f32<T>(v);
  }
  if (kind == 2) return;
  float factor = 1.0f;
  if (p.head_norm) factor = rsqrtf(warp_sum(ss) / (float)d + p.eps);
  if (kind == 0 && p.temp_every > 0) {
    factor *= 1.0f + p.temp_coef * logf(floorf((float)(pos + 1) / (float)p.temp_every) + 1.0f);
  }
  const float* w = p.head_norm ? (kind == 0 ? p.q_norm : p.k_norm) : nullptr;
  __syncwarp();
  const int r = p.rope_table != nullptr ? p.rotary_dim : 0, half = r >> 1;
  const float2* tab = p.rope_table + (size_t)t * half;
  for (int e = lane; e < d; e += 32) {
    float v = x[e] * factor * (w != nullptr ? w[e] : 1.0f);
    if (e < r) {
      int partner, idx; bool first;
      if (p.halves) { first = e < half; partner = first ? e + half : e - half; idx = first ? e : e - half; }
      else { first = !(e & 1); partner = e ^ 1; idx = e >> 1; }
      const float o = x[partner] * factor * (w != nullptr ? w[partner] : 1.0f);
      const float2 cs = tab[idx];
      v = first ? v * cs.x - o * cs.y : v * cs.x + o * cs.y;
    }
    dst[e] = from_f32<T>(v);
  }
}

// The same with 16-byte accesses, for head sizes, column offsets and row lengths that are multiples of 4: a lane
// keeps up to four pieces of four elements of its head in registers; rotation partners are read from the
// warp's copy of the head in shared memory.  Sums and products are formed as in the kernel above.
template <typename T>
__global__ void qkv_heads_vec_kernel(QkvHeadsParams p) {
  __shared__ __align__(16) float s_head[kHeadsWarps][kHeadsMaxDim];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int own_v = p.v_off >= 0 ? p.n_kv_heads : 0;
  const int heads_total = p.n_q_heads + p.n_kv_heads + own_v;
  const int t = blockIdx.x;
  const int h = blockIdx.y * kHeadsWarps + warp;
  if (h >= heads_total) return;
  int kind, head;     // 0 = q, 1 = k, 2 = v
  if (h < p.n_q_heads) { kind = 0; head = h; }
  else if (h < p.n_q_heads + p.n_kv_heads) { kind = 1; head = h - p.n_q_heads; }
  else { kind = 2; head = h - p.n_q_heads - p.n_kv_heads; }
  const int d = kind == 2 ? p.v_dim : p.k_dim;
  const int col = (kind == 0 ? p.q_off : kind == 1 ? p.k_off : p.v_off) + head * d;
  const float* bias = kind == 0 ? p.q_bias : kind == 1 ? p.k_bias : p.v_bias;
  const size_t src = (size_t)t * p.in.row_stride + col;
  const int pos = p.positions[t];
  if (pos < 0) { if (lane == 0) set_error(p.err, kErrPosition, t, pos, 0); return; }

  T* dst = nullptr;
  T* dst_v = nullptr;
  int zero_rows = 0;
  if (kind == 0) {
    dst = (T*)p.q_out + ((size_t)t * p.n_q_heads + head) * d;
  } else {
    const int r = p.tok_req[t];
    if (r < 0 || r >= p.n_reqs) { if (lane == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
    const int pidx = pos / p.page_size;
    const int slot = pos - pidx * p.page_size;
    const int page = (pidx < p.max_pages) ? p.block_table[(size_t)p.req_slot[r] * p.max_pages + pidx] : -1;
    if (page < 0 || page >= p.num_pages) { if (lane == 0) set_error(p.err, kErrPage, t, pidx, page); return; }
    const size_t row = ((size_t)page * p.n_kv_heads + head) * p.page_size + slot;
    dst = (T*)(kind == 1 ? p.k_cache : p.v_cache) + row * d;
    if (kind == 1 && p.v_off < 0) dst_v = (T*)p.v_cache + row * p.v_dim;
    if (p.req_kv_len != nullptr) {
      const int kv_len = p.req_kv_len[r], q_len = p.req_q_len[r];
      if (pos == kv_len - 1 && pos - slot >= kv_len - q_len) zero_rows = p.page_size - 1 - slot;
    }
  }
  const int chunks = d >> 2;
  const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int z = 1; z <= zero_rows; ++z) {
    for (int i = lane; i < chunks; i += 32) {
      st4<T>(dst + (size_t)z * d + 4 * i, zero4);
      if (dst_v != nullptr) st4<T>(dst_v + (size_t)z * d + 4 * i, zero4);
    }
  }

  float* x = s_head[warp];
  float4 own[4];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = lane + 32 * k;
    own[k] = zero4;
    if (i >= chunks) continue;
    float4 v = stacked_ld4<T>(p.in, src + 4 * i);
    if (bias != nullptr) {
      const float4 b = *reinterpret_cast<const float4*>(bias + head * d + 4 * i);
      v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
    }
    own[k] = v;
    *reinterpret_cast<float4*>(x + 4 * i) = v;
    ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
    if (kind == 2) st4<T>(dst + 4 * i, v);
    if (dst_v != nullptr) st4<T>(dst_v + 4 * i, v);
  }
  if (kind == 2) return;
  float factor = 1.0f;
  if (p.head_norm) factor = rsqrtf(warp_sum(ss) / (float)d + p.eps);
  if (kind == 0 && p.temp_every > 0) {
    factor *= 1.0f + p.temp_coef * logf(floorf((float)(pos + 1) / (float)p.temp_every) + 1.0f);
  }
  const float* w = p.head_norm ? (kind == 0 ? p.q_norm : p.k_norm) : nullptr;
  __syncwarp();
  const int r = p.rope_table != nullptr ? p.rotary_dim : 0, half = r >> 1;
  const float2* tab = p.rope_table + (size_t)t * half;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = lane + 32 * k;
    if (i >= chunks) continue;
    const float4 w4 = w != nullptr ? *reinterpret_cast<const float4*>(w + 4 * i) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    float v[4] = {own[k].x * factor * w4.x, own[k].y * factor * w4.y, own[k].z * factor * w4.z, own[k].w * factor * w4.w};
    if (4 * i < r) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = 4 * i + j;
        if (e < r) {
          int partner, idx; bool first;
          if (p.halves) { first = e < half; partner = first ? e + half : e - half; idx = first ? e : e - half; }
          else { first = !(e & 1); partner = e ^ 1; idx = e >> 1; }
          const float o = x[partner] * factor * (w != nullptr ? w[partner] : 1.0f);
          const float2 cs = tab[idx];
          v[j] = first ? v[j] * cs.x - o * cs.y : v[j] * cs.x + o * cs.y;
        }
      }
    }
    st4<T>(dst + 4 * i, make_float4(v[0], v[1], v[2], v[3]));
  }
}

}  // namespace tk

TK_API int tk_qkv_heads(const void* x, const float* parts, int n_parts, long long part_stride, int row_stride,
                        int q_off, int k_off, int v_off, const float* q_bias, const float* k_bias,
                        const float* v_bias, const float* q_norm, const float* k_norm, int head_norm, float eps,
                        const float* rope_table, int rotary_dim, int halves, float temp_coef, int temp_every,
                        void* q_out, void* k_cache, void* v_cache, const int* positions, const int* tok_req,
                        const int* req_slot, const int* block_table, const int* req_q_len, const int* req_kv_len,
                        int* err, int n_tokens, int n_reqs, int n_q_heads, int n_kv_heads, int k_dim, int v_dim,
                        int page_size, int max_pages, int num_pages, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if ((x == nullptr) == (parts == nullptr) || n_q_heads < 1 || n_kv_heads < 1 || k_dim < 1 || v_dim < 1 ||
      k_dim > tk::kHeadsMaxDim || v_dim > tk::kHeadsMaxDim || rotary_dim < 0 || rotary_dim > k_dim ||
      (rotary_dim & 1) || (v_off < 0 && v_dim != k_dim)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::QkvHeadsParams p;
  p.in.x = x; p.in.parts = parts; p.in.n_parts = n_parts; p.in.row_stride = row_stride; p.in.part_stride = part_stride;
  p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.q_bias = q_bias; p.k_bias = k_bias; p.v_bias = v_bias;
  p.q_norm = q_norm; p.k_norm = k_norm; p.head_norm = head_norm; p.eps = eps;
  p.rope_table = (const float2*)rope_table; p.rotary_dim = rotary_dim; p.halves = halves;
  p.temp_coef = temp_coef; p.temp_every = temp_every;
  p.q_out = q_out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.positions = positions; p.tok_req = tok_req; p.req_slot = req_slot; p.block_table = block_table;
  p.req_q_len = req_q_len; p.req_kv_len = req_kv_len; p.err = err;
  p.n_tokens = n_tokens; p.n_reqs = n_reqs; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.k_dim = k_dim;
  p.v_dim = v_dim; p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages;
  const int heads_total = n_q_heads + n_kv_heads + (v_off >= 0 ? n_kv_heads : 0);
  const dim3 grid((unsigned)n_tokens, (unsigned)((heads_total + tk::kHeadsWarps - 1) / tk::kHeadsWarps));
  cudaError_t e = cudaSuccess;
  const bool vec = k_dim % 4 == 0 && v_dim % 4 == 0 && row_stride % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 &&
                   (v_off < 0 || v_off % 4 == 0);
  if (vec) {
    TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::qkv_heads_vec_kernel<T>, grid, dim3(tk::kHeadsWarps * 32), 0, stream, p));
    return (int)e;
  }
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::qkv_heads_kernel<T>, grid, dim3(tk::kHeadsWarps * 32), 0, stream, p));
  return (int)e;
}
