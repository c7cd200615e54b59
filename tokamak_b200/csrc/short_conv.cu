// A short causal convolution over time on every channel, across the steps of a request:
//
//   y[t, c] = (x[t, c] if add_input) + bias[c] + sum_j taps[c, j] x[t - (K - 1) + j, c]      (then silu, if asked)
//
// with zeros before the start of the sequence.  The inputs of the K - 1 positions before a step's first
// token are the request's *tail*, a float32 record [K - 1, channels] in its slot (oldest row first,
// cleared when the slot is handed out).  The sum is float32; the rows come as float32 (the residual
// stream), in the activation type, or as the partial sums of a split-K product.
//
// Kernels: the convolution, a row of blocks per token and a thread per channel (steps of many tokens:
// short_conv_rows_kernel below), and the kernel that moves the tail on
// to the step's last K - 1 inputs, one thread per (request, channel).  Where every request brings a single
// token the first does both (a thread is then the only one that touches its channel of its slot).
#include "common.cuh"
#include "stacked_input.cuh"

namespace tk {

constexpr int kConvMaxTaps = 8;

struct ShortConvParams {
  StackedInput in;          // rows in the activation type or as partial sums, unless rows_f32 is given
  const float* rows_f32;    // [n_tokens, in.row_stride] float32, or null
  int in_off;               // first column of the channels in a row
  const float* taps;        // [channels, K]
  const float* bias;        // [channels] or null
  float* tail;              // [n_slots, K - 1, channels]
  void* out;                // [n_tokens, channels], activation type or float32
  const int* tok_req;
  const int* req_q_start;
  const int* req_q_len;
  const int* req_slot;
  int* err;
  int n_tokens, n_reqs, n_slots, channels, taps_n;
  int add_input, act, out_f32, move_tail;
};

template <typename T>
__device__ __forceinline__ float conv_ld(const ShortConvParams& p, int row, int c) {
  const size_t off = (size_t)row * p.in.row_stride + p.in_off + c;
  return p.rows_f32 != nullptr ? p.rows_f32[off] : stacked_ld<T>(p.in, off);
}

// V neighbouring channels of a row (V = 4: the address is a multiple of four elements)
template <typename T, int V>
__device__ __forceinline__ void conv_ld_v(const ShortConvParams& p, int row, int c, float (&v)[V]) {
  const size_t off = (size_t)row * p.in.row_stride + p.in_off + c;
  if (V == 4 && p.rows_f32 != nullptr) {
    const float4 x = *reinterpret_cast<const float4*>(p.rows_f32 + off);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  } else if (V == 4 && p.in.x != nullptr && sizeof(T) == 2) {
    const uint2 x = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)p.in.x + off);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
    v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
  } else {
#pragma unroll
    for (int e = 0; e < V; ++e) v[e] = conv_ld<T>(p, row, c + e);
  }
}

// One block row per token (blockIdx.x), a thread V neighbouring channels of it.
template <typename T, int V>
__global__ void short_conv_kernel(ShortConvParams p) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (c >= p.channels) return;
  const int r = p.tok_req[t];
  if (r < 0 || r >= p.n_reqs) { set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
  const int slot = p.req_slot[r], q0 = p.req_q_start[r];
  const int K = p.taps_n, i = t - q0;
  if ((K > 1 && (slot < 0 || slot >= p.n_slots)) || q0 > t) { set_error(p.err, kErrRequest, t, slot, q0); return; }
  float* tail = p.tail + (size_t)slot * (K - 1) * p.channels + c;
  const float* w = p.taps + (size_t)c * K;
  float x[kConvMaxTaps][V];
#pragma unroll
  for (int j = 0; j < kConvMaxTaps; ++j) {
    if (j < K) {
      const int s = i - (K - 1) + j;                // place among the step's tokens of the request
      if (s >= 0) {
        conv_ld_v<T, V>(p, q0 + s, c, x[j]);
      } else if (V == 4) {
        const float4 v = *reinterpret_cast<const float4*>(tail + (size_t)(K - 1 + s) * p.channels);
        x[j][0] = v.x; x[j][1] = v.y; x[j][2] = v.z; x[j][3] = v.w;
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) x[j][e] = tail[(size_t)(K - 1 + s) * p.channels + e];
      }
    }
  }
  float y[V];
#pragma unroll
  for (int e = 0; e < V; ++e) {
    float acc = p.bias != nullptr ? p.bias[c + e] : 0.0f, cur = 0.0f;
#pragma unroll
    for (int j = 0; j < kConvMaxTaps; ++j) {
      if (j < K) acc += w[e * K + j] * x[j][e];
      if (j == K - 1) cur = x[j][e];
    }
    if (p.add_input) acc += cur;
    if (p.act == 1) acc = acc / (1.0f + expf(-acc));
    y[e] = acc;
  }
  const size_t idx = (size_t)t * p.channels + c;
  if (V == 4 && (p.out_f32 || sizeof(T) == 4)) {
    *reinterpret_cast<float4*>((float*)p.out + idx) = make_float4(y[0], y[1], y[2], y[3]);
  } else if (V == 4) {
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(y[0], y[1]);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(y[2], y[3]);
    *reinterpret_cast<uint2*>((__nv_bfloat16*)p.out + idx) = o;
  } else {
#pragma unroll
    for (int e = 0; e < V; ++e) {
      if (p.out_f32) ((float*)p.out)[idx + e] = y[e]; else ((T*)p.out)[idx + e] = from_f32<T>(y[e]);
    }
  }
  if (p.move_tail) {
#pragma unroll
    for (int j = 1; j < kConvMaxTaps; ++j) {
      if (j < K) {
#pragma unroll
        for (int e = 0; e < V; ++e) tail[(size_t)(j - 1) * p.channels + e] = x[j][e];
      }
    }
  }
}

// For steps with many tokens: a thread forms four neighbouring channels of kConvRowTokens consecutive
// tokens.  The rows it needs are read once (a token's window overlaps its neighbours'), and the chain of
// dependent loads that leads to a token's request is walked once for all of them.  A tap that lies before
// its request's first token of this step comes from the request's tail.  Sums in the order of the kernel above.
constexpr int kConvRowTokens = 8;

template <typename T, int M>       // M: the most taps this instance takes
__global__ void short_conv_rows_kernel(ShortConvParams p) {
  constexpr int V = 4, TT = kConvRowTokens;
  pdl_trigger();
  pdl_wait();
  const int t0 = blockIdx.x * TT, c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (c >= p.channels) return;
  const int K = p.taps_n;
  int q0s[TT], slots[TT];
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) {
    q0s[tt] = 0x7fffffff; slots[tt] = 0;            // a token that is skipped
    const int t = t0 + tt;
    if (t < p.n_tokens) {
      const int r = p.tok_req[t];
      if (r < 0 || r >= p.n_reqs) { set_error(p.err, kErrRequest, t, r, p.n_reqs); continue; }
      const int slot = p.req_slot[r], q0 = p.req_q_start[r];
      if ((K > 1 && (slot < 0 || slot >= p.n_slots)) || q0 > t || q0 < 0) { set_error(p.err, kErrRequest, t, slot, q0); continue; }
      q0s[tt] = q0; slots[tt] = slot;
    }
  }
  // rows[i] is row t0 - (M - 1) + i of the step
  float rows[TT + M - 1][V];
#pragma unroll
  for (int i = 0; i < TT + M - 1; ++i) {
    const int g = t0 - (M - 1) + i;
    if (i >= M - K && g >= 0 && g < p.n_tokens) {
      conv_ld_v<T, V>(p, g, c, rows[i]);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) rows[i][e] = 0.0f;
    }
  }
  // wd[e][d]: the tap that weighs the input d positions back
  float wd[V][M], bias[V];
#pragma unroll
  for (int e = 0; e < V; ++e) {
    bias[e] = p.bias != nullptr ? p.bias[c + e] : 0.0f;
#pragma unroll
    for (int d = 0; d < M; ++d) wd[e][d] = d < K ? p.taps[(size_t)(c + e) * K + (K - 1 - d)] : 0.0f;
  }
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) {
    const int t = t0 + tt, q0 = q0s[tt];
    if (q0 == 0x7fffffff) continue;
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = bias[e];
#pragma unroll
    for (int d = M - 1; d >= 0; --d) {
      if (d < K) {
        float x[V];
        if (t - d >= q0) {
#pragma unroll
          for (int e = 0; e < V; ++e) x[e] = rows[tt - d + M - 1][e];
        } else {
          const float4 v = *reinterpret_cast<const float4*>(
              p.tail + ((size_t)slots[tt] * (K - 1) + (t - q0) + (K - 1 - d)) * p.channels + c);
          x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
        }
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] += wd[e][d] * x[e];
      }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) {
      if (p.add_input) acc[e] += rows[tt + M - 1][e];
      if (p.act == 1) acc[e] = acc[e] / (1.0f + expf(-acc[e]));
    }
    const size_t idx = (size_t)t * p.channels + c;
    if (p.out_f32 || sizeof(T) == 4) {
      *reinterpret_cast<float4*>((float*)p.out + idx) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(acc[0], acc[1]);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(acc[2], acc[3]);
      *reinterpret_cast<uint2*>((__nv_bfloat16*)p.out + idx) = o;
    }
  }
}

template <typename T>
__global__ void short_conv_tail_kernel(ShortConvParams p) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)p.n_reqs * p.channels) return;
  const int r = (int)(idx / p.channels), c = (int)(idx - (long long)r * p.channels);
  const int slot = p.req_slot[r], q0 = p.req_q_start[r], n = p.req_q_len[r];
  if (slot < 0 || slot >= p.n_slots || q0 < 0 || n < 0 || q0 + n > p.n_tokens) {
    set_error(p.err, kErrRequest, r, slot, q0);
    return;
  }
  const int K = p.taps_n;
  float* tail = p.tail + (size_t)slot * (K - 1) * p.channels + c;
  float x[kConvMaxTaps];
#pragma unroll
  for (int j = 0; j < kConvMaxTaps - 1; ++j) {
    if (j < K - 1) {
      const int s = n - (K - 1) + j;
      x[j] = s >= 0 ? conv_ld<T>(p, q0 + s, c) : tail[(size_t)(K - 1 + s) * p.channels];
    }
  }
#pragma unroll
  for (int j = 0; j < kConvMaxTaps - 1; ++j) {
    if (j < K - 1) tail[(size_t)j * p.channels] = x[j];
  }
}

}  // namespace tk

// move_tail: 0 = leave the tail as it is, 1 = the convolution moves it on itself (every request brings one
// token), 2 = a second kernel moves it on after the convolution.
TK_API int tk_short_conv(const void* x, const float* parts, int n_parts, long long part_stride, const float* rows_f32,
                         int row_stride, int in_off, const float* taps, const float* bias, float* tail, void* out,
                         const int* tok_req, const int* req_q_start, const int* req_q_len, const int* req_slot, int* err,
                         int n_tokens, int n_reqs, int n_slots, int channels, int taps_n, int add_input, int act,
                         int out_f32, int move_tail, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0 || n_reqs <= 0) return 0;
  const int sources = (x != nullptr) + (parts != nullptr) + (rows_f32 != nullptr);
  if (sources != 1 || channels < 1 || taps_n < 1 || taps_n > tk::kConvMaxTaps || in_off < 0 ||
      in_off + channels > row_stride || (taps_n > 1 && tail == nullptr) || move_tail < 0 || move_tail > 2) {
    return (int)cudaErrorInvalidValue;
  }
  tk::ShortConvParams p;
  p.in.x = x; p.in.parts = parts; p.in.n_parts = n_parts; p.in.row_stride = row_stride; p.in.part_stride = part_stride;
  p.rows_f32 = rows_f32; p.in_off = in_off; p.taps = taps; p.bias = bias; p.tail = tail; p.out = out;
  p.tok_req = tok_req; p.req_q_start = req_q_start; p.req_q_len = req_q_len; p.req_slot = req_slot; p.err = err;
  p.n_tokens = n_tokens; p.n_reqs = n_reqs; p.n_slots = n_slots; p.channels = channels; p.taps_n = taps_n;
  p.add_input = add_input; p.act = act; p.out_f32 = out_f32; p.move_tail = move_tail == 1;
  cudaError_t e = cudaSuccess;
  // four channels a thread where every row, the tail and the result can be addressed 16 bytes at a time
  const bool quads = channels % 4 == 0 && in_off % 4 == 0 && row_stride % 4 == 0 && part_stride % 4 == 0 &&
                     (((uintptr_t)x | (uintptr_t)parts | (uintptr_t)rows_f32 | (uintptr_t)tail | (uintptr_t)out) & 15u) == 0;
  if (quads && n_tokens >= 64 && move_tail != 1) {
    const int threads = channels / 4 >= 128 ? 128 : (channels / 4 + 31) / 32 * 32;
    const dim3 grid((unsigned)((n_tokens + tk::kConvRowTokens - 1) / tk::kConvRowTokens),
                    (unsigned)((channels / 4 + threads - 1) / threads));
    if (taps_n <= 4) {
      TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::short_conv_rows_kernel<T, 4>, grid, dim3(threads), 0, stream, p));
    } else {
      TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::short_conv_rows_kernel<T, tk::kConvMaxTaps>, grid, dim3(threads), 0,
                                                 stream, p));
    }
  } else {
    const int threads = channels >= 256 ? 256 : (channels + 31) / 32 * 32;
    const dim3 grid((unsigned)n_tokens, (unsigned)((channels + threads - 1) / threads));
    TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::short_conv_kernel<T, 1>, grid, dim3(threads), 0, stream, p));
  }
  if (e != cudaSuccess || move_tail != 2 || taps_n == 1) return (int)e;
  const long long lanes = (long long)n_reqs * channels;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::short_conv_tail_kernel<T>, dim3((unsigned)((lanes + 255) / 256)),
                                             dim3(256), 0, stream, p));
  return (int)e;
}
