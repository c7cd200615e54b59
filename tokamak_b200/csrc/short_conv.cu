// A short causal convolution over time on every channel, across the steps of a request:
//
//   y[t, c] = (x[t, c] if add_input) + bias[c] + sum_j taps[c, j] x[t - (K - 1) + j, c]      (then silu, if asked)
//
// with zeros before the start of the sequence.  The inputs of the K - 1 positions before a step's first
// token are the request's *tail*, a float32 record [K - 1, channels] in its slot (oldest row first,
// cleared when the slot is handed out).  The sum is float32; the rows come as float32 (the residual
// stream), in the activation type, or as the partial sums of a split-K product.
//
// Two kernels: the convolution, one thread per (token, channel), and the kernel that moves the tail on
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

template <typename T>
__global__ void short_conv_kernel(ShortConvParams p) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)p.n_tokens * p.channels) return;
  const int t = (int)(idx / p.channels), c = (int)(idx - (long long)t * p.channels);
  const int r = p.tok_req[t];
  if (r < 0 || r >= p.n_reqs) { set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
  const int slot = p.req_slot[r], q0 = p.req_q_start[r];
  const int K = p.taps_n, i = t - q0;
  if ((K > 1 && (slot < 0 || slot >= p.n_slots)) || q0 > t) { set_error(p.err, kErrRequest, t, slot, q0); return; }
  float* tail = p.tail + (size_t)slot * (K - 1) * p.channels + c;
  const float* w = p.taps + (size_t)c * K;
  float x[kConvMaxTaps];
#pragma unroll
  for (int j = 0; j < kConvMaxTaps; ++j) {
    if (j < K) {
      const int s = i - (K - 1) + j;                // place among the step's tokens of the request
      x[j] = s >= 0 ? conv_ld<T>(p, q0 + s, c) : tail[(size_t)(K - 1 + s) * p.channels];
    }
  }
  float acc = p.bias != nullptr ? p.bias[c] : 0.0f, cur = 0.0f;
#pragma unroll
  for (int j = 0; j < kConvMaxTaps; ++j) {
    if (j < K) acc += w[j] * x[j];
    if (j == K - 1) cur = x[j];
  }
  if (p.add_input) acc += cur;
  if (p.act == 1) acc = acc / (1.0f + expf(-acc));
  if (p.out_f32) ((float*)p.out)[idx] = acc; else ((T*)p.out)[idx] = from_f32<T>(acc);
  if (p.move_tail) {
#pragma unroll
    for (int j = 1; j < kConvMaxTaps; ++j) {
      if (j < K) tail[(size_t)(j - 1) * p.channels] = x[j];
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
  const long long total = (long long)n_tokens * channels;
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::short_conv_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
                                             stream, p));
  if (e != cudaSuccess || move_tail != 2 || taps_n == 1) return (int)e;
  const long long lanes = (long long)n_reqs * channels;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::short_conv_tail_kernel<T>, dim3((unsigned)((lanes + 255) / 256)),
                                             dim3(256), 0, stream, p));
  return (int)e;
}
