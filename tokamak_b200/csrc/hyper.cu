// A residual stream in several copies ("hyper-connections") and the layer norm that reads it.
//
// The stream is S float32 copies x_1 .. x_S of every token row, [S, n_tokens, width].  A sublayer reads
// one row  u = sum_s read[s] x_s  through a norm, and what it returns, y, is written back to all copies at
// once, from the old ones:
//
//   x_t <- sum_s mix[s, t] x_s + mult * write[t] * y          (mix is indexed [from, to])
//
// One kernel does, for a row, the write of the sublayer before (if one is pending), the read of the next
// one and its norm, so that the copies cross memory once per sublayer:
//
//   norm = layer norm:  (u - mean(u)) / sqrt(mean((u - mean(u))^2) + eps) * w + b
//
// S = 1 with mix = [[1]], write = [1], read = [1] is the plain residual sum  x <- x + mult * y  followed by
// the norm.  With a list of rows only those rows are read and normed and the stream is left as it is (the
// model's last norm on the rows whose logits are wanted; `read` null there: the copies are summed).
// Everything is float32; the normed row is rounded once on store.  One block per row.
#include "common.cuh"
#include "stacked_input.cuh"

namespace tk {

constexpr int kHyperMaxStreams = 8;

struct HyperParams {
  float* streams;           // [S, n_tokens, width]
  StackedInput branch;      // the pending sublayer output, or x and parts both null
  const float* mix;         // [S, S] (from, to); null: the identity
  const float* write;       // [S]; null: ones
  const float* read;        // [S]; null: ones (the sum of the copies)
  const float* norm_w;      // [width]; null: no normed row is produced
  const float* norm_b;      // [width] or null
  void* out;                // [n_rows, width] in the activation type
  float* sum_out;           // [n_rows, width] float32 or null: the read row itself, before the norm
  const int* rows;          // [n_rows] or null: every row, and the stream is updated
  int n_rows, n_tokens, width, n_streams;
  float mult, eps;
};

template <typename T>
__global__ void hyper_mix_norm_kernel(HyperParams p) {
  extern __shared__ float u_row[];          // the read row
  __shared__ float scratch[32];
  __shared__ float s_mix[kHyperMaxStreams * kHyperMaxStreams], s_write[kHyperMaxStreams], s_read[kHyperMaxStreams];
  pdl_trigger();
  const int S = p.n_streams;
  if (threadIdx.x < S * S) {
    const int a = threadIdx.x / S, b = threadIdx.x - a * S;
    s_mix[threadIdx.x] = p.mix != nullptr ? p.mix[threadIdx.x] : (a == b ? 1.0f : 0.0f);
  }
  if (threadIdx.x < S) {
    s_write[threadIdx.x] = (p.write != nullptr ? p.write[threadIdx.x] : 1.0f) * p.mult;
    s_read[threadIdx.x] = p.read != nullptr ? p.read[threadIdx.x] : 1.0f;
  }
  pdl_wait();
  __syncthreads();
  const int t = p.rows != nullptr ? p.rows[blockIdx.x] : blockIdx.x;
  if (t < 0 || t >= p.n_tokens) return;
  const bool pending = p.branch.x != nullptr || p.branch.parts != nullptr;
  const bool store = pending && p.rows == nullptr;
  const size_t copy = (size_t)p.n_tokens * p.width;
  float* x = p.streams + (size_t)t * p.width;
  float sum = 0.0f;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) {
    float old[kHyperMaxStreams];
#pragma unroll
    for (int s = 0; s < kHyperMaxStreams; ++s) old[s] = s < S ? x[(size_t)s * copy + c] : 0.0f;
    float u = 0.0f;
    if (pending) {
      const float y = stacked_ld<T>(p.branch, (size_t)t * p.branch.row_stride + c);
#pragma unroll
      for (int to = 0; to < kHyperMaxStreams; ++to) {
        if (to < S) {
          float v = 0.0f;
#pragma unroll
          for (int s = 0; s < kHyperMaxStreams; ++s) if (s < S) v += s_mix[s * S + to] * old[s];
          v += s_write[to] * y;
          if (store) x[(size_t)to * copy + c] = v;
          u += s_read[to] * v;
        }
      }
    } else {
#pragma unroll
      for (int s = 0; s < kHyperMaxStreams; ++s) if (s < S) u += s_read[s] * old[s];
    }
    u_row[c] = u;
    sum += u;
    if (p.sum_out != nullptr) p.sum_out[(size_t)blockIdx.x * p.width + c] = u;
  }
  if (p.norm_w == nullptr) return;
  const float mean = block_sum(sum, scratch) / (float)p.width;
  float dev = 0.0f;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) { const float d = u_row[c] - mean; dev += d * d; }
  const float rstd = rsqrtf(block_sum(dev, scratch) / (float)p.width + p.eps);
  T* out = (T*)p.out + (size_t)blockIdx.x * p.width;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) {
    out[c] = from_f32<T>((u_row[c] - mean) * rstd * p.norm_w[c] + (p.norm_b != nullptr ? p.norm_b[c] : 0.0f));
  }
}

constexpr int kHyperChunks = 4;     // most pieces of four columns a thread keeps in registers

// The same for rows whose width is a multiple of 4 and at most 16 columns a thread: 16-byte accesses, the read
// row stays in registers between the passes (sum, squared deviations, store), the norm's weight and bias are
// asked for before the wait for the kernel in front.  The sums per column are formed in the same order as in
// the kernel above, so both give the same stream.
// K: pieces a thread holds; SMAX: the most copies the unrolled loops cover (both keep the registers to what is used).
template <typename T, int K, int SMAX>
__global__ void __launch_bounds__(512) hyper_mix_norm_vec_kernel(HyperParams p) {
  __shared__ float scratch[32];
  __shared__ float s_mix[kHyperMaxStreams * kHyperMaxStreams], s_write[kHyperMaxStreams], s_read[kHyperMaxStreams];
  pdl_trigger();
  const int S = p.n_streams;
  const int chunks = p.width >> 2;
  float4 w4[K], b4[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    w4[k] = b4[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (i < chunks && p.norm_w != nullptr) {
      w4[k] = reinterpret_cast<const float4*>(p.norm_w)[i];
      if (p.norm_b != nullptr) b4[k] = reinterpret_cast<const float4*>(p.norm_b)[i];
    }
  }
  if (threadIdx.x < S * S) {
    const int a = threadIdx.x / S, b = threadIdx.x - a * S;
    s_mix[threadIdx.x] = p.mix != nullptr ? p.mix[threadIdx.x] : (a == b ? 1.0f : 0.0f);
  }
  if (threadIdx.x < S) {
    s_write[threadIdx.x] = (p.write != nullptr ? p.write[threadIdx.x] : 1.0f) * p.mult;
    s_read[threadIdx.x] = p.read != nullptr ? p.read[threadIdx.x] : 1.0f;
  }
  pdl_wait();
  __syncthreads();
  const int t = p.rows != nullptr ? p.rows[blockIdx.x] : blockIdx.x;
  if (t < 0 || t >= p.n_tokens) return;
  const bool pending = p.branch.x != nullptr || p.branch.parts != nullptr;
  const bool store = pending && p.rows == nullptr;
  const size_t copy = (size_t)p.n_tokens * p.width;
  float* x = p.streams + (size_t)t * p.width;
  float4 u[K];
  float sum = 0.0f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    u[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (i >= chunks) continue;
    float4 old[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
      if (s < S) old[s] = *reinterpret_cast<const float4*>(x + (size_t)s * copy + 4 * i);
    }
    if (pending) {
      const float4 y = stacked_ld4<T>(p.branch, (size_t)t * p.branch.row_stride + 4 * i);
#pragma unroll
      for (int to = 0; to < SMAX; ++to) {
        if (to < S) {
          float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
          for (int s = 0; s < SMAX; ++s) {
            if (s < S) {
              const float m = s_mix[s * S + to];
              v.x += m * old[s].x; v.y += m * old[s].y; v.z += m * old[s].z; v.w += m * old[s].w;
            }
          }
          const float wr = s_write[to], rd = s_read[to];
          v.x += wr * y.x; v.y += wr * y.y; v.z += wr * y.z; v.w += wr * y.w;
          if (store) *reinterpret_cast<float4*>(x + (size_t)to * copy + 4 * i) = v;
          u[k].x += rd * v.x; u[k].y += rd * v.y; u[k].z += rd * v.z; u[k].w += rd * v.w;
        }
      }
    } else {
#pragma unroll
      for (int s = 0; s < SMAX; ++s) {
        if (s < S) {
          const float rd = s_read[s];
          u[k].x += rd * old[s].x; u[k].y += rd * old[s].y; u[k].z += rd * old[s].z; u[k].w += rd * old[s].w;
        }
      }
    }
    sum += (u[k].x + u[k].y) + (u[k].z + u[k].w);
    if (p.sum_out != nullptr) *reinterpret_cast<float4*>(p.sum_out + (size_t)blockIdx.x * p.width + 4 * i) = u[k];
  }
  if (p.norm_w == nullptr) return;
  const float mean = block_sum(sum, scratch) / (float)p.width;
  float dev = 0.0f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    if ((int)(threadIdx.x + k * blockDim.x) < chunks) {
      u[k].x -= mean; u[k].y -= mean; u[k].z -= mean; u[k].w -= mean;
      dev += (u[k].x * u[k].x + u[k].y * u[k].y) + (u[k].z * u[k].z + u[k].w * u[k].w);
    }
  }
  const float rstd = rsqrtf(block_sum(dev, scratch) / (float)p.width + p.eps);
  T* out = (T*)p.out + (size_t)blockIdx.x * p.width;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < chunks) {
      st4<T>(out + 4 * i, make_float4(u[k].x * rstd * w4[k].x + b4[k].x, u[k].y * rstd * w4[k].y + b4[k].y,
                                            u[k].z * rstd * w4[k].z + b4[k].z, u[k].w * rstd * w4[k].w + b4[k].w));
    }
  }
}

// logits <- cap * tanh(scale * logits / cap)  (cap <= 0: only the scale), float32 in place
__global__ void logits_scale_cap_kernel(float* __restrict__ logits, long long n, float scale, float cap) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float z = logits[i] * scale;
  logits[i] = cap > 0.0f ? cap * tanhf(z / cap) : z;
}

}  // namespace tk

TK_API int tk_hyper_mix_norm(float* streams, const void* y, const float* y_parts, int n_parts, long long part_stride,
                             int y_row_stride, const float* mix, const float* write, const float* read,
                             const float* norm_w, const float* norm_b, void* out, float* sum_out, const int* rows,
                             int n_rows, int n_tokens, int width, int n_streams, float mult, float eps, int dtype,
                             cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (streams == nullptr || width < 1 || n_streams < 1 || n_streams > tk::kHyperMaxStreams ||
      (y != nullptr && y_parts != nullptr) || (norm_w != nullptr && out == nullptr) ||
      (size_t)width * sizeof(float) > 200 * 1024) {
    return (int)cudaErrorInvalidValue;
  }
  tk::HyperParams p;
  p.streams = streams;
  p.branch.x = y; p.branch.parts = y_parts; p.branch.n_parts = n_parts; p.branch.row_stride = y_row_stride;
  p.branch.part_stride = part_stride;
  p.mix = mix; p.write = write; p.read = read; p.norm_w = norm_w; p.norm_b = norm_b; p.out = out; p.sum_out = sum_out;
  p.rows = rows; p.n_rows = n_rows; p.n_tokens = n_tokens; p.width = width; p.n_streams = n_streams;
  p.mult = mult; p.eps = eps;
  cudaError_t e = cudaSuccess;
  // rows of a multiple of four columns (and a branch whose rows start at such multiples): 16-byte accesses, the
  // row in registers; few rows get a thread per piece of four columns, many rows two pieces a thread
  const int chunks = width / 4;
  const bool aligned = width % 4 == 0 && ((y == nullptr && y_parts == nullptr) || y_row_stride % 4 == 0);
  if (aligned && chunks <= 512 * tk::kHyperChunks) {
    int threads = ((n_rows <= 296 ? chunks : (chunks + 1) / 2) + 31) / 32 * 32;
    if (threads > 512) threads = 512;
    if (threads < 64) threads = 64;
    const int per_thread = (chunks + threads - 1) / threads;
#define TK_HYPER_VEC(T, K, SMAX) \
    e = tk::launch(tk::hyper_mix_norm_vec_kernel<T, K, SMAX>, dim3((unsigned)n_rows), dim3(threads), 0, stream, p)
#define TK_HYPER_VEC_K(T, SMAX)                                    \
    do {                                                           \
      if (per_thread <= 1) { TK_HYPER_VEC(T, 1, SMAX); }           \
      else if (per_thread <= 2) { TK_HYPER_VEC(T, 2, SMAX); }      \
      else { TK_HYPER_VEC(T, 4, SMAX); }                           \
    } while (0)
#define TK_HYPER_VEC_S(T)                                          \
    do {                                                           \
      if (n_streams <= 2) { TK_HYPER_VEC_K(T, 2); } else { TK_HYPER_VEC_K(T, 8); }   \
    } while (0)
    if (dtype == tk::kF32) { TK_HYPER_VEC_S(float); } else if (dtype == tk::kBF16) { TK_HYPER_VEC_S(__nv_bfloat16); }
    else return (int)cudaErrorInvalidValue;
#undef TK_HYPER_VEC_S
#undef TK_HYPER_VEC_K
#undef TK_HYPER_VEC
    return (int)e;
  }
  const size_t smem = (size_t)width * sizeof(float);
  int threads = n_rows <= 64 ? 512 : 256;
  while (threads > 64 && threads / 2 >= width) threads /= 2;
#define TK_HYPER(T)                                                                                                    \
  do {                                                                                                                 \
    if (smem > 48 * 1024) {                                                                                            \
      e = cudaFuncSetAttribute(tk::hyper_mix_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      if (e != cudaSuccess) return (int)e;                                                                             \
    }                                                                                                                  \
    e = tk::launch(tk::hyper_mix_norm_kernel<T>, dim3((unsigned)n_rows), dim3(threads), smem, stream, p);              \
  } while (0)
  if (dtype == tk::kF32) { TK_HYPER(float); } else if (dtype == tk::kBF16) { TK_HYPER(__nv_bfloat16); }
  else return (int)cudaErrorInvalidValue;
#undef TK_HYPER
  return (int)e;
}

TK_API int tk_logits_scale_cap(float* logits, long long n, float scale, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  return (int)tk::launch(tk::logits_scale_cap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, logits,
                         n, scale, cap);
}
