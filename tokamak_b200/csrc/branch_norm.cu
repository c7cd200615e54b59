// A branch that is normalised before it joins the residual stream:
//
//   y = branch * rsqrt(mean(branch^2) + eps_b) * post_w (* layer_scale)
//   x = resid + y                      (written back to resid unless `rows` selects rows)
//   out = x * rsqrt(mean(x^2) + eps_n) * next_w          (when a norm follows)
//   out = x                                              (next_w null: the next sublayer reads the stream itself)
//
// in one pass: the norm after a sublayer, the per-channel layer scale, the 32-bit residual sum
// and the norm in front of the next sublayer.  Statistics, sums and the residual stream are
// float32; `out` is rounded once to the activation type.  The branch comes in the activation
// type or as float32 partial sums [parts, tokens, hidden] of a split-K product.
//
// Either norm may work in groups: the row is split into equal consecutive parts and each is divided by
// its own root mean square (branch_norm_add_groups_kernel; one group is the plain norm).  That kernel also
// takes a row without a branch: the norm in front alone.
#include "common.cuh"
#include "group_norm.cuh"

namespace tk {

template <typename T>
__global__ void branch_norm_add_kernel(float* __restrict__ resid, const T* __restrict__ branch,
                                       const float* __restrict__ parts, int n_parts, size_t part_stride,
                                       const float* __restrict__ post_w, const float* __restrict__ layer_scale,
                                       const float* __restrict__ next_w, T* __restrict__ out,
                                       const int* __restrict__ rows, int hidden, float eps_b, float eps_n) {
  extern __shared__ float row[];          // the branch, then the new residual row
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* x = resid + (size_t)r * hidden;
  float ss = 0.0f;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
    float b;
    if (branch != nullptr) {
      b = to_f32<T>(branch[(size_t)r * hidden + h]);
    } else {
      b = 0.0f;
      for (int s = 0; s < n_parts; ++s) b += parts[(size_t)s * part_stride + (size_t)r * hidden + h];
    }
    row[h] = b;
    ss += b * b;
  }
  ss = block_sum(ss, scratch);
  const float rstd_b = rsqrtf(ss / (float)hidden + eps_b);
  float ss2 = 0.0f;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
    float y = row[h] * rstd_b;
    if (post_w != nullptr) y *= post_w[h];
    if (layer_scale != nullptr) y *= layer_scale[h];
    const float v = x[h] + y;
    if (rows == nullptr) x[h] = v;
    row[h] = v;
    ss2 += v * v;
  }
  if (out == nullptr) return;
  T* o = out + (size_t)i * hidden;
  if (next_w == nullptr) {
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = from_f32<T>(row[h]);
    return;
  }
  ss2 = block_sum(ss2, scratch);
  const float rstd = rsqrtf(ss2 / (float)hidden + eps_n);
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = from_f32<T>(row[h] * rstd * next_w[h]);
}

// The general form with groups: the row lies in shared memory, a warp takes a group at a time.
template <typename T>
__global__ void branch_norm_add_groups_kernel(float* __restrict__ resid, const T* __restrict__ branch,
                                              const float* __restrict__ parts, int n_parts, size_t part_stride,
                                              const float* __restrict__ post_w, const float* __restrict__ layer_scale,
                                              const float* __restrict__ next_w, T* __restrict__ out,
                                              const int* __restrict__ rows, int hidden, float eps_b, float eps_n,
                                              int groups_b, int groups_n) {
  extern __shared__ float row[];          // the branch, then the new residual row; behind it the groups' statistics
  float* rstd = row + hidden;
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* x = resid + (size_t)r * hidden;
  const bool has_branch = branch != nullptr || parts != nullptr;
  if (has_branch) {
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
      float b;
      if (branch != nullptr) {
        b = to_f32<T>(branch[(size_t)r * hidden + h]);
      } else {
        b = 0.0f;
        for (int s = 0; s < n_parts; ++s) b += parts[(size_t)s * part_stride + (size_t)r * hidden + h];
      }
      row[h] = b;
    }
    group_rstd(row, hidden, groups_b, eps_b, rstd);
  }
  const int size_b = hidden / groups_b;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
    float v = x[h];
    if (has_branch) {
      float y = row[h] * rstd[h / size_b];
      if (post_w != nullptr) y *= post_w[h];
      if (layer_scale != nullptr) y *= layer_scale[h];
      v += y;
      if (rows == nullptr) x[h] = v;
    }
    row[h] = v;
  }
  if (out == nullptr) return;
  T* o = out + (size_t)i * hidden;
  if (next_w == nullptr) {
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = from_f32<T>(row[h]);
    return;
  }
  group_rstd(row, hidden, groups_n, eps_n, rstd);
  const int size_n = hidden / groups_n;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = from_f32<T>(row[h] * rstd[h / size_n] * next_w[h]);
}

// Four neighbouring elements at once (the address is a multiple of four elements).
template <typename T> __device__ __forceinline__ float4 ld4(const T* p);
template <> __device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
template <typename T> __device__ __forceinline__ void st4(T* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  uint2 o;
  *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = o;
}

// The same for rows whose length is a multiple of 4: a thread keeps kChunks pieces of four elements
// in registers through all three steps, so a row is read once and nothing goes through shared memory;
// the weights, which no kernel writes, are on their way before the kernel in front has finished.
// With a few rows (decoding) the kernel is three memory latencies long instead of a loop of them.
template <typename T, int kChunks>
__global__ void __launch_bounds__(512) branch_norm_add_vec_kernel(float* __restrict__ resid, const T* __restrict__ branch,
                                           const float* __restrict__ parts, int n_parts, size_t part_stride,
                                           const float* __restrict__ post_w, const float* __restrict__ layer_scale,
                                           const float* __restrict__ next_w, T* __restrict__ out,
                                           const int* __restrict__ rows, int hidden, float eps_b, float eps_n) {
  __shared__ float scratch[32];
  pdl_trigger();
  const float4 ones = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
  float4 w[kChunks], nw[kChunks];
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int h = (threadIdx.x + c * blockDim.x) * 4;
    w[c] = ones; nw[c] = ones;
    if (h < hidden) {
      if (post_w != nullptr) w[c] = ld4<float>(post_w + h);
      if (layer_scale != nullptr) {
        const float4 l = ld4<float>(layer_scale + h);
        w[c].x *= l.x; w[c].y *= l.y; w[c].z *= l.z; w[c].w *= l.w;
      }
      if (out != nullptr && next_w != nullptr) nw[c] = ld4<float>(next_w + h);
    }
  }
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* x = resid + (size_t)r * hidden;
  float4 b[kChunks], xv[kChunks];
  float ss = 0.0f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int h = (threadIdx.x + c * blockDim.x) * 4;
    b[c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f); xv[c] = b[c];
    if (h < hidden) {
      xv[c] = ld4<float>(x + h);
      if (branch != nullptr) {
        b[c] = ld4<T>(branch + (size_t)r * hidden + h);
      } else {
        const float* src = parts + (size_t)r * hidden + h;
        for (int s = 0; s < n_parts; ++s) {
          const float4 v = ld4<float>(src + (size_t)s * part_stride);
          b[c].x += v.x; b[c].y += v.y; b[c].z += v.z; b[c].w += v.w;
        }
      }
      ss += b[c].x * b[c].x + b[c].y * b[c].y + b[c].z * b[c].z + b[c].w * b[c].w;
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd_b = rsqrtf(ss / (float)hidden + eps_b);
  float ss2 = 0.0f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int h = (threadIdx.x + c * blockDim.x) * 4;
    // (branch * rstd) * (post_w * layer_scale): the two weights were multiplied on the way in
    float4 y = make_float4(b[c].x * rstd_b, b[c].y * rstd_b, b[c].z * rstd_b, b[c].w * rstd_b);
    if (post_w != nullptr || layer_scale != nullptr) { y.x *= w[c].x; y.y *= w[c].y; y.z *= w[c].z; y.w *= w[c].w; }
    xv[c].x += y.x; xv[c].y += y.y; xv[c].z += y.z; xv[c].w += y.w;
    if (h < hidden) {
      if (rows == nullptr) st4<float>(x + h, xv[c]);
      ss2 += xv[c].x * xv[c].x + xv[c].y * xv[c].y + xv[c].z * xv[c].z + xv[c].w * xv[c].w;
    }
  }
  if (out == nullptr) return;
  // without a norm in front of the next sublayer the row goes out as it is (every thread takes the same branch)
  const float rstd = next_w != nullptr ? rsqrtf(block_sum(ss2, scratch) / (float)hidden + eps_n) : 1.0f;
  T* o = out + (size_t)i * hidden;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int h = (threadIdx.x + c * blockDim.x) * 4;
    if (h < hidden) {
      st4<T>(o + h, make_float4(xv[c].x * rstd * nw[c].x, xv[c].y * rstd * nw[c].y, xv[c].z * rstd * nw[c].z,
                                xv[c].w * rstd * nw[c].w));
    }
  }
}

}  // namespace tk

TK_API int tk_branch_norm_add(float* resid, const void* branch, const float* parts, int n_parts,
                              long long part_stride, const float* post_w, const float* layer_scale,
                              const float* next_w, void* out, const int* rows, int n_rows, int hidden,
                              float eps_b, float eps_n, int groups_b, int groups_n, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const bool grouped = groups_b > 1 || groups_n > 1 || (branch == nullptr && parts == nullptr);
  if (hidden < 1 || hidden > 12288 || (branch != nullptr && parts != nullptr) || groups_b < 1 || groups_n < 1 ||
      hidden % groups_b || hidden % groups_n) {
    return (int)cudaErrorInvalidValue;
  }
  cudaError_t e = cudaSuccess;
  if (grouped) {
    // few rows fill few SMs: more threads a row then (a group's sum is a warp's in either shape, the same bits)
    const int threads = hidden >= 4096 && n_rows <= 64 ? 1024 : hidden >= 2048 && n_rows <= 64 ? 512 : hidden >= 1024 ? 256 : 128;
    const int most = groups_b > groups_n ? groups_b : groups_n;
    const size_t smem = (size_t)(hidden + most) * sizeof(float);
    if (smem > 96 * 1024) return (int)cudaErrorInvalidValue;
#define TK_BRANCH_NORM_GROUPS(T)                                                                                       \
    do {                                                                                                               \
      if (smem > 48 * 1024) {                                                                                          \
        e = cudaFuncSetAttribute(tk::branch_norm_add_groups_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                 (int)smem);                                                                           \
        if (e != cudaSuccess) return (int)e;                                                                           \
      }                                                                                                                \
      e = tk::launch(tk::branch_norm_add_groups_kernel<T>, dim3((unsigned)n_rows), dim3(threads), smem, stream, resid, \
                     (const T*)branch, parts, n_parts, (size_t)part_stride, post_w, layer_scale, next_w, (T*)out,      \
                     rows, hidden, eps_b, eps_n, groups_b, groups_n);                                                  \
    } while (0)
    if (dtype == tk::kF32) { TK_BRANCH_NORM_GROUPS(float); }
    else if (dtype == tk::kBF16) { TK_BRANCH_NORM_GROUPS(__nv_bfloat16); }
    else return (int)cudaErrorInvalidValue;
#undef TK_BRANCH_NORM_GROUPS
    return (int)e;
  }
  if (hidden % 4 == 0) {
    const int quads = hidden / 4;
    const int threads = quads >= 512 ? 512 : (quads + 31) / 32 * 32;
    const int chunks = (quads + threads - 1) / threads;        // at most 6: hidden <= 12288
#define TK_BRANCH_NORM_VEC(K)                                                                                         \
    TK_DISPATCH_DTYPE(dtype, T,                                                                                      \
                      e = tk::launch(tk::branch_norm_add_vec_kernel<T, K>, dim3((unsigned)n_rows), dim3(threads), 0, \
                                     stream, resid, (const T*)branch, parts, n_parts, (size_t)part_stride, post_w,   \
                                     layer_scale, next_w, (T*)out, rows, hidden, eps_b, eps_n))
    if (chunks <= 1) { TK_BRANCH_NORM_VEC(1); }
    else if (chunks <= 2) { TK_BRANCH_NORM_VEC(2); }
    else if (chunks <= 4) { TK_BRANCH_NORM_VEC(4); }
    else { TK_BRANCH_NORM_VEC(8); }
#undef TK_BRANCH_NORM_VEC
    return (int)e;
  }
  const int threads = hidden >= 1024 ? 256 : 128;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::branch_norm_add_kernel<T>, dim3((unsigned)n_rows), dim3(threads),
                                   (size_t)hidden * sizeof(float), stream, resid, (const T*)branch, parts, n_parts,
                                   (size_t)part_stride, post_w, layer_scale, next_w, (T*)out, rows, hidden, eps_b,
                                   eps_n));
  return (int)e;
}
