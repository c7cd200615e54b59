// A row-major activation that is either stored in the activation type or still split into the
// float32 partial sums [parts, tokens, row_stride] of a split-K product; readers add the parts up
// in their order.
#pragma once

#include "common.cuh"

namespace tk {

struct StackedInput {
  const void* x;            // [n_tokens, row_stride] activation type, or null
  const float* parts;       // [n_parts, n_tokens, row_stride] float32, or null
  int n_parts;
  int row_stride;
  long long part_stride;
};

template <typename T>
__device__ __forceinline__ float stacked_ld(const StackedInput& in, size_t off) {
  if (in.parts == nullptr) return to_f32<T>(((const T*)in.x)[off]);
  float acc = 0.0f;
  for (int s = 0; s < in.n_parts; ++s) acc += in.parts[(size_t)s * in.part_stride + off];
  return acc;
}

// Four neighbouring values (the offset is a multiple of four elements), and the store of four.
template <typename T> __device__ __forceinline__ float4 stacked_ld4(const StackedInput& in, size_t off);
template <> __device__ __forceinline__ float4 stacked_ld4<float>(const StackedInput& in, size_t off) {
  if (in.parts == nullptr) return *reinterpret_cast<const float4*>((const float*)in.x + off);
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int s = 0; s < in.n_parts; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(in.parts + (size_t)s * in.part_stride + off);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  return acc;
}
template <> __device__ __forceinline__ float4 stacked_ld4<__nv_bfloat16>(const StackedInput& in, size_t off) {
  if (in.parts == nullptr) {
    const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)in.x + off);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int s = 0; s < in.n_parts; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(in.parts + (size_t)s * in.part_stride + off);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  return acc;
}
template <typename T> __device__ __forceinline__ void st4(T* dst, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
template <> __device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* dst, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(dst) = raw;
}

}  // namespace tk
