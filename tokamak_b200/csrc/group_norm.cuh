// RMS statistics over equal consecutive parts of a row that lies in shared memory.
#pragma once

#include "common.cuh"

namespace tk {

// rstd[g] = rsqrt(mean(row[g * n / groups ... (g + 1) * n / groups)^2) + eps) for every group; a warp
// takes a group at a time, so the order of a group's sum follows its own length alone.  Every thread
// of the block calls it; the row must be complete before (the function opens with a barrier) and
// rstd is complete after (it closes with one).
__device__ __forceinline__ void group_rstd(const float* row, int n, int groups, float eps, float* rstd) {
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int size = n / groups;
  for (int g = warp; g < groups; g += n_warps) {
    const float* part = row + (size_t)g * size;
    float ss = 0.0f;
    for (int i = lane; i < size; i += 32) ss += part[i] * part[i];
    ss = warp_sum(ss);
    if (lane == 0) rstd[g] = rsqrtf(ss / (float)size + eps);
  }
  __syncthreads();
}

}  // namespace tk
