// A mixture of gated feed-forward experts with a sigmoid router.
//
//   s = sigmoid(W_r h)                       scores, float32
//   c = s + correction                       choice scores
//   the experts form equal groups of neighbours; a group's score is the sum of its two largest c; only
//   experts of the `keep` best groups can be chosen; the `top` experts with the largest c are chosen
//   out = sum over the chosen e of s_e * W_down,e (act(W_gate,e h) * (W_up,e h))
//
// Five kernels.  moe_route_kernel: a block per token forms the logits, and its first warp makes the choice
// (ties go to the lower index).  moe_sort_kernel: one block counts the (token, choice) pairs of every expert, lays the
// pairs out expert by expert and lists the row tiles of the products.  moe_ffn_kernel: the experts'
// products over those tiles, first gate and up with the activation, then down; an output element is
// one thread's sum over ascending k, so a pair's result does not depend on what else is in the batch or
// where its row lies in a tile.  moe_combine_kernel: the weighted sum of a token's pairs in the order of
// its choices, float32.
//
// For bfloat16 at sizes that the tensor-core product on pairs of SMs takes, the products run there instead
// (gemm_pair_tcgen05.cu, grouped form): moe_sort_kernel also gives every pair a row in a layout in which
// an expert's rows are padded to whole tiles of kMoePadRows rows and names every tile's expert;
// moe_gather_kernel copies the tokens' rows there; gate/up with the activation in the epilogue and down
// run over that layout, row for row; moe_combine_rows_kernel forms the weighted sum from the pairs' rows.
#include "common.cuh"

namespace tk {

constexpr int kMoeMaxExperts = 1024;
constexpr int kMoeTileRows = 32;
constexpr int kMoeTileCols = 64;
constexpr int kMoeTileK = 32;
constexpr int kMoePadRows = 256;      // the row tile of the product on pairs of SMs

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

__device__ __forceinline__ void ld4_f32(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
__device__ __forceinline__ void ld4_f32(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 x = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x), b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}

constexpr int kMoeRouteWarps = 8;

// h: [n_tokens, width] activation type; router: [experts, width] float32; one block per token.  Every warp
// forms the logits of its share of the experts (a lane sums its elements in ascending order, the lanes are
// added up by a butterfly: the same sum whatever else the step holds); the first warp makes the choice.
template <typename T>
__global__ void __launch_bounds__(kMoeRouteWarps * 32)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router,
                 const float* __restrict__ correction, int* __restrict__ chosen,
                 float* __restrict__ weights, int n_tokens, int width, int experts, int n_groups,
                 int keep, int top) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  float* s = smem;
  float* c = s + experts;
  float* gs = c + experts;
  const T* x = h + (size_t)t * width;
  const bool vec = (width & 3) == 0 && (reinterpret_cast<uintptr_t>(h) & (4 * sizeof(T) - 1)) == 0 &&
                   (reinterpret_cast<uintptr_t>(router) & 15) == 0;
  for (int e = warp; e < experts; e += kMoeRouteWarps) {
    const float* w = router + (size_t)e * width;
    float acc = 0.0f;
    if (vec) {
      for (int i = lane * 4; i < width; i += 128) {
        float xv[4], wv[4];
        ld4_f32(x + i, xv); ld4_f32(w + i, wv);
        acc += xv[0] * wv[0]; acc += xv[1] * wv[1]; acc += xv[2] * wv[2]; acc += xv[3] * wv[3];
      }
    } else {
      for (int i = lane; i < width; i += 32) acc += to_f32<T>(x[i]) * w[i];
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      s[e] = 1.0f / (1.0f + expf(-acc));
      c[e] = s[e] + (correction != nullptr ? correction[e] : 0.0f);
    }
  }
  __syncthreads();
  if (warp != 0) return;
  __syncwarp();
  const int size = experts / n_groups;
  if (keep < n_groups) {
    for (int g = lane; g < n_groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;          // the two largest
      for (int i = 0; i < size; ++i) {
        const float v = c[g * size + i];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gs[g] = size >= 2 ? a + b : a;
    }
    __syncwarp();
    for (int it = 0; it < keep; ++it) {
      float best = -INFINITY; int bi = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && (v > best || (v == best && g < bi))) { best = v; bi = g; }
      }
      warp_argmax(best, bi);
      if (lane == 0 && bi < n_groups) gs[bi] = INFINITY;      // taken
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32) {
      if (gs[e / size] != INFINITY) c[e] = -INFINITY;
    }
    __syncwarp();
  }
  for (int it = 0; it < top; ++it) {
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = c[e];
      if (v > best || (v == best && e < bi && v != -INFINITY)) { best = v; bi = e; }
    }
    warp_argmax(best, bi);
    if (bi >= experts) bi = 0;        // fewer experts allowed than asked for: refused by the host
    if (lane == 0) {
      chosen[(size_t)t * top + it] = bi;
      weights[(size_t)t * top + it] = s[bi];
      c[bi] = -INFINITY;
    }
    __syncwarp();
  }
}

// order: [pairs] the pairs (token * top + choice) expert by expert; tiles: [max_tiles, 3] (expert, first
// place in order, rows) of every tile of kMoeTileRows rows; n_tiles: [1].
// pair_row (or null): [pairs] the row of every pair in the padded layout; tile_expert: [max_pad_tiles] the
// expert of every kMoePadRows-row tile of that layout, -1 for tiles that nobody uses.
__global__ void moe_sort_kernel(const int* __restrict__ chosen, int* __restrict__ order, int* __restrict__ tiles,
                                int* __restrict__ n_tiles, int pairs, int experts, int* __restrict__ pair_row,
                                int* __restrict__ tile_expert, int max_pad_tiles) {
  __shared__ int count[kMoeMaxExperts], start[kMoeMaxExperts], cursor[kMoeMaxExperts], tile0[kMoeMaxExperts];
  __shared__ int pad0[kMoeMaxExperts];
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = chosen[i];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tile = 0, pad = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = at; tile0[e] = tile; pad0[e] = pad;
      at += count[e];
      tile += (count[e] + kMoeTileRows - 1) / kMoeTileRows;
      pad += (count[e] + kMoePadRows - 1) / kMoePadRows;
    }
    *n_tiles = tile;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = chosen[i];
    if (e >= 0 && e < experts) {
      const int at = atomicAdd(&cursor[e], 1);
      order[start[e] + at] = i;
      if (pair_row != nullptr) pair_row[i] = pad0[e] * kMoePadRows + at;
    }
  }
  if (tile_expert != nullptr) {
    for (int t = threadIdx.x; t < max_pad_tiles; t += blockDim.x) tile_expert[t] = -1;
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
      const int n = (count[e] + kMoePadRows - 1) / kMoePadRows;
      for (int i = 0; i < n && pad0[e] + i < max_pad_tiles; ++i) tile_expert[pad0[e] + i] = e;
    }
  }
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int n = (count[e] + kMoeTileRows - 1) / kMoeTileRows;
    for (int i = 0; i < n; ++i) {
      int* tile = tiles + (size_t)(tile0[e] + i) * 3;
      tile[0] = e; tile[1] = start[e] + i * kMoeTileRows; tile[2] = min(kMoeTileRows, count[e] - i * kMoeTileRows);
    }
  }
}

struct MoeFfnParams {
  const void* a;            // rows of the left operand, activation type
  long long a_stride;
  int a_div;                // row of pair i is i / a_div (top for the tokens' rows, 1 for rows per pair)
  const void* b0;           // [experts, n_out, k] activation type
  const void* b1;           // the same for the second product of a gated unit, or null
  void* out;                // row of pair i: gated [pairs, n_out] activation type, else float32
  const int* order; const int* tiles; const int* n_tiles;
  int n_out, k, act;
};

template <typename T, bool kGated>
__global__ void __launch_bounds__(256) moe_ffn_kernel(MoeFfnParams p) {
  __shared__ float As[kMoeTileRows][kMoeTileK + 1];
  __shared__ float Bs[kGated ? 2 : 1][kMoeTileCols][kMoeTileK + 1];
  __shared__ int rows[kMoeTileRows];
  pdl_trigger();
  pdl_wait();
  if ((int)blockIdx.x >= *p.n_tiles) return;
  const int* tile = p.tiles + (size_t)blockIdx.x * 3;
  const int e = tile[0], first = tile[1], n_rows = tile[2];
  const int n0 = blockIdx.y * kMoeTileCols;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (tid < kMoeTileRows) rows[tid] = tid < n_rows ? p.order[first + tid] : -1;
  __syncthreads();
  const T* b0 = (const T*)p.b0 + (size_t)e * p.n_out * p.k;
  const T* b1 = kGated ? (const T*)p.b1 + (size_t)e * p.n_out * p.k : nullptr;
  float acc[2][4] = {}, acc1[2][4] = {};
  const int lk = tid & 31, lr = tid >> 5;
  for (int k0 = 0; k0 < p.k; k0 += kMoeTileK) {
    const bool kin = k0 + lk < p.k;
#pragma unroll
    for (int i = 0; i < kMoeTileRows / 8; ++i) {
      const int r = lr + 8 * i, pair = rows[r];
      As[r][lk] = (pair >= 0 && kin) ? to_f32<T>(((const T*)p.a)[(size_t)(pair / p.a_div) * p.a_stride + k0 + lk]) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < kMoeTileCols / 8; ++i) {
      const int c = lr + 8 * i;
      const bool in = kin && n0 + c < p.n_out;
      Bs[0][c][lk] = in ? to_f32<T>(b0[(size_t)(n0 + c) * p.k + k0 + lk]) : 0.0f;
      if (kGated) Bs[1][c][lk] = in ? to_f32<T>(b1[(size_t)(n0 + c) * p.k + k0 + lk]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kMoeTileK; ++kk) {
      const float a0 = As[2 * ty][kk], a1 = As[2 * ty + 1][kk];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float b = Bs[0][tx + 16 * i][kk];
        acc[0][i] += a0 * b; acc[1][i] += a1 * b;
        if (kGated) {
          const float u = Bs[1][tx + 16 * i][kk];
          acc1[0][i] += a0 * u; acc1[1][i] += a1 * u;
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int pair = rows[2 * ty + j];
    if (pair < 0) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = n0 + tx + 16 * i;
      if (c >= p.n_out) continue;
      if (kGated) ((T*)p.out)[(size_t)pair * p.n_out + c] = from_f32<T>(glu_act(acc[j][i], p.act) * acc1[j][i]);
      else ((float*)p.out)[(size_t)pair * p.n_out + c] = acc[j][i];
    }
  }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights, float* __restrict__ out,
                                   int n_tokens, int width, int top) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * width) return;
  const int t = (int)(idx / width), c = (int)(idx - (long long)t * width);
  float acc = 0.0f;
  for (int k = 0; k < top; ++k) acc += weights[(size_t)t * top + k] * y[((size_t)t * top + k) * width + c];
  out[idx] = acc;
}

// rows[pair_row[pair]] = h[pair / top], 16 bytes a thread (width a multiple of 8 bfloat16).
__global__ void moe_gather_kernel(const uint4* __restrict__ h, long long h_stride16, uint4* __restrict__ rows,
                                  const int* __restrict__ pair_row, int pairs, int top, int width16) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)pairs * width16) return;
  const int pair = (int)(idx / width16), c = (int)(idx - (long long)pair * width16);
  rows[(size_t)pair_row[pair] * width16 + c] = h[(size_t)(pair / top) * h_stride16 + c];
}

// out[t] = sum over the token's choices of weight * y[row of the pair], float32, in the order of the choices.
__global__ void moe_combine_rows_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ weights,
                                        const int* __restrict__ pair_row, float* __restrict__ out, int n_tokens,
                                        int width, int top) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int w2 = width >> 1;
  if (idx >= (long long)n_tokens * w2) return;
  const int t = (int)(idx / w2), c = (int)(idx - (long long)t * w2);
  float a0 = 0.0f, a1 = 0.0f;
  for (int k = 0; k < top; ++k) {
    const float w = weights[(size_t)t * top + k];
    const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(y + (size_t)pair_row[(size_t)t * top + k] * width)[c]);
    a0 += w * v.x; a1 += w * v.y;
  }
  reinterpret_cast<float2*>(out + (size_t)t * width)[c] = make_float2(a0, a1);
}

// ---- steps of few tokens: the chosen experts' weights are streamed once by the CUDA cores
//
// The output rows of the experts that some pair chose, one expert after the other, are dealt out evenly to
// a grid that fills the GPU once, so the load is even whatever the number of chosen experts, and an expert
// that nobody chose is not read.  For a stretch of an expert's rows a block lists the pairs that chose the
// expert, stages their input rows in shared memory (kMoeSmallRows at a time), and every warp forms whole
// output rows: a lane brings 16-byte pieces of the weight row into a ring of its own in shared memory by
// asynchronous copies, kMoeSmallStages - 1 stages of kMoeSmallPieces pieces ahead (what is under way is
// bounded by shared memory, not by registers), adds its products to four running sums in a fixed order, and the lanes are
// added up by a butterfly: a pair's result does not depend on what else is in the step.  Gated: the gate
// and up rows of output n lie in a stacked matrix [experts, 2 n_out, k] in alternating blocks of `block` rows.
constexpr int kMoeSmallRows = 4;
constexpr int kMoeSmallWarps = 8;
constexpr int kMoeSmallStages = 4;
constexpr int kMoeSmallPieces = 4;            // 16-byte pieces of a lane and stage
constexpr int kMoeSmallMaxPairs = 64;
constexpr int kMoeSmallRing = kMoeSmallWarps * kMoeSmallStages * kMoeSmallPieces * 32 * 16;      // bytes

struct MoeSmallParams {
  const __nv_bfloat16* a;       // input rows; pair i reads row i / a_div
  long long a_stride;
  int a_div;
  const __nv_bfloat16* b;       // [experts, n_out, k], or the stacked gate/up matrix
  void* out;                    // gated: bfloat16 [pairs, n_out]; else float32 [pairs, n_out]
  const int* chosen;            // [pairs]
  int pairs, experts, n_out, k, act, block;
};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
}
__device__ __forceinline__ void small_cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void small_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void small_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(kMoeSmallStages - 1) : "memory");
}

// Rows n_begin + warp, + kMoeSmallWarps, ... < n_end of expert e for `count` <= R staged input rows.
// A warp's work is the sequence of (row, stage) items; item i + kMoeSmallStages - 1 is asked for before
// item i is worked through.  ring: this lane's first piece; pieces of a stage are 512 bytes apart.
template <int R, bool kGated>
__device__ __forceinline__ void moe_small_rows(const MoeSmallParams& p, const __nv_bfloat16* xs, uint4* ring,
                                               const int* mine, int count, int e, int n_begin, int n_end) {
  constexpr int kSweeps = kGated ? kMoeSmallPieces / 2 : kMoeSmallPieces;     // sweeps of the warp over k in a stage
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per_row = (p.k + kSweeps * 256 - 1) / (kSweeps * 256);
  const int n_rows = n_end > n_begin + warp ? (n_end - n_begin - warp + kMoeSmallWarps - 1) / kMoeSmallWarps : 0;
  const int items = n_rows * per_row;
  const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring);
  auto ask = [&](int item) {
    if (item < items) {
      const int row = item / per_row, k0 = (item - row * per_row) * kSweeps * 256 + lane * 8;
      const int n = n_begin + warp + row * kMoeSmallWarps;
      const __nv_bfloat16* w0;
      if (kGated) {
        const int j = n / p.block, i = n - j * p.block;
        w0 = p.b + ((size_t)e * 2 * p.n_out + (size_t)(2 * j) * p.block + i) * p.k;
      } else {
        w0 = p.b + ((size_t)e * p.n_out + n) * p.k;
      }
      const uint32_t dst = ring_u32 + (uint32_t)(item % kMoeSmallStages) * (kMoeSmallPieces * 512);
#pragma unroll
      for (int u = 0; u < kSweeps; ++u) {
        const int kk = k0 + u * 256;
        if (kk < p.k) {
          small_cp16(dst + u * 512, w0 + kk);
          if (kGated) small_cp16(dst + (kSweeps + u) * 512, w0 + (size_t)p.block * p.k + kk);
        }
      }
    }
    small_commit();
  };
  for (int i = 0; i < kMoeSmallStages - 1; ++i) ask(i);
  float acc0[R][4], acc1[R][4];
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { acc0[r][i] = 0.0f; acc1[r][i] = 0.0f; }
  }
  for (int item = 0; item < items; ++item) {
    ask(item + kMoeSmallStages - 1);
    small_wait();
    const int row = item / per_row, part = item - row * per_row;
    const int k0 = part * kSweeps * 256 + lane * 8;
    const uint4* src = ring + (size_t)(item % kMoeSmallStages) * (kMoeSmallPieces * 32);
#pragma unroll
    for (int u = 0; u < kSweeps; ++u) {
      const int kk = k0 + u * 256;
      if (kk < p.k) {
        float wa[8], wb[8];
        unpack8(src[u * 32], wa);
        if (kGated) unpack8(src[(kSweeps + u) * 32], wb);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (r < count) {
            float xv[8];
            unpack8(*reinterpret_cast<const uint4*>(xs + (size_t)r * p.k + kk), xv);
#pragma unroll
            for (int i = 0; i < 8; ++i) {       // four running sums a row, so that no product waits for the one before
              acc0[r][i & 3] += xv[i] * wa[i];
              if (kGated) acc1[r][i & 3] += xv[i] * wb[i];
            }
          }
        }
      }
    }
    if (part + 1 < per_row) continue;
    const int n = n_begin + warp + row * kMoeSmallWarps;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (r < count) {              // (the same for every lane)
        const float s0 = warp_sum((acc0[r][0] + acc0[r][1]) + (acc0[r][2] + acc0[r][3]));
        const float s1 = kGated ? warp_sum((acc1[r][0] + acc1[r][1]) + (acc1[r][2] + acc1[r][3])) : 0.0f;
        if (lane == 0) {
          const size_t at = (size_t)mine[r] * p.n_out + n;
          if (kGated) ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(glu_act(s0, p.act) * s1);
          else ((float*)p.out)[at] = s0;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc0[r][i] = 0.0f; acc1[r][i] = 0.0f; }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

template <bool kGated>
__global__ void __launch_bounds__(kMoeSmallWarps * 32) moe_small_kernel(MoeSmallParams p) {
  extern __shared__ __align__(16) unsigned char small_smem[];      // the warps' rings, then the staged input rows
  __shared__ unsigned live_bits[kMoeMaxExperts / 32];
  __shared__ int live_ids[kMoeSmallMaxPairs], mine[kMoeSmallMaxPairs], chosen_s[kMoeSmallMaxPairs];
  __shared__ int n_live_s, total_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint4* ring = reinterpret_cast<uint4*>(small_smem) + (size_t)warp * kMoeSmallStages * kMoeSmallPieces * 32 + lane;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(small_smem + kMoeSmallRing);
  pdl_trigger();
  if (threadIdx.x < kMoeMaxExperts / 32) live_bits[threadIdx.x] = 0u;
  __syncthreads();
  pdl_wait();
  // the experts that were chosen, in ascending order
  if (threadIdx.x < p.pairs) {
    const int e = p.chosen[threadIdx.x];
    chosen_s[threadIdx.x] = e;
    if (e >= 0 && e < p.experts) atomicOr(&live_bits[e >> 5], 1u << (e & 31));
  }
  __syncthreads();
  if (warp == 0) {
    unsigned word = live_bits[lane];
    const int c = __popc(word);
    int before = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, before, o);
      if (lane >= o) before += up;
    }
    if (lane == 31) n_live_s = before;
    before -= c;
    while (word != 0u) {
      const int bit = __ffs(word) - 1;
      live_ids[before++] = lane * 32 + bit;
      word &= word - 1u;
    }
  }
  __syncthreads();
  const long long all_rows = (long long)n_live_s * p.n_out;
  long long g = all_rows * blockIdx.x / gridDim.x;
  const long long g_end = all_rows * (blockIdx.x + 1) / gridDim.x;
  const int k16 = p.k / 8;
  while (g < g_end) {
    const int rank = (int)(g / p.n_out), n_begin = (int)(g - (long long)rank * p.n_out);
    const int n_end = (int)min((long long)p.n_out, n_begin + (g_end - g));
    const int e = live_ids[rank];
    if (warp == 0) {
      int total = 0;
      for (int base = 0; base < p.pairs; base += 32) {
        const bool m = base + lane < p.pairs && chosen_s[base + lane] == e;
        const unsigned votes = __ballot_sync(0xffffffffu, m);
        if (m) mine[total + __popc(votes & ((1u << lane) - 1u))] = base + lane;
        total += __popc(votes);
      }
      if (lane == 0) total_s = total;
    }
    __syncthreads();
    const int total = total_s;
    for (int first = 0; first < total; first += kMoeSmallRows) {
      const int count = min(kMoeSmallRows, total - first);
      for (int i = threadIdx.x; i < count * k16; i += blockDim.x) {
        const int r = i / k16, c = i - r * k16;
        reinterpret_cast<uint4*>(xs)[(size_t)r * k16 + c] =
            reinterpret_cast<const uint4*>(p.a + (size_t)(mine[first + r] / p.a_div) * p.a_stride)[c];
      }
      __syncthreads();
      if (count <= 2) moe_small_rows<2, kGated>(p, xs, ring, mine + first, count, e, n_begin, n_end);
      else moe_small_rows<4, kGated>(p, xs, ring, mine + first, count, e, n_begin, n_end);
      __syncthreads();
    }
    g += n_end - n_begin;
  }
}

}  // namespace tk

TK_API int tk_moe_tile_rows() { return tk::kMoeTileRows; }

TK_API int tk_moe_pad_rows() { return tk::kMoePadRows; }

TK_API int tk_moe_route(const void* h, const float* router, const float* correction, int* chosen, float* weights,
                        int* order, int* tiles, int* n_tiles, int* pair_row, int* tile_expert, int max_pad_tiles,
                        int n_tokens, int width, int experts, int n_groups, int keep, int top, int dtype,
                        cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (experts < 1 || experts > tk::kMoeMaxExperts || n_groups < 1 || experts % n_groups || keep < 1 || keep > n_groups ||
      top < 1 || top > keep * (experts / n_groups)) {
    return (int)cudaErrorInvalidValue;
  }
  const size_t smem = (size_t)(2 * experts + n_groups) * sizeof(float);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::moe_route_kernel<T>, dim3((unsigned)n_tokens),
                                             dim3(tk::kMoeRouteWarps * 32), smem, stream, (const T*)h, router, correction, chosen,
                                             weights, n_tokens, width, experts, n_groups, keep, top));
  if (e != cudaSuccess) return (int)e;
  e = tk::launch(tk::moe_sort_kernel, dim3(1), dim3(1024), 0, stream, (const int*)chosen, order, tiles, n_tiles,
                 n_tokens * top, experts, pair_row, tile_expert, max_pad_tiles);
  return (int)e;
}

TK_API int tk_moe_gather(const void* h, long long h_stride, void* rows, const int* pair_row, int n_tokens, int top,
                         int width, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (width % 8 != 0 || h_stride % 8 != 0 || ((uintptr_t)h & 15u) != 0 || ((uintptr_t)rows & 15u) != 0) {
    return (int)cudaErrorInvalidValue;
  }
  const long long total = (long long)n_tokens * top * (width / 8);
  return (int)tk::launch(tk::moe_gather_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                         (const uint4*)h, h_stride / 8, (uint4*)rows, pair_row, n_tokens * top, top, width / 8);
}

TK_API int tk_moe_combine_rows(const void* y, const float* weights, const int* pair_row, float* out, int n_tokens,
                               int width, int top, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (width % 2 != 0) return (int)cudaErrorInvalidValue;
  const long long total = (long long)n_tokens * (width / 2);
  return (int)tk::launch(tk::moe_combine_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                         (const __nv_bfloat16*)y, weights, pair_row, out, n_tokens, width, top);
}

// gated != 0: out[pair] = act(a[pair / a_div] b0^T) * (a[pair / a_div] b1^T) in the activation type;
// else out[pair] = a[pair / a_div] b0^T in float32.
TK_API int tk_moe_ffn(const void* a, long long a_stride, int a_div, const void* b0, const void* b1, void* out,
                      const int* order, const int* tiles, const int* n_tiles, int max_tiles, int n_out, int k, int act,
                      int dtype, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (n_out < 1 || k < 1 || a_div < 1) return (int)cudaErrorInvalidValue;
  tk::MoeFfnParams p;
  p.a = a; p.a_stride = a_stride; p.a_div = a_div; p.b0 = b0; p.b1 = b1; p.out = out;
  p.order = order; p.tiles = tiles; p.n_tiles = n_tiles; p.n_out = n_out; p.k = k; p.act = act;
  const dim3 grid((unsigned)max_tiles, (unsigned)((n_out + tk::kMoeTileCols - 1) / tk::kMoeTileCols));
  cudaError_t e = cudaSuccess;
  if (b1 != nullptr) {
    TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::moe_ffn_kernel<T, true>, grid, dim3(256), 0, stream, p));
  } else {
    TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::moe_ffn_kernel<T, false>, grid, dim3(256), 0, stream, p));
  }
  return (int)e;
}

TK_API int tk_moe_combine(const float* y, const float* weights, float* out, int n_tokens, int width, int top,
                          cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const long long total = (long long)n_tokens * width;
  return (int)tk::launch(tk::moe_combine_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, y, weights,
                         out, n_tokens, width, top);
}

TK_API int tk_moe_small_max_pairs() { return tk::kMoeSmallMaxPairs; }

// bfloat16.  block > 0: b is the stacked gate/up matrix [experts, 2 n_out, k] (alternating blocks of `block`
// rows), out[pair] = act(gate) * up in bfloat16; block == 0: b is [experts, n_out, k], out[pair] float32.
TK_API int tk_moe_small(const void* a, long long a_stride, int a_div, const void* b, void* out, const int* chosen,
                        int pairs, int experts, int n_out, int k, int act, int block, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  const size_t smem = (size_t)tk::kMoeSmallRing + (size_t)tk::kMoeSmallRows * k * sizeof(__nv_bfloat16);
  if (pairs > tk::kMoeSmallMaxPairs || experts < 1 || experts > tk::kMoeMaxExperts || n_out < 1 || k < 8 || k % 8 ||
      a_stride % 8 || a_div < 1 || block < 0 || (block > 0 && n_out % block) || smem > 200 * 1024 ||
      ((uintptr_t)a & 15u) || ((uintptr_t)b & 15u)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::MoeSmallParams p;
  p.a = (const __nv_bfloat16*)a; p.a_stride = a_stride; p.a_div = a_div; p.b = (const __nv_bfloat16*)b; p.out = out;
  p.chosen = chosen; p.pairs = pairs; p.experts = experts; p.n_out = n_out; p.k = k; p.act = act; p.block = block;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) {
    return (int)cudaErrorInvalidValue;
  }
  cudaError_t e = cudaSuccess;
  // as many blocks as run at once, and no more than there are rows for the warps of each
#define TK_MOE_SMALL(G)                                                                                                 \
  do {                                                                                                                  \
    e = cudaFuncSetAttribute(tk::moe_small_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
    if (e != cudaSuccess) return (int)e;                                                                                \
    int per_sm = 0;                                                                                                     \
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tk::moe_small_kernel<G>, tk::kMoeSmallWarps * 32, smem); \
    if (e != cudaSuccess || per_sm < 1) return (int)(e != cudaSuccess ? e : cudaErrorInvalidValue);                     \
    const long long most = ((long long)(pairs < experts ? pairs : experts) * n_out + tk::kMoeSmallWarps - 1) /          \
                           tk::kMoeSmallWarps;                                                                          \
    const long long blocks = (long long)sms * per_sm < most ? (long long)sms * per_sm : most;                           \
    e = tk::launch(tk::moe_small_kernel<G>, dim3((unsigned)blocks), dim3(tk::kMoeSmallWarps * 32), smem, stream, p);    \
  } while (0)
  if (block > 0) { TK_MOE_SMALL(true); } else { TK_MOE_SMALL(false); }
#undef TK_MOE_SMALL
  return (int)e;
}
