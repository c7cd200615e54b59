// Gated linear attention: a matrix-valued recurrent state per (request, head) with a decay per
// key channel,
//
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        S: [key_dim, value_dim], float32
//   o_t = S_t^T q_t
//
// and what surrounds it: the decays from a low-rank projection,
//   log alpha = log(sigmoid(W_2 a + b)) / tau,   a = the rank-r projection of the layer input,
// and the output stage, an RMS norm of every head's o over value_dim with one weight vector
// shared by the heads, times silu(gate).
//
// The state, the decays and their logarithms, the recurrence and the norm are float32 in every
// engine dtype.  A request's tokens are walked in order by the blocks that own its state, so the
// result at a position is bit-equal however the prompt was cut into steps and whatever else is
// in the batch: the state is read at the start of a step's portion and stored at its end.
//
// The inputs are columns of one stacked projection output [tokens, row_stride] (in the
// activation type, or float32 partial sums [parts, tokens, row_stride] of a split-K product).
// Three kernels: gla_prepare_kernel turns them into the recurrence's float32 inputs (scaled q, k,
// decays, v) once per step, gla_scan_kernel is the recurrence, gla_out_kernel the output stage.
#include "common.cuh"
#include "mma_utils.cuh"
#include "tcgen05_utils.cuh"

namespace tk {

struct GlaInput {
  const void* x;            // [n_tokens, row_stride] activation type, or null
  const float* parts;       // [n_parts, n_tokens, row_stride] float32, or null
  int n_parts;
  int row_stride;
  long long part_stride;
};

template <typename T>
__device__ __forceinline__ float gla_ld(const GlaInput& in, size_t off) {
  if (in.parts == nullptr) return to_f32<T>(((const T*)in.x)[off]);
  float acc = 0.0f;
  for (int s = 0; s < in.n_parts; ++s) acc += in.parts[(size_t)s * in.part_stride + off];
  return acc;
}

// Eight neighbouring elements as float32 (the address is a multiple of eight elements).
template <typename T> __device__ __forceinline__ void gla_ld8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void gla_ld8<float>(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void gla_ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}

// What the recurrence reads, float32 whatever the engine's dtype, head by head so that a head's
// tokens lie one after the other and a batch of them is one bulk copy:
//   [heads][tokens][dks / 4 pieces of  q * q_scale [4] | k [4] | alpha [4]  (four key channels each)]
//   [heads][tokens][v [dvs]]
// with dks = key_dim and dvs = value_dim rounded up to a multiple of 4 (16 bytes), the padding zero;
// a thread of the recurrence finds its four rows' inputs in one stretch of 48 bytes;
// and alpha = sigmoid(sum_j a[t, j] w2[c, j] + bias[c]) ^ (1 / tau), computed through its logarithm
// log(sigmoid(z)) = min(z, 0) - log1p(exp(-|z|)).  One thread per element.
template <typename T>
__global__ void gla_prepare_kernel(GlaInput in, int q_off, int k_off, int v_off, int a_off, const T* __restrict__ w2,
                                   const float* __restrict__ bias, float* __restrict__ prep, int n_tokens, int heads,
                                   int dk, int dv, int dks, int dvs, int rank, float inv_tau, float q_scale) {
  pdl_trigger();
  pdl_wait();
  const int per = dks + dvs;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * heads * per) return;
  const long long th = idx / per;
  const int e = (int)(idx - th * per);
  const int t = (int)(th / heads), h = (int)(th - (long long)t * heads);
  const size_t row = (size_t)t * in.row_stride;
  const size_t ht = (size_t)h * n_tokens + t;
  if (e >= dks) {
    const int c = e - dks;
    prep[(size_t)heads * n_tokens * 3 * dks + ht * dvs + c] = c < dv ? gla_ld<T>(in, row + v_off + h * dv + c) : 0.0f;
    return;
  }
  float* out = prep + ht * 3 * dks;
  float* piece = out + (e / 4) * 12 + (e & 3);
  if (e >= dk) { piece[0] = 0.0f; piece[4] = 0.0f; piece[8] = 0.0f; return; }
  const int ch = h * dk + e;
  float z = 0.0f;
  if (in.parts == nullptr && (rank & 7) == 0 && ((row + a_off) & 7) == 0) {
    // the usual case: eight factors a load (the dot product of `rank` steps is what this kernel waits for);
    // the sum runs in the order of the plain loop
    const T* arow = (const T*)in.x + row + a_off;
    const T* wrow = w2 + (size_t)ch * rank;
    for (int j = 0; j < rank; j += 8) {
      float a8[8], w8[8];
      gla_ld8<T>(arow + j, a8);
      gla_ld8<T>(wrow + j, w8);
#pragma unroll
      for (int i = 0; i < 8; ++i) z += a8[i] * w8[i];
    }
  } else {
    for (int j = 0; j < rank; ++j) z += gla_ld<T>(in, row + a_off + j) * to_f32<T>(w2[(size_t)ch * rank + j]);
  }
  if (bias != nullptr) z += bias[ch];
  piece[0] = gla_ld<T>(in, row + q_off + ch) * q_scale;
  piece[4] = gla_ld<T>(in, row + k_off + ch);
  piece[8] = expf((fminf(z, 0.0f) - log1pf(expf(-fabsf(z)))) * inv_tau);
}

constexpr int kGlaTile = 4;       // a thread keeps 4 rows (key channels) x 4 columns (value channels) of the state
constexpr int kGlaMaxWarps = 16;  // working warps of a block
constexpr int kGlaService = 5;    // serving warps: one copies the inputs in, four add the partial outputs up
constexpr int kGlaBatch = 8;      // tokens staged in shared memory at a time
constexpr int kGlaChunk = 16;     // row groups that one lane adds up when the partial outputs are joined (8 was measured slower)
constexpr int kGlaChunkPad = 16;  // floats of padding behind a chunk in the buffer of partial outputs
constexpr int kGlaStages = 4;     // staging buffers: a batch is asked for three batches before it is needed
constexpr int kGlaMaxKey = 256;   // key_dim: 16 warps of 16 rows at 32 columns a block

struct GlaScanParams {
  const float* prep;        // [heads, n_tokens, 3 dks] and [heads, n_tokens, dvs], see gla_prepare_kernel
  float* state;             // [n_slots, heads, key_dim, value_dim]
  float* out;               // [n_tokens, heads, value_dim]
  const int* req_q_start;
  const int* req_q_len;
  const int* req_slot;
  int* err;
  int n_tokens, n_slots, heads, key_dim, value_dim, dks, dvs;
};

// One block per (request, head, kCols value channels); it walks the request's tokens in order.
//
// Working warps: a thread keeps a 4 x 4 tile of the state in registers; per token it loads q, k and
// the decays of its four rows and the values of its four columns (four 16-byte loads of shared
// memory for 48 multiply-adds; with a column a thread the loads' way back into registers was the
// bound), two columns an instruction, and leaves its four partial outputs in shared memory.  A
// warp's lanes are kCols / 4 column groups times 128 / kCols row groups.
//
// Five more warps serve them, so that nothing but the recurrence stands in the chain of tokens.
// One brings the batches of eight tokens into four staging buffers, three batches ahead (a batch
// is worked through in less time than memory takes to answer): a bulk copy for the q | k | alpha
// pieces, which reports to the buffer's barrier, and 16-byte asynchronous copies for the values.
// Four add up the partial outputs of the batch before from the other of two output buffers.  One
// barrier per batch joins all warps.  A token's output is a sum over rows in an order that follows
// the rows alone, so the result does not depend on kCols, which the host picks by the number of
// blocks: a prompt alone has only heads * value_dim columns to share out.
// size bytes (a multiple of 16, both addresses 16-byte aligned) from global to this block's shared
// memory by the copy unit; the bytes are counted off at the barrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t size, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(dst), "l"(src), "r"(size), "r"(bar) : "memory");
}
__device__ __forceinline__ void gla_block_barrier() {
  asm volatile("bar.sync 1, %0;\n" ::"r"((int)blockDim.x) : "memory");
}

template <int kCols>
__global__ void __launch_bounds__((kGlaMaxWarps + kGlaService) * 32, 1) gla_scan_kernel(GlaScanParams p) {
  constexpr int kColGroups = kCols / kGlaTile;      // column groups of a warp
  constexpr int kRowGroups = 32 / kColGroups;       // row groups of a warp
  constexpr int kBatch = kGlaBatch;
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  const int r = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * kCols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x >> 5) - kGlaService;
  const int n_groups = n_warps * kRowGroups;
  const int qka_len = 3 * p.dks;                            // a staged token's q | k | alpha pieces
  const int per_buf = kBatch * (qka_len + kCols);           // staging buffers (stage0 + i * per_buf): the pieces, then the values
  // partial outputs [kBatch][n_groups][kCols], two of them; every chunk of row groups is followed by 64
  // bytes of padding, so that the lanes that add up neighbouring chunks read different banks
  const int out_tok = n_groups * kCols + ((n_groups + kGlaChunk - 1) / kGlaChunk) * kGlaChunkPad;
  const int per_out = kBatch * out_tok;
  // the first 32 floats: a barrier per staging buffer, and from the 16th on twelve zeros, the inputs of
  // rows beyond key_dim's last piece
  const uint32_t bars = smem_u32(smem);
  const float* zeros = smem + 16;
  float* stage0 = smem + 32;
  float* so = stage0 + kGlaStages * per_buf;
  // (the staging buffers need no clearing: what is read of them was copied, or filled with zeros by the copy)
  if (threadIdx.x < 16) smem[16 + threadIdx.x] = 0.0f;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kGlaStages; ++i) mbar_init(bars + 8 * i, 1);
  }
  fence_async_shared();       // the barriers, before the copy unit reports to them
  __syncthreads();
  volatile __shared__ int no_abort;
  if (threadIdx.x == 0) no_abort = 0;
  pdl_wait();
  const int dk = p.key_dim, dv = p.value_dim;
  const int slot = p.req_slot[r];
  const int q0 = p.req_q_start[r], n = p.req_q_len[r];
  if (slot < 0 || slot >= p.n_slots || q0 < 0 || n < 0 || q0 + n > p.n_tokens) {
    if (threadIdx.x == 0) set_error(p.err, kErrRequest, r, slot, q0);
    return;
  }
  const int n_batches = (n + kBatch - 1) / kBatch;

  if (warp >= n_warps) {
    // ---- serving warps
    const int sw = warp - n_warps, st = (sw - 1) * 32 + lane;      // warp 0 copies, the others add up
    // Serving warp 0 brings a batch in: the tokens' q | k | alpha pieces lie one after the other in
    // memory and are one bulk copy that reports to the stage's barrier; the block's values are
    // 16-byte asynchronous copies, a group a batch (an empty one beyond the last batch).
    const float* qka = p.prep + ((size_t)h * p.n_tokens + q0) * qka_len;
    const float* val = p.prep + (size_t)p.heads * p.n_tokens * qka_len + ((size_t)h * p.n_tokens + q0) * p.dvs + j0;
    auto copy = [&](int b) {
      if (sw != 0) return;
      if (b < n_batches) {
        const int t0 = b * kBatch, nb = min(kBatch, n - t0);
        float* buf = stage0 + (b % kGlaStages) * per_buf;
        const uint32_t bar = bars + 8 * (b % kGlaStages);
        if (lane == 0) {
          const uint32_t bytes = (uint32_t)(nb * qka_len * sizeof(float));
          mbar_expect_tx(bar, bytes);
          bulk_load(smem_u32(buf), qka + (size_t)t0 * qka_len, bytes, bar);
        }
        for (int i = lane; i < nb * kColGroups; i += 32) {
          const int tb = i / kColGroups, c = (i % kColGroups) * kGlaTile;
          const bool live = j0 + c < p.dvs;
          cp_async16(smem_u32(buf + kBatch * qka_len + tb * kCols + c), val + (size_t)(t0 + tb) * p.dvs + (live ? c : 0), live);
        }
      }
      cp_async_commit();
    };
    // ... and waits for it, with a limit: past it the error is flagged and the block goes on with what it has
    auto landed = [&](int b) {
      if (sw != 0) return;
      cp_async_wait<kGlaStages - 2>();      // all but the last two groups: this batch's values
      if (b >= n_batches) return;
      const uint32_t bar = bars + 8 * (b % kGlaStages), parity = (uint32_t)(b / kGlaStages) & 1u;
      if (!mbar_wait(bar, parity, &no_abort) && !mbar_wait(bar, parity, &no_abort)) {
        if (lane == 0) set_error(p.err, kErrWait, 40, b, r);
      }
    };
    // Four columns of a token are added up by 1, 2 or 4 neighbouring lanes: a lane takes sixteen row
    // groups (64 rows) in their order, then the lanes' sums are joined pairwise, (0 + 1) + (2 + 3).
    // The grouping follows the rows alone (rows that do not exist add zeros), so the sum is the same
    // whatever the block's shape.
    const int lanes_per = n_groups <= kGlaChunk ? 1 : n_groups <= 2 * kGlaChunk ? 2 : n_groups <= 4 * kGlaChunk ? 4 : 8;
    auto reduce = [&](int b) {
      if (sw == 0) return;
      const int t0 = b * kBatch, nb = min(kBatch, n - t0);
      const float* part = so + (b & 1) * per_out;
      const int items = nb * kColGroups * lanes_per;
      for (int base = 0; base < items; base += (kGlaService - 1) * 32) {       // whole warps stay together for the shuffles
        const int idx = base + st;
        const bool live = idx < items;
        const int item = live ? idx / lanes_per : 0, piece = idx % lanes_per;
        const int tb = item / kColGroups, c = (item % kColGroups) * kGlaTile;
        const int w0 = piece * kGlaChunk, w1 = live ? min(n_groups, w0 + kGlaChunk) : w0;
        const float4* src = reinterpret_cast<const float4*>(part + tb * out_tok + piece * kGlaChunkPad + c);
        float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
        for (int w = w0; w < w1; ++w) {
          const float4 x = src[w * (kCols / 4)];
          o.x += x.x; o.y += x.y; o.z += x.z; o.w += x.w;
        }
        for (int d = 1; d < lanes_per; d <<= 1) {
          o.x += __shfl_xor_sync(0xffffffffu, o.x, d); o.y += __shfl_xor_sync(0xffffffffu, o.y, d);
          o.z += __shfl_xor_sync(0xffffffffu, o.z, d); o.w += __shfl_xor_sync(0xffffffffu, o.w, d);
        }
        if (!live || piece != 0) continue;
        float* dst = p.out + ((size_t)(q0 + t0 + tb) * p.heads + h) * dv + j0 + c;
        const float t[kGlaTile] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int e = 0; e < kGlaTile; ++e) {
          if (j0 + c + e < dv) dst[e] = t[e];
        }
      }
    };
    for (int b = 0; b < kGlaStages - 1; ++b) copy(b);
    landed(0);
    gla_block_barrier();
    for (int b = 0; b < n_batches; ++b) {
      copy(b + kGlaStages - 1);             // into the buffer that batch b - 1 was worked through from
      if (b > 0) reduce(b - 1);
      landed(b + 1);
      gla_block_barrier();                  // batch b is worked through, batch b + 1 has landed
    }
    if (n_batches > 0) reduce(n_batches - 1);
    return;
  }

  // ---- working warps
  const int cg = lane % kColGroups, group = warp * kRowGroups + lane / kColGroups;
  const int row0 = group * kGlaTile, j = j0 + cg * kGlaTile;
  float* stile = p.state + (((size_t)slot * p.heads + h) * dk + row0) * dv + j;
  float2 s[kGlaTile][2];        // [row][column pair]
#pragma unroll
  for (int rr = 0; rr < kGlaTile; ++rr) {
    float t[kGlaTile];
#pragma unroll
    for (int c = 0; c < kGlaTile; ++c) t[c] = (row0 + rr < dk && j + c < dv) ? stile[(size_t)rr * dv + c] : 0.0f;
    s[rr][0] = make_float2(t[0], t[1]); s[rr][1] = make_float2(t[2], t[3]);
  }
  gla_block_barrier();
  for (int b = 0; b < n_batches; ++b) {
    const int nb = min(kBatch, n - b * kBatch);
    const float* buf = stage0 + (b % kGlaStages) * per_buf;
    // (the copy unit's writes are seen by whoever has seen the stage's barrier flip: it has, long ago)
    mbar_wait(bars + 8 * (b % kGlaStages), (uint32_t)(b / kGlaStages) & 1u, &no_abort);
    // One token: its inputs come from registers that were loaded while the token before was worked
    // on, and the next token's are loaded first of all.
    const bool padded = row0 >= p.dks;          // rows beyond the last piece read zeros
    const float4* mine = reinterpret_cast<const float4*>(padded ? zeros : buf + group * (3 * kGlaTile));
    const float4* vals = reinterpret_cast<const float4*>(buf + kBatch * qka_len + cg * kGlaTile);
    const int step = padded ? 0 : qka_len / 4;
    float4* part = reinterpret_cast<float4*>(so + (b & 1) * per_out + group * kCols + (group / kGlaChunk) * kGlaChunkPad + cg * kGlaTile);
    float4 q, k, a, v;
    auto load = [&]() {
      q = mine[0]; k = mine[1]; a = mine[2]; v = vals[0];
      mine += step; vals += kCols / 4;
    };
    auto token = [&](bool more) {
      const float4 qc = q, kc = k, ac = a;
      const float2 v01 = make_float2(v.x, v.y), v23 = make_float2(v.z, v.w);
      if (more) load();
      const float qs[kGlaTile] = {qc.x, qc.y, qc.z, qc.w}, ks[kGlaTile] = {kc.x, kc.y, kc.z, kc.w},
                  as[kGlaTile] = {ac.x, ac.y, ac.z, ac.w};
      float2 o01 = make_float2(0.0f, 0.0f), o23 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int rr = 0; rr < kGlaTile; ++rr) {
        const float2 a2 = make_float2(as[rr], as[rr]), k2 = make_float2(ks[rr], ks[rr]), q2 = make_float2(qs[rr], qs[rr]);
        s[rr][0] = fma2(a2, s[rr][0], mul2(k2, v01));
        s[rr][1] = fma2(a2, s[rr][1], mul2(k2, v23));
        o01 = fma2(q2, s[rr][0], o01);
        o23 = fma2(q2, s[rr][1], o23);
      }
      *part = make_float4(o01.x, o01.y, o23.x, o23.y);
      part += out_tok / 4;
    };
    load();
    if (nb == kBatch) {       // a full batch: a loop of known length
#pragma unroll
      for (int tb = 0; tb < kBatch; ++tb) token(tb + 1 < kBatch);
    } else {
      for (int tb = 0; tb < nb; ++tb) token(tb + 1 < nb);
    }
    gla_block_barrier();
  }
#pragma unroll
  for (int rr = 0; rr < kGlaTile; ++rr) {
    const float t[kGlaTile] = {s[rr][0].x, s[rr][0].y, s[rr][1].x, s[rr][1].y};
#pragma unroll
    for (int c = 0; c < kGlaTile; ++c) {
      if (row0 + rr < dk && j + c < dv) stile[(size_t)rr * dv + c] = t[c];
    }
  }
}

// y[t, h, e] = o[t, h, e] * rsqrt(mean_e o^2 + eps) * w[e] * silu(g[t, h, e]) * out_scale;   one warp per (token, head);
// rows of y are y_stride elements apart (a column range of wider rows)
template <typename T>
__global__ void gla_out_kernel(const float* __restrict__ o, GlaInput in, int g_off, const float* __restrict__ w,
                               T* __restrict__ y, int y_stride, float out_scale, int n_tokens, int heads, int dv,
                               float eps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
  const float* orow = o + (size_t)item * dv;
  float ss = 0.0f;
  for (int e = lane; e < dv; e += 32) ss += orow[e] * orow[e];
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)dv + eps);
  for (int e = lane; e < dv; e += 32) {
    float v = orow[e] * rstd;
    if (w != nullptr) v *= w[e];
    if (g_off >= 0) {
      const float g = gla_ld<T>(in, (size_t)t * in.row_stride + g_off + h * dv + e);
      v *= g / (1.0f + expf(-g));
    }
    y[(size_t)t * y_stride + h * dv + e] = from_f32<T>(v * out_scale);
  }
}

}  // namespace tk

static tk::GlaInput gla_input(const void* x, const float* parts, int n_parts, int n_tokens, int row_stride) {
  tk::GlaInput in;
  in.x = x; in.parts = parts; in.n_parts = n_parts; in.row_stride = row_stride;
  in.part_stride = (long long)n_tokens * row_stride;
  return in;
}

// prep: float32, n_tokens * heads * (3 dks + dvs) numbers with dks, dvs = key_dim, value_dim rounded up to a multiple of 4.
TK_API int tk_gla_prepare(const void* x, const float* parts, int n_parts, int row_stride, int q_off, int k_off,
                          int v_off, int a_off, const void* w2, const float* bias, float* prep, int n_tokens,
                          int heads, int key_dim, int value_dim, int rank, float tau, float q_scale, int dtype,
                          cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads < 1 || key_dim < 1 || value_dim < 1 || rank < 1 || !(tau > 0.0f) || (x == nullptr) == (parts == nullptr)) {
    return (int)cudaErrorInvalidValue;
  }
  const int dks = (key_dim + 3) / 4 * 4, dvs = (value_dim + 3) / 4 * 4;
  const long long total = (long long)n_tokens * heads * (dks + dvs);
  const tk::GlaInput in = gla_input(x, parts, n_parts, n_tokens, row_stride);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::gla_prepare_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                   in, q_off, k_off, v_off, a_off, (const T*)w2, bias, prep, n_tokens, heads, key_dim,
                                   value_dim, dks, dvs, rank, 1.0f / tau, q_scale));
  return (int)e;
}

template <int kCols>
static cudaError_t gla_scan_launch(const tk::GlaScanParams& p, int n_reqs, cudaStream_t stream) {
  constexpr int kRowGroups = 32 / (kCols / tk::kGlaTile), kBatch = tk::kGlaBatch;
  const int rows_per_warp = kRowGroups * tk::kGlaTile;
  const int n_warps = (p.key_dim + rows_per_warp - 1) / rows_per_warp;
  const int n_groups = n_warps * kRowGroups;
  const int col_tiles = (p.value_dim + kCols - 1) / kCols;
  if (n_warps > tk::kGlaMaxWarps || col_tiles > 65535) return cudaErrorInvalidValue;
  const size_t out_tok = (size_t)n_groups * kCols + (size_t)((n_groups + tk::kGlaChunk - 1) / tk::kGlaChunk) * tk::kGlaChunkPad;
  const size_t smem = sizeof(float) * (32 + (size_t)tk::kGlaStages * kBatch * (3 * p.dks + kCols) + 2 * kBatch * out_tok);
  cudaError_t e = cudaSuccess;
  if (smem > 48 * 1024) {
    e = cudaFuncSetAttribute(tk::gla_scan_kernel<kCols>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  return tk::launch(tk::gla_scan_kernel<kCols>, dim3((unsigned)n_reqs, (unsigned)p.heads, (unsigned)col_tiles),
                    dim3((n_warps + tk::kGlaService) * 32), smem, stream, p);
}

static int gla_sm_count() {
  static int sm_count[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  int sms = (dev >= 0 && dev < 64) ? sm_count[dev] : 0;
  if (sms == 0) {
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < 64) sm_count[dev] = sms;
  }
  return sms;
}

// cols: value channels per block (32, 16 or 8), or 0 for the launcher's choice by the number of blocks.
TK_API int tk_gla_scan(const float* prep, float* state, float* out, const int* req_q_start, const int* req_q_len,
                       const int* req_slot, int* err, int n_tokens, int n_reqs, int n_slots, int heads, int key_dim,
                       int value_dim, int cols, cudaStream_t stream) {
  if (n_tokens <= 0 || n_reqs <= 0) return 0;
  if (key_dim < 1 || key_dim > tk::kGlaMaxKey || value_dim < 1 || heads < 1 || heads > 65535 || prep == nullptr ||
      (cols != 0 && cols != 8 && cols != 16 && cols != 32)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::GlaScanParams p;
  p.prep = prep; p.state = state; p.out = out;
  p.req_q_start = req_q_start; p.req_q_len = req_q_len; p.req_slot = req_slot; p.err = err;
  p.n_tokens = n_tokens; p.n_slots = n_slots; p.heads = heads; p.key_dim = key_dim; p.value_dim = value_dim;
  p.dks = (key_dim + 3) / 4 * 4; p.dvs = (value_dim + 3) / 4 * 4;
  if (cols == 0) {
    const long long sms = gla_sm_count();
    if (sms <= 0) return (int)cudaErrorInvalidDevice;
    // measured on prompts of 2,048 tokens (8 and 16 heads of 128 x 256): 16 columns a block unless that
    // makes more than two blocks an SM (then 32) or fewer than one for every other SM (then 8)
    const long long blocks16 = (long long)n_reqs * heads * ((value_dim + 15) / 16);
    cols = blocks16 > 2 * sms ? 32 : 2 * blocks16 >= sms ? 16 : 8;
  }
  if (cols == 32 && key_dim > 128) cols = 16;      // the buffers of 32 columns and 256 rows are more than a block may have
  const cudaError_t e = cols == 32 ? gla_scan_launch<32>(p, n_reqs, stream)
                        : cols == 16 ? gla_scan_launch<16>(p, n_reqs, stream) : gla_scan_launch<8>(p, n_reqs, stream);
  return (int)e;
}

TK_API int tk_gla_out(const float* o, const void* x, const float* parts, int n_parts, int row_stride, int g_off,
                      const float* w, void* y, int y_stride, float out_scale, int n_tokens, int heads, int value_dim,
                      float eps, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads < 1 || value_dim < 1 || (g_off >= 0 && (x == nullptr) == (parts == nullptr))) return (int)cudaErrorInvalidValue;
  const tk::GlaInput in = gla_input(x, parts, n_parts, n_tokens, row_stride);
  const long long items = (long long)n_tokens * heads;
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::gla_out_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, o, in,
                                   g_off, w, (T*)y, y_stride, out_scale, n_tokens, heads, value_dim, eps));
  return (int)e;
}
