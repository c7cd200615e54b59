// Three more mixers on the recurrence of gated linear attention,
//
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t        (gla.cu: gla_scan_kernel)
//
// Each has a kernel that lays the recurrence's float32 inputs out (the layout of gla_prepare_kernel:
// per head and token, pieces of four key channels q | k | alpha, then the values) and a kernel for what
// follows the recurrence.  Gates, decays, their logarithms and exponentials, step sizes, the state and
// the norms are float32 in every engine dtype.
//
// * Forget-gated linear attention whose gate is also the key (HGRN2):
//     f = l + (1 - l) sigmoid(z_f + b),  alpha = f,  k = 1 - f,  q = silu(z_q),  v = z_v.
// * A matrix memory with exponential gates (mLSTM): per head the logarithms of an input gate
//   i = cap tanh((z_i + b_i) / cap) and a forget gate f = logsigmoid(cap tanh((z_f + b_f) / cap)), a running
//   maximum m_t = max(f + m_(t-1), i) that starts at zero, alpha = exp(f + m_(t-1) - m_t) for every row,
//   k = exp(i - m_t) z_k, q = z_q * q_scale.  The normaliser n_t = alpha n_(t-1) + k is one more column of the
//   state: the values get a column of ones, and o's last column is n_t . q_t.  The output stage divides by
//   max(|n . q|, exp(-m_t)) + 1e-6, scales every head to unit root mean square, and applies a weight per
//   channel and a sigmoid gate.
// * A state-space layer with a scalar decay per head (Mamba-2): dt = softplus(z_dt + dt_bias),
//   alpha = exp(-exp(A_log) dt) for every row, k = B, q = C (shared by the heads of a group), v = dt x; the
//   output stage adds D x, multiplies by silu(z) and applies an RMS norm in equal groups with a weight.
// * Retention: a fixed decay per head and rotated queries and keys: alpha = decay_h for every row,
//   q and k rotated over their first `rotary_dim` elements (neighbouring pairs or halves), k then scaled.
#include "common.cuh"
#include "group_norm.cuh"
#include "stacked_input.cuh"

namespace tk {

struct PrepLayout {
  float* prep;
  int n_tokens, heads, dk, dv, dks, dvs;
};

__device__ __forceinline__ void prep_qka(const PrepLayout& l, int h, int t, int e, float q, float k, float a) {
  float* piece = l.prep + ((size_t)h * l.n_tokens + t) * 3 * l.dks + (e / 4) * 12 + (e & 3);
  piece[0] = q; piece[4] = k; piece[8] = a;
}
__device__ __forceinline__ void prep_v(const PrepLayout& l, int h, int t, int c, float v) {
  l.prep[(size_t)l.heads * l.n_tokens * 3 * l.dks + ((size_t)h * l.n_tokens + t) * l.dvs + c] = v;
}

// (token, head, element of dks + dvs) of a thread, or false beyond the end
__device__ __forceinline__ bool prep_item(const PrepLayout& l, int& t, int& h, int& e) {
  const int per = l.dks + l.dvs;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)l.n_tokens * l.heads * per) return false;
  const long long th = idx / per;
  e = (int)(idx - th * per);
  t = (int)(th / l.heads);
  h = (int)(th - (long long)t * l.heads);
  return true;
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float log_sigmoidf_(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

template <typename T>
__global__ void hgrn2_prepare_kernel(StackedInput in, int q_off, int f_off, int v_off, const float* __restrict__ f_bias,
                                     const float* __restrict__ lower, PrepLayout l) {
  pdl_trigger();
  pdl_wait();
  int t, h, e;
  if (!prep_item(l, t, h, e)) return;
  const size_t row = (size_t)t * in.row_stride;
  if (e >= l.dks) {
    const int c = e - l.dks;
    prep_v(l, h, t, c, c < l.dv ? stacked_ld<T>(in, row + v_off + h * l.dv + c) : 0.0f);
    return;
  }
  if (e >= l.dk) { prep_qka(l, h, t, e, 0.0f, 0.0f, 0.0f); return; }
  const int ch = h * l.dk + e;
  const float zq = stacked_ld<T>(in, row + q_off + ch);
  const float lo = lower[ch];
  const float f = lo + (1.0f - lo) * sigmoidf_(stacked_ld<T>(in, row + f_off + ch) + f_bias[ch]);
  prep_qka(l, h, t, e, zq * sigmoidf_(zq), 1.0f - f, f);
}

// One warp per (request, head) walks the request's tokens, 32 * kMlstmPerLane at a time:
// gates[t, h] = (alpha, exp(i - m_t), exp(-m_t)), and the running maximum in the slot's record moves on.
// A token is the map m -> max(a + m, b) with a = f, b = i; maps compose to maps of the same form,
// (a2, b2) after (a1, b1) = (a1 + a2, max(a2 + b1, b2)), so the maxima of a stretch come from a scan: every lane
// composes its own consecutive tokens, the lanes' maps are scanned with shuffles, and each lane then walks
// its tokens again from the maximum that precedes them.
constexpr int kMlstmPerLane = 4;

template <typename T>
__global__ void mlstm_gates_kernel(StackedInput in, int i_off, int f_off, const float* __restrict__ i_bias,
                                   const float* __restrict__ f_bias, float cap, float* __restrict__ m_state,
                                   float* __restrict__ gates, const int* __restrict__ req_q_start,
                                   const int* __restrict__ req_q_len, const int* __restrict__ req_slot, int* err,
                                   int n_tokens, int n_reqs, int n_slots, int heads) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int idx = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (idx >= n_reqs * heads) return;
  const int r = idx / heads, h = idx - r * heads;
  const int slot = req_slot[r], q0 = req_q_start[r], n = req_q_len[r];
  if (slot < 0 || slot >= n_slots || q0 < 0 || n < 0 || q0 + n > n_tokens) {
    if (lane == 0) set_error(err, kErrRequest, r, slot, q0);
    return;
  }
  float m = m_state[(size_t)slot * heads + h];          // the maximum before the stretch, the same in every lane
  const float inv_cap = 1.0f / cap, bi = i_bias[h], bf = f_bias[h];
  for (int base = 0; base < n; base += 32 * kMlstmPerLane) {
    const int t0 = q0 + base + lane * kMlstmPerLane;
    float gi[kMlstmPerLane], gf[kMlstmPerLane];
    float a = 0.0f, b = -INFINITY;                      // the lane's tokens as one map; (0, -inf) changes nothing
#pragma unroll
    for (int j = 0; j < kMlstmPerLane; ++j) {
      if (t0 + j < q0 + n) {
        const size_t row = (size_t)(t0 + j) * in.row_stride;
        gi[j] = cap * tanhf((stacked_ld<T>(in, row + i_off + h) + bi) * inv_cap);
        gf[j] = log_sigmoidf_(cap * tanhf((stacked_ld<T>(in, row + f_off + h) + bf) * inv_cap));
        b = fmaxf(gf[j] + b, gi[j]);
        a += gf[j];
      }
    }
    // inclusive scan of the lanes' maps
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float pa = __shfl_up_sync(0xffffffffu, a, o);
      const float pb = __shfl_up_sync(0xffffffffu, b, o);
      if (lane >= o) { b = fmaxf(a + pb, b); a += pa; }
    }
    // the maximum in front of this lane's tokens: the lanes before it applied to m
    float ea = __shfl_up_sync(0xffffffffu, a, 1), eb = __shfl_up_sync(0xffffffffu, b, 1);
    float mj = lane == 0 ? m : fmaxf(ea + m, eb);
#pragma unroll
    for (int j = 0; j < kMlstmPerLane; ++j) {
      if (t0 + j < q0 + n) {
        const float m_new = fmaxf(gf[j] + mj, gi[j]);
        float* g = gates + ((size_t)(t0 + j) * heads + h) * 3;
        g[0] = expf(gf[j] + mj - m_new);
        g[1] = expf(gi[j] - m_new);
        g[2] = expf(-m_new);
        mj = m_new;
      }
    }
    m = __shfl_sync(0xffffffffu, fmaxf(a + m, b), 31);
  }
  if (lane == 0) m_state[(size_t)slot * heads + h] = m;
}

// l.dv counts the column of ones: the values proper are l.dv - 1 wide.
template <typename T>
__global__ void mlstm_prepare_kernel(StackedInput in, int q_off, int k_off, int v_off, const float* __restrict__ gates,
                                     float q_scale, PrepLayout l) {
  pdl_trigger();
  pdl_wait();
  int t, h, e;
  if (!prep_item(l, t, h, e)) return;
  const size_t row = (size_t)t * in.row_stride;
  const int dv = l.dv - 1;
  if (e >= l.dks) {
    const int c = e - l.dks;
    prep_v(l, h, t, c, c < dv ? stacked_ld<T>(in, row + v_off + h * dv + c) : c == dv ? 1.0f : 0.0f);
    return;
  }
  if (e >= l.dk) { prep_qka(l, h, t, e, 0.0f, 0.0f, 0.0f); return; }
  const float* g = gates + ((size_t)t * l.heads + h) * 3;
  const int ch = h * l.dk + e;
  prep_qka(l, h, t, e, stacked_ld<T>(in, row + q_off + ch) * q_scale, stacked_ld<T>(in, row + k_off + ch) * g[1], g[0]);
}

// o: [tokens, heads, dv + 1] (the last column is n . q).  One warp per (token, head).
template <typename T>
__global__ void mlstm_out_kernel(const float* __restrict__ o, const float* __restrict__ gates, StackedInput in, int g_off,
                                 const float* __restrict__ w, T* __restrict__ y, int y_stride, int n_tokens, int heads,
                                 int dv, float eps, float out_scale) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
  const float* orow = o + (size_t)item * (dv + 1);
  const float inv = 1.0f / (fmaxf(fabsf(orow[dv]), gates[(size_t)item * 3 + 2]) + 1e-6f);
  float ss = 0.0f;
  for (int e = lane; e < dv; e += 32) { const float v = orow[e] * inv; ss += v * v; }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)dv + eps) * inv;
  for (int e = lane; e < dv; e += 32) {
    const int c = h * dv + e;
    const float g = stacked_ld<T>(in, (size_t)t * in.row_stride + g_off + c);
    y[(size_t)t * y_stride + c] = from_f32<T>(orow[e] * rstd * w[c] * sigmoidf_(g) * out_scale);
  }
}

// xbc: float32 [tokens, inner + 2 groups dk] after the convolution and its silu: x | B | C.
template <typename T>
__global__ void ssd_prepare_kernel(const float* __restrict__ xbc, StackedInput in, int dt_off,
                                   const float* __restrict__ dt_bias, const float* __restrict__ a_log, int groups,
                                   PrepLayout l) {
  pdl_trigger();
  pdl_wait();
  int t, h, e;
  if (!prep_item(l, t, h, e)) return;
  const int inner = l.heads * l.dv, width = inner + 2 * groups * l.dk;
  const float* row = xbc + (size_t)t * width;
  const float dt = softplusf_(stacked_ld<T>(in, (size_t)t * in.row_stride + dt_off + h) + dt_bias[h]);
  if (e >= l.dks) {
    const int c = e - l.dks;
    prep_v(l, h, t, c, c < l.dv ? dt * row[h * l.dv + c] : 0.0f);
    return;
  }
  if (e >= l.dk) { prep_qka(l, h, t, e, 0.0f, 0.0f, 0.0f); return; }
  const int g = h / (l.heads / groups);
  prep_qka(l, h, t, e, row[inner + (groups + g) * l.dk + e], row[inner + g * l.dk + e], expf(-expf(a_log[h]) * dt));
}

// Retention's inputs: q and k rotated by the token's angles (table [tokens, rotary_dim / 2] of (cos, sin)), k times
// k_scale after the rotation, q times q_scale, alpha = decay[h] on every row of the head.
template <typename T>
__global__ void retention_prepare_kernel(StackedInput in, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                                         const float2* __restrict__ table, int rotary_dim, int halves, float q_scale,
                                         float k_scale, PrepLayout l) {
  pdl_trigger();
  pdl_wait();
  int t, h, e;
  if (!prep_item(l, t, h, e)) return;
  const size_t row = (size_t)t * in.row_stride;
  if (e >= l.dks) {
    const int c = e - l.dks;
    prep_v(l, h, t, c, c < l.dv ? stacked_ld<T>(in, row + v_off + h * l.dv + c) : 0.0f);
    return;
  }
  if (e >= l.dk) { prep_qka(l, h, t, e, 0.0f, 0.0f, 0.0f); return; }
  const int ch = h * l.dk + e;
  float q = stacked_ld<T>(in, row + q_off + ch), k = stacked_ld<T>(in, row + k_off + ch);
  if (table != nullptr && e < rotary_dim) {
    const int half = rotary_dim >> 1;
    int partner, idx; bool first;
    if (halves) { first = e < half; partner = first ? e + half : e - half; idx = first ? e : e - half; }
    else { first = !(e & 1); partner = e ^ 1; idx = e >> 1; }
    const float2 cs = table[(size_t)t * half + idx];
    const float qo = stacked_ld<T>(in, row + q_off + h * l.dk + partner);
    const float ko = stacked_ld<T>(in, row + k_off + h * l.dk + partner);
    q = first ? q * cs.x - qo * cs.y : q * cs.x + qo * cs.y;
    k = first ? k * cs.x - ko * cs.y : k * cs.x + ko * cs.y;
  }
  prep_qka(l, h, t, e, q * q_scale, k * k_scale, decay[h]);
}

// y = norm_groups((o + D x) silu(z)) * w * out_scale; one block per token, the row in shared memory.
template <typename T>
__global__ void ssd_out_kernel(const float* __restrict__ o, const float* __restrict__ xbc, int xbc_stride,
                               StackedInput in, int z_off, const float* __restrict__ skip, const float* __restrict__ w,
                               T* __restrict__ y, int y_stride, int heads, int dv, int norm_groups, float eps,
                               float out_scale) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, inner = heads * dv;
  float* row = smem;
  float* rstd = smem + inner;
  for (int c = threadIdx.x; c < inner; c += blockDim.x) {
    const float z = stacked_ld<T>(in, (size_t)t * in.row_stride + z_off + c);
    row[c] = (o[(size_t)t * inner + c] + skip[c / dv] * xbc[(size_t)t * xbc_stride + c]) * (z * sigmoidf_(z));
  }
  group_rstd(row, inner, norm_groups, eps, rstd);
  const int size = inner / norm_groups;
  for (int c = threadIdx.x; c < inner; c += blockDim.x) {
    y[(size_t)t * y_stride + c] = from_f32<T>(row[c] * rstd[c / size] * w[c] * out_scale);
  }
}

// y[t, c] = x[t, c] * sigmoid(g[t, g_off + c]) * scale, into rows of their own stride.
template <typename T>
__global__ void gate_scale_kernel(const T* __restrict__ x, StackedInput in, int g_off, T* __restrict__ y, int y_stride,
                                  int n_tokens, int cols, float scale, int gate_group) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * cols) return;
  const int t = (int)(idx / cols), c = (int)(idx - (long long)t * cols);
  const float g = stacked_ld<T>(in, (size_t)t * in.row_stride + g_off + c / gate_group);
  y[(size_t)t * y_stride + c] = from_f32<T>(to_f32<T>(x[idx]) * sigmoidf_(g) * scale);
}

}  // namespace tk

static tk::StackedInput stacked(const void* x, const float* parts, int n_parts, long long part_stride, int row_stride) {
  tk::StackedInput in;
  in.x = x; in.parts = parts; in.n_parts = n_parts; in.row_stride = row_stride; in.part_stride = part_stride;
  return in;
}

static tk::PrepLayout layout(float* prep, int n_tokens, int heads, int dk, int dv) {
  tk::PrepLayout l;
  l.prep = prep; l.n_tokens = n_tokens; l.heads = heads; l.dk = dk; l.dv = dv;
  l.dks = (dk + 3) / 4 * 4; l.dvs = (dv + 3) / 4 * 4;
  return l;
}

static unsigned prep_blocks(const tk::PrepLayout& l) {
  return (unsigned)(((long long)l.n_tokens * l.heads * (l.dks + l.dvs) + 255) / 256);
}

TK_API int tk_hgrn2_prepare(const void* x, const float* parts, int n_parts, long long part_stride, int row_stride,
                            int q_off, int f_off, int v_off, const float* f_bias, const float* lower, float* prep,
                            int n_tokens, int heads, int dk, int dv, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if ((x == nullptr) == (parts == nullptr) || heads < 1 || dk < 1 || dv < 1) return (int)cudaErrorInvalidValue;
  const tk::PrepLayout l = layout(prep, n_tokens, heads, dk, dv);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::hgrn2_prepare_kernel<T>, dim3(prep_blocks(l)), dim3(256), 0, stream,
                                             stacked(x, parts, n_parts, part_stride, row_stride), q_off, f_off, v_off,
                                             f_bias, lower, l));
  return (int)e;
}

// gates: float32 [tokens, heads, 3]; prep for values of dv + 1 columns; m_state: [n_slots, heads].
TK_API int tk_mlstm_prepare(const void* x, const float* parts, int n_parts, long long part_stride, int row_stride,
                            int q_off, int k_off, int v_off, int i_off, int f_off, const float* i_bias,
                            const float* f_bias, float cap, float q_scale, float* m_state, float* gates, float* prep,
                            const int* req_q_start, const int* req_q_len, const int* req_slot, int* err, int n_tokens,
                            int n_reqs, int n_slots, int heads, int dk, int dv, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0 || n_reqs <= 0) return 0;
  if ((x == nullptr) == (parts == nullptr) || heads < 1 || dk < 1 || dv < 1 || !(cap > 0.0f)) return (int)cudaErrorInvalidValue;
  const tk::StackedInput in = stacked(x, parts, n_parts, part_stride, row_stride);
  const tk::PrepLayout l = layout(prep, n_tokens, heads, dk, dv + 1);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::mlstm_gates_kernel<T>, dim3((unsigned)((n_reqs * heads + 1) / 2)),
                                             dim3(64), 0, stream, in, i_off, f_off, i_bias, f_bias, cap, m_state, gates,
                                             req_q_start, req_q_len, req_slot, err, n_tokens, n_reqs, n_slots, heads));
  if (e != cudaSuccess) return (int)e;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::mlstm_prepare_kernel<T>, dim3(prep_blocks(l)), dim3(256), 0, stream, in,
                                             q_off, k_off, v_off, (const float*)gates, q_scale, l));
  return (int)e;
}

TK_API int tk_mlstm_out(const float* o, const float* gates, const void* x, const float* parts, int n_parts,
                        long long part_stride, int row_stride, int g_off, const float* w, void* y, int y_stride,
                        int n_tokens, int heads, int dv, float eps, float out_scale, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if ((x == nullptr) == (parts == nullptr) || heads < 1 || dv < 1) return (int)cudaErrorInvalidValue;
  const long long items = (long long)n_tokens * heads;
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::mlstm_out_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0,
                                             stream, o, gates, stacked(x, parts, n_parts, part_stride, row_stride), g_off,
                                             w, (T*)y, y_stride, n_tokens, heads, dv, eps, out_scale));
  return (int)e;
}

TK_API int tk_retention_prepare(const void* x, const float* parts, int n_parts, long long part_stride, int row_stride,
                                int q_off, int k_off, int v_off, const float* decay, const float* table, int rotary_dim,
                                int halves, float q_scale, float k_scale, float* prep, int n_tokens, int heads, int dk,
                                int dv, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if ((x == nullptr) == (parts == nullptr) || heads < 1 || dk < 1 || dv < 1 || rotary_dim < 0 || rotary_dim > dk ||
      (rotary_dim & 1) || decay == nullptr) {
    return (int)cudaErrorInvalidValue;
  }
  const tk::PrepLayout l = layout(prep, n_tokens, heads, dk, dv);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::retention_prepare_kernel<T>, dim3(prep_blocks(l)), dim3(256), 0, stream,
                                             stacked(x, parts, n_parts, part_stride, row_stride), q_off, k_off, v_off,
                                             decay, (const float2*)table, rotary_dim, halves, q_scale, k_scale, l));
  return (int)e;
}

TK_API int tk_ssd_prepare(const float* xbc, const void* x, const float* parts, int n_parts, long long part_stride,
                          int row_stride, int dt_off, const float* dt_bias, const float* a_log, float* prep,
                          int n_tokens, int heads, int groups, int dk, int dv, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if ((x == nullptr) == (parts == nullptr) || heads < 1 || groups < 1 || heads % groups || dk < 1 || dv < 1) {
    return (int)cudaErrorInvalidValue;
  }
  const tk::PrepLayout l = layout(prep, n_tokens, heads, dk, dv);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::ssd_prepare_kernel<T>, dim3(prep_blocks(l)), dim3(256), 0, stream, xbc,
                                             stacked(x, parts, n_parts, part_stride, row_stride), dt_off, dt_bias, a_log,
                                             groups, l));
  return (int)e;
}

TK_API int tk_ssd_out(const float* o, const float* xbc, int xbc_stride, const void* x, const float* parts, int n_parts,
                      long long part_stride, int row_stride, int z_off, const float* skip, const float* w, void* y,
                      int y_stride, int n_tokens, int heads, int dv, int norm_groups, float eps, float out_scale,
                      int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int inner = heads * dv;
  if ((x == nullptr) == (parts == nullptr) || heads < 1 || dv < 1 || norm_groups < 1 || inner % norm_groups ||
      (size_t)(inner + norm_groups) * sizeof(float) > 200 * 1024) {
    return (int)cudaErrorInvalidValue;
  }
  const size_t smem = (size_t)(inner + norm_groups) * sizeof(float);
  cudaError_t e = cudaSuccess;
  // few tokens fill few SMs: more threads a row then (a group's sum is a warp's in either shape, the same bits)
  const int threads = n_tokens <= 64 && heads * dv >= 2048 ? 1024 : 256;
#define TK_SSD_OUT(T)                                                                                                  \
  do {                                                                                                                 \
    if (smem > 48 * 1024) {                                                                                            \
      e = cudaFuncSetAttribute(tk::ssd_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
      if (e != cudaSuccess) return (int)e;                                                                             \
    }                                                                                                                  \
    e = tk::launch(tk::ssd_out_kernel<T>, dim3((unsigned)n_tokens), dim3(threads), smem, stream, o, xbc, xbc_stride,   \
                   stacked(x, parts, n_parts, part_stride, row_stride), z_off, skip, w, (T*)y, y_stride, heads, dv,    \
                   norm_groups, eps, out_scale);                                                                       \
  } while (0)
  if (dtype == tk::kF32) { TK_SSD_OUT(float); } else if (dtype == tk::kBF16) { TK_SSD_OUT(__nv_bfloat16); }
  else return (int)cudaErrorInvalidValue;
#undef TK_SSD_OUT
  return (int)e;
}

TK_API int tk_gate_scale(const void* x, const void* g, const float* g_parts, int n_parts, long long part_stride,
                         int row_stride, int g_off, void* y, int y_stride, int n_tokens, int cols, float scale,
                         int gate_group, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0 || cols <= 0) return 0;
  if ((g == nullptr) == (g_parts == nullptr) || gate_group < 1) return (int)cudaErrorInvalidValue;
  const long long total = (long long)n_tokens * cols;
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::gate_scale_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256),
                                             0, stream, (const T*)x, stacked(g, g_parts, n_parts, part_stride, row_stride),
                                             g_off, (T*)y, y_stride, n_tokens, cols, scale, gate_group));
  return (int)e;
}
