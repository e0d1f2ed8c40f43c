// Kernels of mixers that carry a state of fixed size from token to token, and the row-wise
// kernels around them.
//
//   pair_rope_cache_write_kernel  neighbouring pairs (2i, 2i+1) of q and k turn by tabulated
//                                 angles; k and v go to their cache slots; the projection's row
//                                 may hold further columns behind q | k | v
//   head_gate_kernel              out[t, h, :] *= sigmoid(logit[t, h])
//   conv_tokens_kernel            causal convolution per channel over a sequence's tokens, the
//                                 taps before the portion's first token taken from the state
//   conv_state_update_kernel      the last taps - 1 inputs of every sequence into its state
//   rglru_gates_kernel            block-diagonal gate matrices, decay a and gated input b of the
//                                 recurrence S <- a S + b, all in float32
//   rglru_scan_kernel             the recurrence over a sequence's tokens, times the other branch
//   ssd_scan_kernel               S <- exp(A dt) S + dt B x^T,  y = S^T C + D x  per head
//   delta_rule_scan_kernel        S <- diag(w) S - (a u)(u^T S) + k v^T,  o = S^T r  per head, with the
//                                 decay w, the removal rate a and the unit key u made on the way in
//   gated_group_norm_kernel       (y * silu(z)) normed in equal parts by their own RMS, times w; or
//                                 y normed in equal parts, times w, times sigmoid(z)
//   dual_norm_mean_kernel         (rms(a) wa + rms(b) wb) / 2, written or added to the stream
//   act_rows_kernel               gelu (tanh form), squared relu, silu on strided columns
//   residual_add_kernel, gated_rows_add_kernel
//
// What a recurrence reads and keeps is float32 whatever the storage type of the projections.
// A sequence is rows q_start[s] .. q_start[s] + q_len[s] - 1 of the step; its state lives in
// row seq_slots[s] of a slot-indexed array.  Every sum has an order that depends on the sizes
// only, so a row's result does not depend on what else is in the step.
#include "common.cuh"

#include <math_constants.h>

namespace vx {

__device__ __forceinline__ float sq_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float sq_softplus(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }
__device__ __forceinline__ float sq_silu(float v) { return v * sq_sigmoid(v); }
__device__ __forceinline__ float sq_gelu_tanh(float v) {
  return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}
__device__ __forceinline__ float sq_act(float v, int kind) {
  if (kind == 1) return sq_silu(v);
  if (kind == 2) return sq_gelu_tanh(v);
  if (kind == 3) { const float r = fmaxf(v, 0.f); return r * r; }
  if (kind == 4) return tanhf(v);
  return v;
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void pair_rope_cache_write_kernel(T* __restrict__ qkv, long long stride,
                                             const int* __restrict__ positions,
                                             const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                             const int* __restrict__ slots, T* __restrict__ k_cache,
                                             T* __restrict__ v_cache, int H, int G, int D, int rot, int max_pos,
                                             long long num_slots, int write_cache, int* status) {
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // 0..H-1 q, H..H+G-1 k, H+G.. v
  const int half = rot >> 1;
  const bool is_q = head < H, is_k = !is_q && head < H + G;
  if (!is_q && !write_cache) return;
  int pos = positions[t];
  if (rot > 0 && (pos < 0 || pos >= max_pos)) {
    if (threadIdx.x == 0 && head == 0) atomicOr(status, VX_STATUS_BAD_POSITION);
    pos = 0;
  }
  const float* c = cos_t + (size_t)pos * half;
  const float* s = sin_t + (size_t)pos * half;
  T* row = qkv + (size_t)t * stride + (size_t)head * D;
  T* dst = row;
  if (!is_q) {
    const int slot = slots[t];
    if (slot < 0) return;
    if ((long long)slot >= num_slots) {
      if (threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_SLOT);
      return;
    }
    const int g = is_k ? head - H : head - H - G;
    dst = (is_k ? k_cache : v_cache) + ((size_t)slot * G + g) * D;
  }
  if (is_q || is_k) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float u = to_float(row[2 * i]), v = to_float(row[2 * i + 1]);
      dst[2 * i] = from_float<T>(u * c[i] - v * s[i]);
      dst[2 * i + 1] = from_float<T>(v * c[i] + u * s[i]);
    }
    if (is_k)
      for (int i = rot + threadIdx.x; i < D; i += blockDim.x) dst[i] = row[i];
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = row[i];
  }
}

template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ logits,
                                 long long logit_stride, int H, int D) {
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  for (int idx = threadIdx.x; idx < H * D; idx += blockDim.x) {
    const int h = idx / D;
    const float g = sq_sigmoid(to_float(logits[(size_t)t * logit_stride + h]));
    T* p = out + (size_t)t * out_stride + idx;
    *p = from_float<T>(to_float(*p) * g);
  }
}

// ---------------------------------------------------------------------------------------------
// Convolution.  state[slot][m][c], m = 0 .. taps - 2, is the input at the portion's first
// position minus (taps - 1 - m); zero before the sequence's start.
template <typename T>
__global__ void conv_tokens_kernel(const T* __restrict__ x, long long x_stride, int channels, int taps,
                                   const float* __restrict__ w, const float* __restrict__ bias,
                                   const float* __restrict__ state, long long state_stride,
                                   float* __restrict__ out, long long out_stride,
                                   const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ seq_slots, int act) {
  allow_dependents();
  grid_dependency_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= channels) return;
  const int n = q_len[s], start = q_start[s];
  const float* st = state + (size_t)seq_slots[s] * state_stride;
  const float b = bias[c];
  for (int i = blockIdx.z; i < n; i += gridDim.z) {
    float acc = b;
    for (int k = 0; k < taps; ++k) {
      const int j = i - (taps - 1) + k;
      const float v = j >= 0 ? to_float(x[(size_t)(start + j) * x_stride + c])
                             : st[(size_t)(taps - 1 + j) * channels + c];
      acc = fmaf(w[(size_t)c * taps + k], v, acc);
    }
    out[(size_t)(start + i) * out_stride + c] = sq_act(acc, act);
  }
}

template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ x, long long x_stride, int channels, int taps,
                                         float* __restrict__ state, long long state_stride,
                                         const int* __restrict__ q_start, const int* __restrict__ q_len,
                                         const int* __restrict__ seq_slots) {
  allow_dependents();
  grid_dependency_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= channels) return;
  const int n = q_len[s], start = q_start[s];
  if (n <= 0) return;
  float* st = state + (size_t)seq_slots[s] * state_stride;
  // Ascending m: what is read lies at or behind what has been written.
  for (int m = 0; m < taps - 1; ++m) {
    const int j = n - (taps - 1) + m;
    const float v = j >= 0 ? to_float(x[(size_t)(start + j) * x_stride + c]) : st[(size_t)(m + n) * channels + c];
    st[(size_t)m * channels + c] = v;
  }
}

// ---------------------------------------------------------------------------------------------
// Gates of the real-gated linear recurrent unit.  u [tokens, width] float32 is cut into `blocks`
// equal parts; in part b, r = sigmoid(Wa[b] u_b + ba[b]) and i = sigmoid(Wi[b] u_b + bi[b]) with
// the matrices stored transposed, [blocks][in][out].  a = exp(-c r softplus(lam)),
// b = sqrt(1 - a^2) i u.
template <int TT>
__global__ void rglru_gates_kernel(const float* __restrict__ u, long long u_stride, int part,
                                   const float* __restrict__ wa_t, const float* __restrict__ ba,
                                   const float* __restrict__ wi_t, const float* __restrict__ bi,
                                   const float* __restrict__ lam, float decay_scale, float* __restrict__ a_out,
                                   float* __restrict__ b_out, long long ab_stride, int num_tokens) {
  extern __shared__ __align__(16) float u_s[];  // [part][TT]: a thread reads all tokens of one input at once
  allow_dependents();
  grid_dependency_wait();
  const int t0 = blockIdx.x * TT;
  const int blk = blockIdx.y;
  for (int idx = threadIdx.x; idx < TT * part; idx += blockDim.x) {
    const int tt = idx / part, i = idx - tt * part;
    u_s[i * TT + tt] = t0 + tt < num_tokens ? u[(size_t)(t0 + tt) * u_stride + (size_t)blk * part + i] : 0.f;
  }
  __syncthreads();
  const float* wa = wa_t + (size_t)blk * part * part;
  const float* wi = wi_t + (size_t)blk * part * part;
  for (int o = threadIdx.x; o < part; o += blockDim.x) {
    float ar[TT], ai[TT];
    const int c = blk * part + o;
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) { ar[tt] = ba[c]; ai[tt] = bi[c]; }
#pragma unroll 4
    for (int i = 0; i < part; ++i) {
      const float wr = wa[(size_t)i * part + o], wg = wi[(size_t)i * part + o];
      if (TT % 4 == 0) {
        const float4* u4 = reinterpret_cast<const float4*>(u_s + i * TT);
#pragma unroll
        for (int q = 0; q < TT / 4; ++q) {
          const float4 uv = u4[q];
          ar[4 * q] = fmaf(wr, uv.x, ar[4 * q]);         ai[4 * q] = fmaf(wg, uv.x, ai[4 * q]);
          ar[4 * q + 1] = fmaf(wr, uv.y, ar[4 * q + 1]); ai[4 * q + 1] = fmaf(wg, uv.y, ai[4 * q + 1]);
          ar[4 * q + 2] = fmaf(wr, uv.z, ar[4 * q + 2]); ai[4 * q + 2] = fmaf(wg, uv.z, ai[4 * q + 2]);
          ar[4 * q + 3] = fmaf(wr, uv.w, ar[4 * q + 3]); ai[4 * q + 3] = fmaf(wg, uv.w, ai[4 * q + 3]);
        }
      } else {
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
          const float uv = u_s[i * TT + tt];
          ar[tt] = fmaf(wr, uv, ar[tt]);
          ai[tt] = fmaf(wg, uv, ai[tt]);
        }
      }
    }
    const float sp = sq_softplus(lam[c]);
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      if (t0 + tt >= num_tokens) break;
      const float r = sq_sigmoid(ar[tt]), g = sq_sigmoid(ai[tt]);
      const float log_a = -decay_scale * r * sp;
      const float a = expf(log_a);
      const float mult = sqrtf(fmaxf(-expm1f(2.0f * log_a), 0.f));
      a_out[(size_t)(t0 + tt) * ab_stride + c] = a;
      b_out[(size_t)(t0 + tt) * ab_stride + c] = mult * g * u_s[o * TT + tt];
    }
  }
}

// The same for a few tokens: one warp per (token, output), the inputs of a part dealt to its
// lanes; the matrices as stored, [blocks][out][in].
__global__ void rglru_gates_rows_kernel(const float* __restrict__ u, long long u_stride, int part, int width,
                                        const float* __restrict__ wa, const float* __restrict__ ba,
                                        const float* __restrict__ wi, const float* __restrict__ bi,
                                        const float* __restrict__ lam, float decay_scale, float* __restrict__ a_out,
                                        float* __restrict__ b_out, long long ab_stride) {
  allow_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int t = blockIdx.y;
  if (c >= width) return;
  const int blk = c / part, o = c - blk * part;
  const float* ur = u + (size_t)t * u_stride + (size_t)blk * part;
  const float* war = wa + ((size_t)blk * part + o) * part;
  const float* wir = wi + ((size_t)blk * part + o) * part;
  float ar = 0.f, ai = 0.f;
#pragma unroll 4
  for (int i = lane; i < part; i += 32) {
    const float uv = ur[i];
    ar = fmaf(war[i], uv, ar);
    ai = fmaf(wir[i], uv, ai);
  }
  ar = warp_sum(ar) + ba[c];
  ai = warp_sum(ai) + bi[c];
  if (lane == 0) {
    const float r = sq_sigmoid(ar), g = sq_sigmoid(ai);
    const float log_a = -decay_scale * r * sq_softplus(lam[c]);
    a_out[(size_t)t * ab_stride + c] = expf(log_a);
    b_out[(size_t)t * ab_stride + c] = sqrtf(fmaxf(-expm1f(2.0f * log_a), 0.f)) * g * ur[o];
  }
}

// S <- a S + b over a sequence's tokens; out = S * gelu(y).  One thread per (channel, sequence).
template <typename T>
__global__ void rglru_scan_kernel(const float* __restrict__ a_in, const float* __restrict__ b_in,
                                  long long ab_stride, const T* __restrict__ y, long long y_stride, int width,
                                  float* __restrict__ state, long long state_stride, T* __restrict__ out,
                                  long long out_stride, const int* __restrict__ q_start,
                                  const int* __restrict__ q_len, const int* __restrict__ seq_slots, int y_act) {
  allow_dependents();
  grid_dependency_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= width) return;
  const int n = q_len[s], start = q_start[s];
  if (n <= 0) return;
  float* st = state + (size_t)seq_slots[s] * state_stride + c;
  float S = *st;
  int i = 0;
  for (; i + 4 <= n; i += 4) {
    float a[4], b[4], yv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const size_t row = (size_t)(start + i + k);
      a[k] = a_in[row * ab_stride + c];
      b[k] = b_in[row * ab_stride + c];
      yv[k] = to_float(y[row * y_stride + c]);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      S = fmaf(a[k], S, b[k]);
      out[(size_t)(start + i + k) * out_stride + c] = from_float<T>(S * sq_act(yv[k], y_act));
    }
  }
  for (; i < n; ++i) {
    const size_t row = (size_t)(start + i);
    S = fmaf(a_in[row * ab_stride + c], S, b_in[row * ab_stride + c]);
    out[row * out_stride + c] = from_float<T>(S * sq_act(to_float(y[row * y_stride + c]), y_act));
  }
  *st = S;
}

// The same recurrence for long portions, in two launches over chunks of RG_CHUNK tokens: first
// every chunk's product of decays and its result from a zero state (and, for a sequence's first
// chunk, a copy of the state it starts from); then every chunk finds its starting state by
// folding the chunks before it, in order, and runs its tokens.  The chunks of sequence s lie at
// places q_start[s] / RG_CHUNK + s + c of the summaries.
constexpr int RG_CHUNK = 64;

__global__ void rglru_chunk_kernel(const float* __restrict__ a_in, const float* __restrict__ b_in,
                                   long long ab_stride, int width, const float* __restrict__ state,
                                   long long state_stride, float* __restrict__ prod, float* __restrict__ part,
                                   float* __restrict__ init, const int* __restrict__ q_start,
                                   const int* __restrict__ q_len, const int* __restrict__ seq_slots) {
  allow_dependents();
  grid_dependency_wait();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int c = blockIdx.y, s = blockIdx.z;
  const int n = q_len[s], start = q_start[s];
  if (ch >= width || c * RG_CHUNK >= n) return;
  const int lo = c * RG_CHUNK, hi = min(n, lo + RG_CHUNK);
  float P = 1.f, Q = 0.f;
  for (int i = lo; i < hi; ++i) {
    const size_t row = (size_t)(start + i);
    const float a = a_in[row * ab_stride + ch];
    Q = fmaf(a, Q, b_in[row * ab_stride + ch]);
    P *= a;
  }
  const size_t place = (size_t)(start / RG_CHUNK + s + c);
  prod[place * width + ch] = P;
  part[place * width + ch] = Q;
  if (c == 0) init[(size_t)s * width + ch] = state[(size_t)seq_slots[s] * state_stride + ch];
}

template <typename T>
__global__ void rglru_apply_kernel(const float* __restrict__ a_in, const float* __restrict__ b_in,
                                   long long ab_stride, const T* __restrict__ y, long long y_stride, int width,
                                   float* __restrict__ state, long long state_stride,
                                   const float* __restrict__ prod, const float* __restrict__ part,
                                   const float* __restrict__ init, T* __restrict__ out, long long out_stride,
                                   const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ seq_slots, int y_act) {
  allow_dependents();
  grid_dependency_wait();
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  const int c = blockIdx.y, s = blockIdx.z;
  const int n = q_len[s], start = q_start[s];
  if (ch >= width || c * RG_CHUNK >= n) return;
  const size_t first = (size_t)(start / RG_CHUNK + s);
  float S = init[(size_t)s * width + ch];
  for (int k = 0; k < c; ++k) S = fmaf(prod[(first + k) * width + ch], S, part[(first + k) * width + ch]);
  const int lo = c * RG_CHUNK, hi = min(n, lo + RG_CHUNK);
  for (int i = lo; i < hi; ++i) {
    const size_t row = (size_t)(start + i);
    S = fmaf(a_in[row * ab_stride + ch], S, b_in[row * ab_stride + ch]);
    out[row * out_stride + ch] = from_float<T>(S * sq_act(to_float(y[row * y_stride + ch]), y_act));
  }
  if (hi == n) state[(size_t)seq_slots[s] * state_stride + ch] = S;
}

// ---------------------------------------------------------------------------------------------
// State-space recurrence with a scalar decay per head.  The columns of a head's state (one per
// value dim p) never meet: y[p] = sum_n S[n, p] C[n].  A block takes SSD_WARPS * 32 / RL columns of
// one head of one sequence; RL lanes of a warp share a column, each keeping up to SSD_NS state
// rows of it in registers, and their shares of y meet by warp shuffles, so the token loop has no
// block barrier.  Tokens are taken SSD_TC at a time: their B, C, x and dt go to shared memory
// together, the next ones while these are used (two buffers).
constexpr int SSD_NS = 16;
constexpr int SSD_TC = 16;
constexpr int SSD_WARPS = 4;

// Long portions run in chunks of SSD_CHUNK tokens side by side, in three launches: every chunk
// from a zero state, keeping its last state and the product of its decays (mode 1); per sequence
// the chunks' starting states, folded in order, and the sequence's new state (ssd_combine_kernel);
// every chunk again from its starting state, writing y (mode 2).  Mode 0 is a whole sequence in
// one block: from the slot's state, writing y and the state.  The chunks of sequence s lie at
// places q_start[s] / SSD_CHUNK + s + c.
constexpr int SSD_CHUNK = 256;
constexpr int SSD_SLICE = SSD_NS + 4;  // a lane's B (C) values in shared memory: padded against bank conflicts

template <typename T, int RL, int MODE>
__global__ void __launch_bounds__(SSD_WARPS * 32) ssd_scan_kernel(
    const float* __restrict__ xbc, long long xbc_stride, const T* __restrict__ dt_in, long long dt_stride,
    const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
    float* __restrict__ state, long long state_stride, float* __restrict__ y_out, long long y_stride, int heads,
    int groups, int N, int P, int col_blocks, const int* __restrict__ q_start, const int* __restrict__ q_len,
    const int* __restrict__ seq_slots, float* __restrict__ chunk_states, float* __restrict__ chunk_decay) {
  constexpr int mode = MODE;
  extern __shared__ __align__(16) float ssd_s[];
  allow_dependents();
  grid_dependency_wait();
  constexpr int COLS = SSD_WARPS * 32 / RL;  // columns of a block
  const int h = blockIdx.x / col_blocks, p0 = (blockIdx.x - h * col_blocks) * COLS;
  const int s = blockIdx.y;
  const int seq_tokens = q_len[s], seq_start = q_start[s];
  const int lo = mode == 0 ? 0 : (int)blockIdx.z * SSD_CHUNK;
  if (lo >= seq_tokens) return;
  const int n_tok = mode == 0 ? seq_tokens : min(SSD_CHUNK, seq_tokens - lo);
  const int start = seq_start + lo;
  const size_t place = (size_t)(seq_start / SSD_CHUNK + s) + blockIdx.z;
  const int tid = threadIdx.x;
  const int r = tid % RL, col = tid / RL, p = p0 + col;
  const bool live = p < P;
  const int g = h / (heads / groups);
  const int inner = heads * P;
  constexpr int NP = RL * SSD_NS;      // state rows a block's lanes hold
  constexpr int NPP = RL * SSD_SLICE;  // their places in shared memory
  // Two buffers of: B [TC][NPP], C [TC][NPP], x [TC][COLS], dt [TC], decay [TC].
  const int buf_floats = 2 * SSD_TC * NPP + SSD_TC * COLS + 2 * SSD_TC;
  float* st = mode == 0 ? state + (size_t)seq_slots[s] * state_stride + (size_t)h * N * P
                        : chunk_states + (place * heads + h) * (size_t)N * P;
  float S[SSD_NS];
#pragma unroll
  for (int k = 0; k < SSD_NS; ++k) {
    const int n = r * SSD_NS + k;
    S[k] = (mode != 1 && live && n < N) ? st[(size_t)n * P + p] : 0.f;
  }
  const float neg_a = -expf(a_log[h]);
  const float bias = dt_bias[h], dskip = d_skip[h];
  float decay_product = 1.f;
  // What a thread fetches of the next tokens while these are used: it waits for the values only
  // when it puts them into the other buffer, after the token loop.
  constexpr int THREADS = SSD_WARPS * 32;
  constexpr int BC_PER = 2 * SSD_TC * NP / THREADS;
  constexpr int X_PER = (SSD_TC * COLS + THREADS - 1) / THREADS;
  float pre_bc[BC_PER], pre_x[X_PER], pre_dt = 0.f;
  auto fetch = [&](int i0) {
    const int tc = min(SSD_TC, n_tok - i0);
#pragma unroll
    for (int u = 0; u < BC_PER; ++u) {
      const int idx = tid + u * THREADS;
      const int arr = idx / (SSD_TC * NP), rem = idx - arr * (SSD_TC * NP);
      const int k = rem / NP, n = rem - k * NP;
      pre_bc[u] = (k < tc && n < N && (mode != 1 || arr == 0))  // a pass that writes no y needs no C
                      ? xbc[(size_t)(start + i0 + k) * xbc_stride + inner + arr * groups * N + g * N + n]
                      : 0.f;
    }
#pragma unroll
    for (int u = 0; u < X_PER; ++u) {
      const int idx = tid + u * THREADS;
      const int k = idx / COLS, q = idx - k * COLS;
      pre_x[u] = (k < tc && p0 + q < P) ? xbc[(size_t)(start + i0 + k) * xbc_stride + (size_t)h * P + p0 + q] : 0.f;
    }
    if (tid < tc) pre_dt = to_float(dt_in[(size_t)(start + i0 + tid) * dt_stride + h]);
  };
  auto put = [&](float* buf) {
#pragma unroll
    for (int u = 0; u < BC_PER; ++u) {
      const int idx = tid + u * THREADS;
      const int arr = idx / (SSD_TC * NP), rem = idx - arr * (SSD_TC * NP);
      const int k = rem / NP, n = rem - k * NP;
      buf[arr * (SSD_TC * NPP) + k * NPP + (n / SSD_NS) * SSD_SLICE + (n % SSD_NS)] = pre_bc[u];
    }
    float* x_s = buf + 2 * SSD_TC * NPP;
#pragma unroll
    for (int u = 0; u < X_PER; ++u)
      if (tid + u * THREADS < SSD_TC * COLS) x_s[tid + u * THREADS] = pre_x[u];
    if (tid < SSD_TC) {
      float* dt_s = x_s + SSD_TC * COLS;
      const float dt = sq_softplus(pre_dt + bias);
      dt_s[tid] = dt;
      dt_s[SSD_TC + tid] = expf(neg_a * dt);
    }
  };
  fetch(0);
  put(ssd_s);
  __syncthreads();
  int which = 0;
  for (int i0 = 0; i0 < n_tok; i0 += SSD_TC) {
    const int tc = min(SSD_TC, n_tok - i0);
    float* buf = ssd_s + which * buf_floats;
    const bool more = i0 + SSD_TC < n_tok;
    if (more) fetch(i0 + SSD_TC);
    const float* b_s = buf;
    const float* c_s = b_s + SSD_TC * NPP;
    const float* x_s = c_s + SSD_TC * NPP;
    const float* dt_s = x_s + SSD_TC * COLS;
    for (int k = 0; k < tc; ++k) {
      const float dt = dt_s[k], decay = dt_s[SSD_TC + k];
      const float xv = x_s[k * COLS + col];
      const float xin = dt * xv;
      decay_product *= decay;
      const float4* b4 = reinterpret_cast<const float4*>(b_s + k * NPP + r * SSD_SLICE);
      const float4* c4 = reinterpret_cast<const float4*>(c_s + k * NPP + r * SSD_SLICE);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < SSD_NS / 4; ++j) {
        const float4 bv = b4[j];
        const float4 cv = mode != 1 ? c4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
        S[4 * j] = fmaf(decay, S[4 * j], bv.x * xin);
        S[4 * j + 1] = fmaf(decay, S[4 * j + 1], bv.y * xin);
        S[4 * j + 2] = fmaf(decay, S[4 * j + 2], bv.z * xin);
        S[4 * j + 3] = fmaf(decay, S[4 * j + 3], bv.w * xin);
        if (mode != 1) {
          acc[0] = fmaf(S[4 * j], cv.x, acc[0]);
          acc[1] = fmaf(S[4 * j + 1], cv.y, acc[1]);
          acc[2] = fmaf(S[4 * j + 2], cv.z, acc[2]);
          acc[3] = fmaf(S[4 * j + 3], cv.w, acc[3]);
        }
      }
      if (mode != 1) {
        float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
        for (int off = RL / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (r == 0 && live) y_out[(size_t)(start + i0 + k) * y_stride + (size_t)h * P + p] = sum + dskip * xv;
      }
    }
    if (more) put(ssd_s + (which ^ 1) * buf_floats);
    __syncthreads();  // the next tokens are in place, and these may be overwritten
    which ^= 1;
  }
  if (mode == 2) return;
  if (live) {
#pragma unroll
    for (int k = 0; k < SSD_NS; ++k) {
      const int n = r * SSD_NS + k;
      if (n < N) st[(size_t)n * P + p] = S[k];
    }
  }
  if (mode == 1 && tid == 0 && p0 == 0) chunk_decay[place * heads + h] = decay_product;
}

// Per sequence: the state its chunks start from, in order, and its new state.  In place: a
// chunk's own last state (from zero) is replaced by the state it starts from.
__global__ void ssd_combine_kernel(float* __restrict__ state, long long state_stride, float* __restrict__ chunk_states,
                                   const float* __restrict__ chunk_decay, int heads, int per_head,
                                   const int* __restrict__ q_start, const int* __restrict__ q_len,
                                   const int* __restrict__ seq_slots) {
  allow_dependents();
  grid_dependency_wait();
  const int s = blockIdx.y;
  const int n = q_len[s];
  if (n <= 0) return;
  const size_t total = (size_t)heads * per_head;
  const size_t first = (size_t)(q_start[s] / SSD_CHUNK + s);
  const int chunks = (n + SSD_CHUNK - 1) / SSD_CHUNK;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const int h = (int)(e / per_head);
    float* st = state + (size_t)seq_slots[s] * state_stride + e;
    float S = *st;
    for (int c = 0; c < chunks; ++c) {
      float* at = chunk_states + (first + c) * total + e;
      const float own = *at;
      *at = S;
      S = fmaf(chunk_decay[(first + c) * heads + h], S, own);
    }
    *st = S;
  }
}

// ---------------------------------------------------------------------------------------------
// Generalized delta rule.  Per head, with key size Dk and value size Dv, the state S is Dk x Dv:
//     w_t = exp(-decay * sigmoid(wl_t + w0)),   a_t = sigmoid(al_t + a_bias),
//     u_t = k_t / sqrt(sum(k_t^2) + key_eps)
//     S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,     o_t = S_t^T r_t
// Both middle terms read the old state.  Two kernels.
//
// delta_rule_prepare_kernel: a warp per (token, head) makes the token's vectors over the key
// channels in float32 (decay, removal rate times unit key, unit key, key, receptance) and copies
// the values, into packed rows [head][token]: [w | a u | u | k | r] of KD floats each (Dk padded
// with zeros to the lanes' rows) and then v (Dv padded to a multiple of four).  A head's rows of
// consecutive tokens are contiguous, so a tile of tokens is one bulk copy.
//
// delta_rule_scan_kernel: a column of S (one value channel) never meets another column, so a
// block takes CB columns of one head of one sequence; RL lanes share a column, each with KP rows
// of it in registers, and the two sums over the rows (u^T S and S^T r) meet by shuffles.  Every
// token waits for the token before it, and a warp alone on its scheduler issues an instruction
// every five to six cycles, so what counts is how few instructions a thread has per token: four
// rows a thread (sixteen lanes a column) for key sizes up to 128, sixteen rows beyond.  A block
// asks for more than half of an SM's shared memory, so that no two of the few blocks share an SM.  The
// tokens' packed rows come in tiles of TT tokens, one bulk copy a tile, into a ring of two stages,
// each with its mbarrier, so the next tile arrives while this one is worked through.  The state is
// stored [head][column][row]: a thread's rows are contiguous.  Every sum has a fixed order, so a
// token's result does not depend on how the sequence was cut into steps.
//
// Long portions (a step of at least two chunks of DR_CHUNK tokens) run in three launches, chunks
// side by side.  A token's transition, diag(w) - (a u) u^T, is not diagonal, so a chunk's
// transition P is a dense Dk x Dk matrix: its columns are the images of the unit vectors, that is,
// Dk more columns of state that start as the identity and see no k v^T.  Pass A (mode 1) runs every
// chunk but a portion's last from zero over Dv + Dk columns and keeps the result Z | P; the fold
// kernel makes the chunks' starting states in order, S_0 the state, S_(c+1) = P_c S_c + Z_c; pass B (mode 2) runs
// every chunk again from its start and writes the outputs, its last chunk the state.  A portion of
// one chunk skips pass A and the fold.  In this form a token's result depends, within float32
// rounding, on where its chunk began.
constexpr int DR_KP_SMALL = 4, DR_KP_LARGE = 16, DR_SMALL_MAX_DK = 128;
constexpr size_t DR_MIN_SMEM = 116 * 1024;
constexpr int DR_CHUNK = 256;

// Where chunk `chunk` of sequence `seq` keeps its Z | P and its starting state: chunks of one
// sequence begin DR_CHUNK rows apart, and later sequences begin at later rows, so the number is
// taken by nobody else; it is below ceil(tokens / DR_CHUNK) + sequences.
__device__ __forceinline__ int dr_chunk_slot(int seq, int first_row) { return first_row / DR_CHUNK + seq; }

template <typename T>
__global__ void __launch_bounds__(256)
delta_rule_prepare_kernel(const T* __restrict__ r_in, const T* __restrict__ k_in, const T* __restrict__ v_in,
                          const T* __restrict__ a_in, long long in_stride, const T* __restrict__ w_in,
                          long long w_stride, const float* __restrict__ w0, const float* __restrict__ a_bias,
                          float decay, float key_eps, float* __restrict__ packed, long long head_stride,
                          int heads, int Dk, int Dv, int KD, int Dvp, int num_tokens) {
  allow_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= (long long)num_tokens * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit - (long long)t * heads);
  const size_t hk = (size_t)h * Dk;
  const T* k_row = k_in + (size_t)t * in_stride + hk;
  float ss = 0.f;
  for (int ch = lane; ch < Dk; ch += 32) {
    const float kv = to_float(k_row[ch]);
    ss = fmaf(kv, kv, ss);
  }
  const float inv = 1.0f / sqrtf(warp_sum(ss) + key_eps);
  float* dst = packed + (size_t)h * head_stride + (size_t)t * (5 * KD + Dvp);
  for (int ch = lane; ch < KD; ch += 32) {
    float wv = 0.f, au = 0.f, u = 0.f, kv = 0.f, rv = 0.f;
    if (ch < Dk) {
      const size_t at = (size_t)t * in_stride + hk + ch;
      kv = to_float(k_row[ch]);
      rv = to_float(r_in[at]);
      u = kv * inv;
      au = sq_sigmoid(to_float(a_in[at]) + a_bias[hk + ch]) * u;
      wv = expf(-decay * sq_sigmoid(to_float(w_in[(size_t)t * w_stride + hk + ch]) + w0[hk + ch]));
    }
    dst[ch] = wv;
    dst[KD + ch] = au;
    dst[2 * KD + ch] = u;
    dst[3 * KD + ch] = kv;
    dst[4 * KD + ch] = rv;
  }
  for (int c = lane; c < Dvp; c += 32)
    dst[5 * KD + c] = c < Dv ? to_float(v_in[(size_t)t * in_stride + (size_t)h * Dv + c]) : 0.f;
}

template <int DR_KP, int RL>
__global__ void delta_rule_scan_kernel(const float* __restrict__ packed, long long head_stride,
                                       float* __restrict__ state, long long state_stride, float* __restrict__ out,
                                       long long out_stride, int Dk, int Dv, int Dvp, int CB, int TT,
                                       const int* __restrict__ q_start, const int* __restrict__ q_len,
                                       const int* __restrict__ seq_slots, int mode, int max_chunks, int heads,
                                       float* __restrict__ chunk_results, float* __restrict__ chunk_starts,
                                       int* status) {
  extern __shared__ __align__(16) float dr_smem[];
  __shared__ __align__(8) unsigned long long dr_bars[2];
  // The successor is let in when the scan is over: its blocks would share the few busy SMs'
  // issue slots with a kernel whose every token waits for the token before it.
  const int seq = blockIdx.x / max_chunks, chunk = blockIdx.x - seq * max_chunks;
  const int h = blockIdx.y, tile = blockIdx.z;
  const int n_all = q_len[seq];
  const int chunks = mode == 0 ? 1 : (n_all + DR_CHUNK - 1) / DR_CHUNK;
  // Pass A has nothing to do for a portion's last chunk (nobody starts behind it).
  if (n_all <= 0 || chunk >= chunks || (mode == 1 && chunk == chunks - 1)) {
    allow_dependents();
    return;
  }
  const int t_first = q_start[seq] + (mode == 0 ? 0 : chunk * DR_CHUNK);
  const int n = mode == 0 ? n_all : min(DR_CHUNK, n_all - chunk * DR_CHUNK);
  constexpr int KD = RL * DR_KP;
  constexpr int vec = 5 * KD;                   // floats of a token's vectors over the key channels
  const int token_floats = vec + Dvp;
  const int p = threadIdx.x % RL, c = threadIdx.x / RL;
  const int col = tile * CB + c;
  const int num_cols = mode == 1 ? Dv + Dk : Dv;  // pass A: Dk more columns carry the chunk's transition
  const bool live = col < num_cols;
  const bool value_col = col < Dv;
  const size_t safe_col = live ? col : 0;
  // Where this thread's rows come from and go to.
  float* state_rows = state + (size_t)seq_slots[seq] * state_stride + ((size_t)h * Dv + (value_col ? col : 0)) * Dk;
  const int slot_here = dr_chunk_slot(seq, t_first);
  const float* from = state_rows;
  float* mine = state_rows;
  if (mode == 1) {
    from = nullptr;
    mine = chunk_results + (((size_t)slot_here * heads + h) * (size_t)(Dv + Dk) + safe_col) * Dk;
  } else if (mode == 2 && chunks > 1) {
    // Every chunk of a cut portion starts from the fold kernel's copy, the first one too: the block
    // of the last chunk writes the state row, and nothing says that it does so after the first
    // chunk's block has read it.
    from = chunk_starts + (((size_t)slot_here * heads + h) * (size_t)Dv + safe_col) * Dk;
    if (chunk < chunks - 1) mine = nullptr;  // only a portion's last chunk leaves the state behind
  }
  const uint32_t bar0 = smem_u32(&dr_bars[0]), bar1 = smem_u32(&dr_bars[1]);
  if (threadIdx.x == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar1, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  const int num_tiles = (n + TT - 1) / TT;
  const float* src_base = packed + (size_t)h * head_stride + (size_t)t_first * token_floats;
  auto issue = [&](int index) {
    const int stage = index & 1;
    const int tt = min(TT, n - index * TT);
    const uint32_t bar = stage ? bar1 : bar0;
    const uint32_t bytes = (uint32_t)tt * (uint32_t)token_floats * 4u;
    mbar_expect_tx(bar, bytes);
    bulk_copy_g2s(smem_u32(dr_smem + (size_t)stage * TT * token_floats),
                  src_base + (size_t)index * TT * token_floats, bytes, bar);
  };
  grid_dependency_wait();
  if (threadIdx.x == 0) {
    issue(0);
    if (num_tiles > 1) issue(1);
  }
  float S[DR_KP];
#pragma unroll
  for (int q = 0; q < DR_KP; ++q) {
    const int row = p * DR_KP + q;
    if (from != nullptr) S[q] = (live && row < Dk) ? from[row] : 0.f;
    else S[q] = (live && !value_col && row == col - Dv) ? 1.f : 0.f;  // zero, or a column of the identity
  }
  // One pass over the rows per token makes both sums that read the state as it is before the
  // token's update: u_t^T S for this token and S^T r for the token before (whose update is the last
  // one S has seen).  Their shuffle trees run side by side.  `pending` says that a token's output is
  // still to be made; r_prev are its receptance values for this thread's rows.
  float r_prev[DR_KP];
#pragma unroll
  for (int q = 0; q < DR_KP; ++q) r_prev[q] = 0.f;
  bool pending = false;
  int pending_row = 0;
  for (int index = 0; index < num_tiles; ++index) {
    const int stage = index & 1;
    const int tt = min(TT, n - index * TT);
    mbar_wait(stage ? bar1 : bar0, (uint32_t)(index >> 1) & 1u, status);
    const float* buf = dr_smem + (size_t)stage * TT * token_floats;
    const float* tok = buf + p * DR_KP;
    int row_now = t_first + index * TT;
#pragma unroll 2
    for (int i = 0; i < tt; ++i, tok += token_floats, ++row_now) {
      const float4* w4 = reinterpret_cast<const float4*>(tok);
      const float4* a4 = reinterpret_cast<const float4*>(tok + KD);
      const float4* u4 = reinterpret_cast<const float4*>(tok + 2 * KD);
      const float4* k4 = reinterpret_cast<const float4*>(tok + 3 * KD);
      const float4* r4 = reinterpret_cast<const float4*>(tok + 4 * KD);
      float us0 = 0.f, us1 = 0.f, us2 = 0.f, us3 = 0.f;
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int q = 0; q < DR_KP / 4; ++q) {
        const float4 u = u4[q];
        us0 = fmaf(u.x, S[4 * q], us0);
        us1 = fmaf(u.y, S[4 * q + 1], us1);
        us2 = fmaf(u.z, S[4 * q + 2], us2);
        us3 = fmaf(u.w, S[4 * q + 3], us3);
        o0 = fmaf(S[4 * q], r_prev[4 * q], o0);
        o1 = fmaf(S[4 * q + 1], r_prev[4 * q + 1], o1);
        o2 = fmaf(S[4 * q + 2], r_prev[4 * q + 2], o2);
        o3 = fmaf(S[4 * q + 3], r_prev[4 * q + 3], o3);
      }
      float us = (us0 + us1) + (us2 + us3);
      float o = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        if (off < RL) {
          us += __shfl_xor_sync(0xffffffffu, us, off);
          o += __shfl_xor_sync(0xffffffffu, o, off);
        }
      }
      if (pending && mode != 1 && live && p == 0) out[(size_t)pending_row * out_stride + (size_t)h * Dv + col] = o;
      const float vj = value_col ? tok[vec - p * DR_KP + col] : 0.f;
#pragma unroll
      for (int q = 0; q < DR_KP / 4; ++q) {
        const float4 w = w4[q], a = a4[q], k = k4[q], r = r4[q];
        S[4 * q] = fmaf(w.x, S[4 * q], fmaf(-a.x, us, k.x * vj));
        S[4 * q + 1] = fmaf(w.y, S[4 * q + 1], fmaf(-a.y, us, k.y * vj));
        S[4 * q + 2] = fmaf(w.z, S[4 * q + 2], fmaf(-a.z, us, k.z * vj));
        S[4 * q + 3] = fmaf(w.w, S[4 * q + 3], fmaf(-a.w, us, k.w * vj));
        r_prev[4 * q] = r.x;
        r_prev[4 * q + 1] = r.y;
        r_prev[4 * q + 2] = r.z;
        r_prev[4 * q + 3] = r.w;
      }
      pending = true;
      pending_row = row_now;
    }
    __syncthreads();  // every thread is done with this stage before it is filled again
    if (threadIdx.x == 0 && index + 2 < num_tiles) issue(index + 2);
  }
  {
    // The last token's output, from the state as it is now.
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int q = 0; q < DR_KP / 4; ++q) {
      o0 = fmaf(S[4 * q], r_prev[4 * q], o0);
      o1 = fmaf(S[4 * q + 1], r_prev[4 * q + 1], o1);
      o2 = fmaf(S[4 * q + 2], r_prev[4 * q + 2], o2);
      o3 = fmaf(S[4 * q + 3], r_prev[4 * q + 3], o3);
    }
    float o = (o0 + o1) + (o2 + o3);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      if (off < RL) o += __shfl_xor_sync(0xffffffffu, o, off);
    if (pending && mode != 1 && live && p == 0) out[(size_t)pending_row * out_stride + (size_t)h * Dv + col] = o;
  }
  allow_dependents();
  if (live && mine != nullptr) {
#pragma unroll
    for (int q = 0; q < DR_KP; ++q) {
      const int row = p * DR_KP + q;
      if (row < Dk) mine[row] = S[q];
    }
  }
}

// The chunks' starting states, in order: S_(c+1) = P_c S_c + Z_c with S_0 the sequence's state.  A
// block takes some value columns of one head of one sequence and keeps them in shared memory;
// thread (row k, column j) sums over the rows i of S in rising order, reading column i of P, which is
// stored as a run of Dk floats.
__global__ void delta_rule_fold_kernel(const float* __restrict__ state, long long state_stride,
                                       const float* __restrict__ chunk_results, float* __restrict__ chunk_starts,
                                       int Dk, int Dv, int CBF, int heads, const int* __restrict__ q_start,
                                       const int* __restrict__ q_len, const int* __restrict__ seq_slots,
                                       int stage_p) {
  extern __shared__ __align__(16) float fold_smem[];  // two buffers [CBF][Dk], then (stage_p) P [Dk][Dk]
  allow_dependents();
  const int seq = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * CBF;
  const int n_all = q_len[seq];
  const int chunks = (n_all + DR_CHUNK - 1) / DR_CHUNK;
  if (n_all <= 0 || chunks < 2) return;
  const int cols = min(CBF, Dv - col0);
  float* now = fold_smem;
  float* next = fold_smem + (size_t)CBF * Dk;
  grid_dependency_wait();
  const float* start = state + (size_t)seq_slots[seq] * state_stride + ((size_t)h * Dv + col0) * Dk;
  const int first_row = q_start[seq];
  float* first_start = chunk_starts + (((size_t)dr_chunk_slot(seq, first_row) * heads + h) * (size_t)Dv + col0) * Dk;
  for (int idx = threadIdx.x; idx < cols * Dk; idx += blockDim.x) {
    now[idx] = start[idx];
    first_start[idx] = start[idx];  // the first chunk's start is the state as the step found it
  }
  __syncthreads();
  for (int chunk = 0; chunk + 1 < chunks; ++chunk) {
    const size_t here = ((size_t)dr_chunk_slot(seq, first_row + chunk * DR_CHUNK) * heads + h) * (size_t)(Dv + Dk) * Dk;
    const float* Z = chunk_results + here + (size_t)col0 * Dk;   // [column j][row k]
    const float* P = chunk_results + here + (size_t)Dv * Dk;     // [column i][row k]; 16-byte aligned when Dk % 4 == 0
    float* dst = chunk_starts +
                 (((size_t)dr_chunk_slot(seq, first_row + (chunk + 1) * DR_CHUNK) * heads + h) * (size_t)Dv + col0) * Dk;
    if (stage_p) {
      // The chunk's transition into shared memory, every load under way at once.
      float* staged = fold_smem + 2 * (size_t)CBF * Dk;
      for (int idx = threadIdx.x * 4; idx < Dk * Dk; idx += blockDim.x * 4)
        *reinterpret_cast<float4*>(staged + idx) = *reinterpret_cast<const float4*>(P + idx);
      __syncthreads();
      P = staged;
    }
    // Four outputs a thread at a time, so that the loads of P (global memory, one per row i) of
    // several rows are under way together: a single output's sum would wait for each in turn.
    for (int base = threadIdx.x; base < cols * Dk; base += 4 * blockDim.x) {
      int j[4], k[4];
      float acc[4];
#pragma unroll
      for (int o = 0; o < 4; ++o) {
        const int idx = min(base + o * (int)blockDim.x, cols * Dk - 1);
        j[o] = idx / Dk;
        k[o] = idx - j[o] * Dk;
        acc[o] = Z[idx];
      }
#pragma unroll 8
      for (int i = 0; i < Dk; ++i) {
#pragma unroll
        for (int o = 0; o < 4; ++o) acc[o] = fmaf(P[(size_t)i * Dk + k[o]], now[j[o] * Dk + i], acc[o]);
      }
#pragma unroll
      for (int o = 0; o < 4; ++o) {
        const int idx = base + o * (int)blockDim.x;
        if (idx < cols * Dk) {
          next[idx] = acc[o];
          dst[idx] = acc[o];
        }
      }
    }
    __syncthreads();
    float* swap = now;
    now = next;
    next = swap;
  }
}

// out[t, part] = (y * silu(z)) / rms over the part * w, parts of equal size.
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, long long y_stride, const T* __restrict__ z,
                                        long long z_stride, const float* __restrict__ w, float eps, int part,
                                        T* __restrict__ out, long long out_stride, int gate_after) {
  __shared__ float scratch[32];
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x, gidx = blockIdx.y;
  const size_t off = (size_t)gidx * part;
  float ss = 0.f;
  if (gate_after) {
    // The part is normed as it is; weight and sigmoid(z) come after.
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
      const float v = y[(size_t)t * y_stride + off + i];
      ss = fmaf(v, v, ss);
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
      const float v = y[(size_t)t * y_stride + off + i] * inv * w[off + i];
      out[(size_t)t * out_stride + off + i] = from_float<T>(v * sq_sigmoid(to_float(z[(size_t)t * z_stride + off + i])));
    }
    return;
  }
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float v = y[(size_t)t * y_stride + off + i] * sq_silu(to_float(z[(size_t)t * z_stride + off + i]));
    ss = fmaf(v, v, ss);
  }
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)part + eps);
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float v = y[(size_t)t * y_stride + off + i] * sq_silu(to_float(z[(size_t)t * z_stride + off + i]));
    out[(size_t)t * out_stride + off + i] = from_float<T>(v * inv * w[off + i]);
  }
}

// ---------------------------------------------------------------------------------------------
// value = scale * (a / rms(a) * wa + b / rms(b) * wb); resid += value when resid is given, else
// out = value.
template <typename T>
__global__ void dual_norm_mean_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ wa,
                                      const float* __restrict__ wb, float eps, float scale, int width,
                                      float* __restrict__ resid, T* __restrict__ out) {
  __shared__ float scratch[32];
  allow_dependents();
  grid_dependency_wait();
  const size_t base = (size_t)blockIdx.x * width;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float va = to_float(a[base + i]), vb = to_float(b[base + i]);
    sa = fmaf(va, va, sa);
    sb = fmaf(vb, vb, sb);
  }
  const float ia = rsqrtf(block_sum(sa, scratch) / (float)width + eps);
  const float ib = rsqrtf(block_sum(sb, scratch) / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = scale * (to_float(a[base + i]) * ia * wa[i] + to_float(b[base + i]) * ib * wb[i]);
    if (resid != nullptr) resid[base + i] += v;
    else out[base + i] = from_float<T>(v);
  }
}

template <typename T>
__global__ void act_rows_kernel(const T* __restrict__ x, long long x_stride, T* __restrict__ out,
                                long long out_stride, int width, long long total, int kind) {
  allow_dependents();
  grid_dependency_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / width;
    const int i = (int)(idx - t * width);
    out[t * out_stride + i] = from_float<T>(sq_act(to_float(x[t * x_stride + i]), kind));
  }
}

// bfloat16 rows whose starts and widths are whole 16-byte chunks: eight values a thread.
__global__ void act_rows_vec_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride,
                                    __nv_bfloat16* __restrict__ out, long long out_stride, int chunks,
                                    long long total, int kind) {
  allow_dependents();
  grid_dependency_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / chunks;
    const int i = (int)(idx - t * chunks) * 8;
    uint4 raw = *reinterpret_cast<const uint4*>(x + t * x_stride + i);
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(pairs[k]);
      pairs[k] = __floats2bfloat162_rn(sq_act(f.x, kind), sq_act(f.y, kind));
    }
    *reinterpret_cast<uint4*>(out + t * out_stride + i) = raw;
  }
}

template <typename T>
__global__ void residual_add_kernel(float* __restrict__ resid, const T* __restrict__ delta, long long total) {
  allow_dependents();
  grid_dependency_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x)
    resid[idx] += to_float(delta[idx]);
}

// resid[t, :] += sigmoid(logit[t]) * x[t, :]
template <typename T>
__global__ void gated_rows_add_kernel(float* __restrict__ resid, const T* __restrict__ x, const T* __restrict__ logit,
                                      long long logit_stride, int width, long long total) {
  allow_dependents();
  grid_dependency_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / width;
    resid[idx] += sq_sigmoid(to_float(logit[t * logit_stride])) * to_float(x[idx]);
  }
}

}  // namespace vx

using namespace vx;

#define VX_BY_DTYPE(dtype, CALL)                      \
  if ((dtype) == VX_DTYPE_F32) { using T = float; CALL; } \
  else { using T = __nv_bfloat16; CALL; }

static inline int grid_for(long long total, int block) {
  long long blocks = (total + block - 1) / block;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return blocks < 1 ? 1 : (int)blocks;
}

VX_API int vx_pair_rope_cache_write(void* qkv, int dtype, long long stride, const int* positions, const float* cos_t,
                                    const float* sin_t, const int* slots, void* k_cache, void* v_cache,
                                    int num_tokens, int H, int G, int D, int rot, int max_pos, long long num_slots,
                                    int write_cache, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const dim3 grid(num_tokens, H + 2 * G);
  const int threads = D >= 128 ? 64 : 32;
  VX_BY_DTYPE(dtype, launch_pdl(pair_rope_cache_write_kernel<T>, grid, dim3(threads), 0, stream, (T*)qkv, stride,
                                positions, cos_t, sin_t, slots, (T*)k_cache, (T*)v_cache, H, G, D, rot, max_pos,
                                num_slots, write_cache, status));
  return (int)cudaGetLastError();
}

VX_API int vx_head_gate(void* out, int dtype, long long out_stride, const void* logits, long long logit_stride,
                        int num_tokens, int H, int D, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int work = H * D;
  const int threads = work >= 256 ? 256 : (work + 31) / 32 * 32;
  VX_BY_DTYPE(dtype, launch_pdl(head_gate_kernel<T>, dim3(num_tokens), dim3(threads), 0, stream, (T*)out,
                                out_stride, (const T*)logits, logit_stride, H, D));
  return (int)cudaGetLastError();
}

VX_API int vx_conv_tokens(const void* x, int dtype, long long x_stride, int channels, int taps, const float* w,
                          const float* bias, float* state, long long state_stride, float* out,
                          long long out_stride, const int* q_start, const int* q_len, const int* seq_slots,
                          int num_seqs, int token_lanes, int act, cudaStream_t stream) {
  if (num_seqs <= 0 || channels <= 0) return 0;
  if (token_lanes < 1) token_lanes = 1;
  if (token_lanes > 64) token_lanes = 64;
  const dim3 grid((channels + 127) / 128, num_seqs, token_lanes);
  VX_BY_DTYPE(dtype, launch_pdl(conv_tokens_kernel<T>, grid, dim3(128), 0, stream, (const T*)x, x_stride, channels,
                                taps, w, bias, (const float*)state, state_stride, out, out_stride, q_start, q_len,
                                seq_slots, act));
  int e = (int)cudaGetLastError();
  if (e != 0) return e;
  const dim3 grid2((channels + 127) / 128, num_seqs);
  VX_BY_DTYPE(dtype, launch_pdl(conv_state_update_kernel<T>, grid2, dim3(128), 0, stream, (const T*)x, x_stride,
                                channels, taps, state, state_stride, q_start, q_len, seq_slots));
  return (int)cudaGetLastError();
}

// wa, wi: the matrices as stored, [blocks][out][in] (used for a few tokens; may be null).
VX_API int vx_rglru_gates(const float* u, long long u_stride, int width, int blocks, const float* wa_t,
                          const float* ba, const float* wi_t, const float* bi, const float* lam, float decay_scale,
                          float* a_out, float* b_out, long long ab_stride, int num_tokens, const float* wa,
                          const float* wi, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int part = width / blocks;
  if (wa != nullptr && wi != nullptr && num_tokens <= 16) {
    launch_pdl(rglru_gates_rows_kernel, dim3((width + 7) / 8, num_tokens), dim3(256), 0, stream, u, u_stride, part,
               width, wa, ba, wi, bi, lam, decay_scale, a_out, b_out, ab_stride);
    return (int)cudaGetLastError();
  }
  const int threads = part >= 256 ? 256 : (part + 31) / 32 * 32;
  if (num_tokens <= 8) {
    constexpr int TT = 2;
    const size_t smem = sizeof(float) * TT * part;
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    launch_pdl(rglru_gates_kernel<TT>, dim3((num_tokens + TT - 1) / TT, blocks), dim3(threads), smem, stream, u,
               u_stride, part, wa_t, ba, wi_t, bi, lam, decay_scale, a_out, b_out, ab_stride, num_tokens);
  } else if (num_tokens < 128 || (size_t)32 * part * sizeof(float) > 200 * 1024) {
    constexpr int TT = 16;
    const size_t smem = sizeof(float) * TT * part;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
      cudaError_t e = cudaFuncSetAttribute(rglru_gates_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem);
      if (e != cudaSuccess) return (int)e;
      configured = smem;
    }
    launch_pdl(rglru_gates_kernel<TT>, dim3((num_tokens + TT - 1) / TT, blocks), dim3(threads), smem, stream, u,
               u_stride, part, wa_t, ba, wi_t, bi, lam, decay_scale, a_out, b_out, ab_stride, num_tokens);
  } else {
    // Long steps: 32 tokens a block, so that a block's pass over the two matrices (read from the
    // L2 by every block) serves twice the tokens.
    constexpr int TT = 32;
    const size_t smem = sizeof(float) * TT * part;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
      cudaError_t e = cudaFuncSetAttribute(rglru_gates_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem);
      if (e != cudaSuccess) return (int)e;
      configured = smem;
    }
    launch_pdl(rglru_gates_kernel<TT>, dim3((num_tokens + TT - 1) / TT, blocks), dim3(threads), smem, stream, u,
               u_stride, part, wa_t, ba, wi_t, bi, lam, decay_scale, a_out, b_out, ab_stride, num_tokens);
  }
  return (int)cudaGetLastError();
}

VX_API int vx_rglru_chunk_rows() { return RG_CHUNK; }

// scratch (float32, or null for the one-launch form): 2 * (num_tokens / RG_CHUNK + num_seqs + 1)
// * width floats for the chunks' summaries and num_seqs * width for the starting states.
VX_API int vx_rglru_scan(const float* a_in, const float* b_in, long long ab_stride, const void* y, int dtype,
                         long long y_stride, int width, float* state, long long state_stride, void* out,
                         long long out_stride, const int* q_start, const int* q_len, const int* seq_slots,
                         int num_seqs, int y_act, float* scratch, int num_tokens, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (scratch != nullptr && num_tokens > RG_CHUNK) {
    const size_t places = (size_t)(num_tokens / RG_CHUNK + num_seqs + 1);
    float* prod = scratch;
    float* part = prod + places * width;
    float* init = part + places * width;
    const dim3 grid((width + 127) / 128, (num_tokens + RG_CHUNK - 1) / RG_CHUNK, num_seqs);
    launch_pdl(rglru_chunk_kernel, grid, dim3(128), 0, stream, a_in, b_in, ab_stride, width, (const float*)state,
               state_stride, prod, part, init, q_start, q_len, seq_slots);
    VX_BY_DTYPE(dtype, launch_pdl(rglru_apply_kernel<T>, grid, dim3(128), 0, stream, a_in, b_in, ab_stride,
                                  (const T*)y, y_stride, width, state, state_stride, (const float*)prod,
                                  (const float*)part, (const float*)init, (T*)out, out_stride, q_start, q_len,
                                  seq_slots, y_act));
    return (int)cudaGetLastError();
  }
  const dim3 grid((width + 63) / 64, num_seqs);
  VX_BY_DTYPE(dtype, launch_pdl(rglru_scan_kernel<T>, grid, dim3(64), 0, stream, a_in, b_in, ab_stride,
                                (const T*)y, y_stride, width, state, state_stride, (T*)out, out_stride, q_start,
                                q_len, seq_slots, y_act));
  return (int)cudaGetLastError();
}

template <typename T, int RL>
static int launch_ssd(const float* xbc, long long xbc_stride, const void* dt_in, long long dt_stride,
                      const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                      long long state_stride, float* y_out, long long y_stride, int heads, int groups, int N, int P,
                      const int* q_start, const int* q_len, const int* seq_slots, int num_seqs, float* scratch,
                      int num_tokens, cudaStream_t stream) {
  constexpr int COLS = SSD_WARPS * 32 / RL;
  const int col_blocks = (P + COLS - 1) / COLS;
  const size_t smem = sizeof(float) * 2 * ((size_t)2 * SSD_TC * RL * SSD_SLICE + (size_t)SSD_TC * COLS + 2 * SSD_TC);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(ssd_scan_kernel<T, RL, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(ssd_scan_kernel<T, RL, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(ssd_scan_kernel<T, RL, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  const dim3 block(SSD_WARPS * 32);
  if (scratch == nullptr || num_tokens <= SSD_CHUNK) {
    launch_pdl(ssd_scan_kernel<T, RL, 0>, dim3(heads * col_blocks, num_seqs), block, smem, stream, xbc, xbc_stride,
               (const T*)dt_in, dt_stride, dt_bias, a_log, d_skip, state, state_stride, y_out, y_stride, heads, groups,
               N, P, col_blocks, q_start, q_len, seq_slots, (float*)nullptr, (float*)nullptr);
    return (int)cudaGetLastError();
  }
  const size_t places = (size_t)(num_tokens / SSD_CHUNK + num_seqs + 1);
  float* chunk_states = scratch;
  float* chunk_decay = scratch + places * heads * N * P;
  const dim3 grid(heads * col_blocks, num_seqs, (num_tokens + SSD_CHUNK - 1) / SSD_CHUNK);
  launch_pdl(ssd_scan_kernel<T, RL, 1>, grid, block, smem, stream, xbc, xbc_stride, (const T*)dt_in, dt_stride, dt_bias,
             a_log, d_skip, state, state_stride, y_out, y_stride, heads, groups, N, P, col_blocks, q_start, q_len,
             seq_slots, chunk_states, chunk_decay);
  const int per_head = N * P;
  int cblocks = (int)(((size_t)heads * per_head + 255) / 256);
  if (cblocks > 148 * 4) cblocks = 148 * 4;
  launch_pdl(ssd_combine_kernel, dim3(cblocks, num_seqs), dim3(256), 0, stream, state, state_stride, chunk_states,
             (const float*)chunk_decay, heads, per_head, q_start, q_len, seq_slots);
  launch_pdl(ssd_scan_kernel<T, RL, 2>, grid, block, smem, stream, xbc, xbc_stride, (const T*)dt_in, dt_stride, dt_bias,
             a_log, d_skip, state, state_stride, y_out, y_stride, heads, groups, N, P, col_blocks, q_start, q_len,
             seq_slots, chunk_states, chunk_decay);
  return (int)cudaGetLastError();
}

VX_API int vx_ssd_chunk_rows() { return SSD_CHUNK; }

// scratch (float32, or null: every sequence in one block per head and column block):
// (num_tokens / SSD_CHUNK + num_seqs + 1) * heads * (N * P + 1) floats.
VX_API int vx_ssd_scan(const float* xbc, long long xbc_stride, const void* dt_in, int dtype, long long dt_stride,
                       const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                       long long state_stride, float* y_out, long long y_stride, int heads, int groups, int N,
                       int P, const int* q_start, const int* q_len, const int* seq_slots, int num_seqs,
                       float* scratch, int num_tokens, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (N > 32 * SSD_NS) return (int)cudaErrorInvalidValue;
#define VX_SSD(RL)                                                                                              \
  VX_BY_DTYPE(dtype, return (launch_ssd<T, RL>(xbc, xbc_stride, dt_in, dt_stride, dt_bias, a_log, d_skip, state, \
                                               state_stride, y_out, y_stride, heads, groups, N, P, q_start,     \
                                               q_len, seq_slots, num_seqs, scratch, num_tokens, stream)))
  if (N <= SSD_NS) { VX_SSD(1); }
  if (N <= 2 * SSD_NS) { VX_SSD(2); }
  if (N <= 4 * SSD_NS) { VX_SSD(4); }
  if (N <= 8 * SSD_NS) { VX_SSD(8); }
  if (N <= 16 * SSD_NS) { VX_SSD(16); }
  VX_SSD(32);
#undef VX_SSD
}

static int dr_pow2_at_least(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

// Floats of scratch the chunked form wants for a step of up to `num_tokens` tokens of `num_seqs` sequences.
VX_API long long vx_delta_rule_chunk_scratch(int num_tokens, int num_seqs, int heads, int Dk, int Dv) {
  const long long slots = (num_tokens + DR_CHUNK - 1) / DR_CHUNK + num_seqs;
  return slots * heads * ((long long)(Dv + Dk) * Dk + (long long)Dv * Dk);
}

// Floats of one token's packed row (all heads), or -1 for a key size beyond the lanes of a warp.
static int dr_rows_per_lane(int Dk) { return Dk <= DR_SMALL_MAX_DK ? DR_KP_SMALL : DR_KP_LARGE; }

VX_API int vx_delta_rule_packed_width(int heads, int Dk, int Dv) {
  const int KP = dr_rows_per_lane(Dk);
  const int RL = dr_pow2_at_least((Dk + KP - 1) / KP);
  if (RL > 32) return -1;
  return heads * (5 * RL * KP + (Dv + 3) / 4 * 4);
}

template <int KP, int RL>
static int dr_launch_scan(const float* packed, long long head_stride, float* state, long long state_stride,
                          float* out, long long out_stride, int heads, int Dk, int Dv, int Dvp,
                          const int* q_start, const int* q_len, const int* seq_slots, int num_seqs, int mode,
                          int max_chunks, float* chunk_results, float* chunk_starts, int* status,
                          cudaStream_t stream) {
  constexpr int KD = RL * KP;
  // Columns a block: four warps' worth where the lanes allow, a whole number of warps at least.
  int CB = 128 / RL;
  if (CB > 32) CB = 32;
  if (CB < 1) CB = 1;
  const int TT = KD <= 64 ? 16 : (KD <= 128 ? 8 : 4);
  size_t smem = sizeof(float) * 2 * (size_t)TT * (5 * KD + Dvp);
  const dim3 grid(num_seqs * max_chunks, heads, ((mode == 1 ? Dv + Dk : Dv) + CB - 1) / CB);
  // Few blocks (a prompt's portion): each gets an SM of its own.  Many blocks (single tokens of
  // many sequences) share the SMs as they fit.
  static int num_sms = 0;
  if (num_sms == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device);
  }
  if ((long long)grid.x * grid.y * grid.z <= num_sms && smem < DR_MIN_SMEM) smem = DR_MIN_SMEM;
  // The kernel has a few bytes of static shared memory beside these: ask from a kilobyte below
  // the default limit on.
  static size_t limit = 0;  // one per instantiation
  if (smem + 1024 > 48 * 1024 && smem > limit) {
    cudaFuncSetAttribute(delta_rule_scan_kernel<KP, RL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    limit = smem;
  }
  launch_pdl(delta_rule_scan_kernel<KP, RL>, grid, dim3(CB * RL), smem, stream, packed, head_stride, state,
             state_stride, out, out_stride, Dk, Dv, Dvp, CB, TT, q_start, q_len, seq_slots, mode, max_chunks, heads,
             chunk_results, chunk_starts, status);
  return (int)cudaGetLastError();
}

VX_API int vx_delta_rule_scan(const void* r, const void* k, const void* v, const void* a, int dtype, long long in_stride,
                              const void* w, long long w_stride, const float* w0, const float* a_bias, float decay,
                              float key_eps, float* packed, long long packed_rows, float* state, long long state_stride,
                              float* out,
                              long long out_stride, int heads, int Dk, int Dv, const int* q_start, const int* q_len,
                              const int* seq_slots, int num_seqs, int num_tokens, float* chunk_scratch,
                              long long chunk_scratch_floats, int* status, cudaStream_t stream) {
  if (num_seqs <= 0 || num_tokens <= 0) return 0;
  if (heads <= 0 || Dk <= 0 || Dv <= 0) return (int)cudaErrorInvalidValue;
  const int KP = dr_rows_per_lane(Dk);
  const int RL = dr_pow2_at_least((Dk + KP - 1) / KP);
  if (RL > 32) return -1;
  const int KD = RL * KP, Dvp = (Dv + 3) / 4 * 4;
  if (packed_rows < num_tokens) return (int)cudaErrorInvalidValue;
  const long long packed_stride = packed_rows * (5 * KD + Dvp);  // from one head's rows to the next head's
  const long long units = (long long)num_tokens * heads;
  VX_BY_DTYPE(dtype, launch_pdl(delta_rule_prepare_kernel<T>, dim3((unsigned)((units + 7) / 8)), dim3(256), 0, stream,
                                (const T*)r, (const T*)k, (const T*)v, (const T*)a, in_stride, (const T*)w, w_stride,
                                w0, a_bias, decay, key_eps, packed, packed_stride, heads, Dk, Dv, KD, Dvp, num_tokens));
  int code = (int)cudaGetLastError();
  if (code != 0) return code;
  // Long steps run in chunks when the caller has brought the scratch for it.
  const bool chunked = num_tokens >= 2 * DR_CHUNK && chunk_scratch != nullptr &&
                       chunk_scratch_floats >= vx_delta_rule_chunk_scratch(num_tokens, num_seqs, heads, Dk, Dv);
  const int max_chunks = chunked ? (num_tokens + DR_CHUNK - 1) / DR_CHUNK : 1;
  const long long slots = (long long)max_chunks + num_seqs;
  float* chunk_results = chunk_scratch;
  float* chunk_starts = chunked ? chunk_scratch + slots * heads * (long long)(Dv + Dk) * Dk : nullptr;
  auto scan = [&](int mode) -> int {
#define VX_DR(KPV, RLV)                                                                                          \
  if (KP == KPV && RL == RLV)                                                                                    \
    return dr_launch_scan<KPV, RLV>(packed, packed_stride, state, state_stride, out, out_stride, heads, Dk, Dv, Dvp, \
                                    q_start, q_len, seq_slots, num_seqs, mode, max_chunks, chunk_results,        \
                                    chunk_starts, status, stream)
    VX_DR(DR_KP_SMALL, 1);
    VX_DR(DR_KP_SMALL, 2);
    VX_DR(DR_KP_SMALL, 4);
    VX_DR(DR_KP_SMALL, 8);
    VX_DR(DR_KP_SMALL, 16);
    VX_DR(DR_KP_SMALL, 32);
    VX_DR(DR_KP_LARGE, 16);
    VX_DR(DR_KP_LARGE, 32);
#undef VX_DR
    return -1;
  };
  if (!chunked) return scan(0);
  code = scan(1);
  if (code != 0) return code;
  const int CBF = Dk <= 128 ? 16 : 4;
  size_t fold_smem = sizeof(float) * 2 * (size_t)CBF * Dk;
  // The chunk's Dk x Dk transition beside them where it fits (and its rows are whole 16-byte packs).
  const int stage_p = Dk % 4 == 0 && fold_smem + sizeof(float) * (size_t)Dk * Dk <= 96 * 1024;
  if (stage_p) fold_smem += sizeof(float) * (size_t)Dk * Dk;
  static size_t fold_limit = 0;
  if (fold_smem > 47 * 1024 && fold_smem > fold_limit) {
    cudaFuncSetAttribute(delta_rule_fold_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fold_smem);
    fold_limit = fold_smem;
  }
  launch_pdl(delta_rule_fold_kernel, dim3(num_seqs, heads, (Dv + CBF - 1) / CBF), dim3(256), fold_smem, stream,
             (const float*)state, state_stride, (const float*)chunk_results, chunk_starts, Dk, Dv, CBF, heads, q_start,
             q_len, seq_slots, stage_p);
  code = (int)cudaGetLastError();
  if (code != 0) return code;
  return scan(2);
}

VX_API int vx_gated_group_norm(const float* y, long long y_stride, const void* z, int dtype, long long z_stride,
                               const float* w, float eps, int inner, int parts, void* out, long long out_stride,
                               int num_tokens, int gate_after, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int part = inner / parts;
  const int threads = part >= 256 ? 256 : (part + 31) / 32 * 32;
  VX_BY_DTYPE(dtype, launch_pdl(gated_group_norm_kernel<T>, dim3(num_tokens, parts), dim3(threads), 0, stream, y,
                                y_stride, (const T*)z, z_stride, w, eps, part, (T*)out, out_stride, gate_after));
  return (int)cudaGetLastError();
}

VX_API int vx_dual_norm_mean(const void* a, const void* b, int dtype, const float* wa, const float* wb, float eps,
                             float scale, int width, float* resid, void* out, int num_tokens,
                             cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  VX_BY_DTYPE(dtype, launch_pdl(dual_norm_mean_kernel<T>, dim3(num_tokens), dim3(threads), 0, stream, (const T*)a,
                                (const T*)b, wa, wb, eps, scale, width, resid, (T*)out));
  return (int)cudaGetLastError();
}

VX_API int vx_act_rows(const void* x, int dtype, long long x_stride, void* out, long long out_stride, int width,
                       int num_tokens, int kind, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const long long total = (long long)num_tokens * width;
  if (dtype == VX_DTYPE_BF16 && width % 8 == 0 && x_stride % 8 == 0 && out_stride % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    launch_pdl(act_rows_vec_kernel, dim3(grid_for(total / 8, 256)), dim3(256), 0, stream, (const __nv_bfloat16*)x,
               x_stride, (__nv_bfloat16*)out, out_stride, width / 8, total / 8, kind);
    return (int)cudaGetLastError();
  }
  VX_BY_DTYPE(dtype, launch_pdl(act_rows_kernel<T>, dim3(grid_for(total, 256)), dim3(256), 0, stream, (const T*)x,
                                x_stride, (T*)out, out_stride, width, total, kind));
  return (int)cudaGetLastError();
}

VX_API int vx_residual_add(float* resid, const void* delta, int dtype, long long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  VX_BY_DTYPE(dtype, launch_pdl(residual_add_kernel<T>, dim3(grid_for(total, 256)), dim3(256), 0, stream, resid,
                                (const T*)delta, total));
  return (int)cudaGetLastError();
}

VX_API int vx_gated_rows_add(float* resid, const void* x, const void* logit, int dtype, long long logit_stride,
                             int width, int num_tokens, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const long long total = (long long)num_tokens * width;
  VX_BY_DTYPE(dtype, launch_pdl(gated_rows_add_kernel<T>, dim3(grid_for(total, 256)), dim3(256), 0, stream, resid,
                                (const T*)x, (const T*)logit, logit_stride, width, total));
  return (int)cudaGetLastError();
}
