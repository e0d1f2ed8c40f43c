// Row kernels around attention heads and gated feed-forwards (the `heads` library; float32 and
// bfloat16 instantiations of each):
//
//   norm_shift_kernel        one RMS statistic per row, two weighted outputs; the first output is
//                            mixed with the previous token's (token shift), whose last value per
//                            request lives in a slot-indexed state row
//   norm_conv_kernel         RMS norm, then h + a causal convolution of h over the request's
//                            tokens per channel; the last taps - 1 values of h per request live
//                            in a slot-indexed state row
//   add_rows_kernel          stream += scale_a * a (+ scale_b * b), float32 sums
//   diff_prepare_kernel      differential attention: per (head, map) RMS norm of q and k, rotation
//                            of the first dims of every map, q into a buffer whose "heads" are
//                            (head, map) pairs with the map's dims at the map's offset, k of both
//                            maps side by side into one cached row, v into its page
//   diff_combine_kernel      o = a1 - lambda a2, unit RMS over the head, times (1 - lambda_init),
//                            times sigmoid(gate)
//   clamped_glu_kernel       g = min(g, limit), u = clamp(u, +-limit),
//                            g sigmoid(alpha (g + cubic g^3)) (u + shift)
//
// Everything between the loads and the stores is float32.  Every sum has an order that depends
// on the sizes only.
#include "common.cuh"

#include <math_constants.h>

namespace vx {

__device__ __forceinline__ float hd_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
// For outputs that are rounded to bfloat16: the special-function unit's exponential and reciprocal
// (relative error about 2^-21), a fifth of the instructions.  float32 outputs keep the accurate one.
template <typename T>
__device__ __forceinline__ float sigmoid_for(float v) {
  if constexpr (sizeof(T) == 2) return __fdividef(1.0f, 1.0f + __expf(-v));
  else return hd_sigmoid(v);
}

// Sixteen bytes of a row at a time: four float32 or eight bfloat16, as floats.
template <typename T>
struct Pack {
  static constexpr int N = 16 / (int)sizeof(T);
};
__device__ __forceinline__ void load_pack(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x, v[1] = x.y, v[2] = x.z, v[3] = x.w;
}
__device__ __forceinline__ void load_pack(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 x = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void store_pack(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store_pack(__nv_bfloat16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------------------------------------
// Token shift.  With h_t = x_t / rms(x_t) * w1 the first output of row t is
//     h_t + (h_(t-1) - h_t) * shift
// where h_(t-1) is the same norm of the request's previous token: recomputed from row t - 1 when
// that row is in this step, read from the request's state row when t is the first row of its
// portion (zero for the first token of a request: a state row is zero when a slot is taken).
// The block of a portion's first row also writes the portion's last h into the state row, after
// it has read it, so no other block touches the row.  The second output is x_t / rms(x_t) * w2.
// One block per row.
template <typename T>
__global__ void norm_shift_kernel(const float* __restrict__ resid, long long resid_stride, int width, float eps,
                                  const float* __restrict__ w1, const float* __restrict__ w2,
                                  const float* __restrict__ shift, float* __restrict__ state,
                                  long long state_stride, T* __restrict__ out1, T* __restrict__ out2,
                                  const int* __restrict__ q_start, const int* __restrict__ q_len,
                                  const int* __restrict__ seq_slots, int num_seqs) {
  __shared__ float scratch[32];
  allow_dependents();
  const int t = blockIdx.x;
  // Which request's row this is (rows of no request: padding of a rounded step).
  int seq = -1, first = 0, last = 0;
  for (int s = 0; s < num_seqs; ++s) {
    const int b = q_start[s], n = q_len[s];
    if (n > 0 && t >= b && t < b + n) {
      seq = s;
      first = b;
      last = b + n - 1;
    }
  }
  grid_dependency_wait();
  const float* x = resid + (size_t)t * resid_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) ss += x[i] * x[i];
  const float r = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
  const bool shifted = shift != nullptr;
  const float* prev_x = nullptr;
  const float* prev_h = nullptr;
  float prev_r = 0.f;
  if (shifted && seq >= 0) {
    if (t > first) {
      prev_x = x - resid_stride;
      float ps = 0.f;
      for (int i = threadIdx.x; i < width; i += blockDim.x) ps += prev_x[i] * prev_x[i];
      prev_r = rsqrtf(block_sum(ps, scratch) / (float)width + eps);
    } else {
      prev_h = state + (size_t)seq_slots[seq] * state_stride;
    }
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float n = x[i] * r;
    float h = n * w1[i];
    if (shifted) {
      const float before = prev_x != nullptr ? prev_x[i] * prev_r * w1[i] : (prev_h != nullptr ? prev_h[i] : 0.f);
      h = h + (before - h) * shift[i];
    }
    out1[(size_t)t * width + i] = from_float<T>(h);
    if (w2 != nullptr) out2[(size_t)t * width + i] = from_float<T>(n * w2[i]);
  }
  if (shifted && seq >= 0 && t == first) {
    // The portion's last row, normed once more, is what the next step's first row looks back at.
    __syncthreads();
    const float* xl = resid + (size_t)last * resid_stride;
    float ls = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ls += xl[i] * xl[i];
    const float lr = rsqrtf(block_sum(ls, scratch) / (float)width + eps);
    float* dst = state + (size_t)seq_slots[seq] * state_stride;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = xl[i] * lr * w1[i];
  }
}

// ---------------------------------------------------------------------------------------------
// Input convolution.  With h_t = x_t / rms(x_t) * w the output of row t is
//     h_t + sum_j cw[:, j] * h_(t - taps + 1 + j),   j = 0 .. taps - 1
// over the request's own tokens, zeros before its first token.  h of a token of this step is
// recomputed from its row of the stream; h of the taps - 1 tokens before the portion comes from the
// request's state row [(taps - 1) x width] (oldest first; zero when a slot is taken).  A value of h
// is the same float whether it was recomputed or stored: a row's sum of squares is made by one
// warp in one order, and the products x * r * w one by one.
// A block takes a tile of NC_ROWS rows of one portion: its warps make the inverse root mean square
// of the tile's rows and of the taps - 1 rows before them, then all threads write the tile's
// outputs.  The block of a portion's first tile is the only one that reads the state row, and it
// writes the portion's last taps - 1 values of h there when its outputs are done (entries of a
// portion shorter than that move up).  A portion of one token (decode) moves its channels' entries up
// and appends its h in the same loop that writes its output: a thread holds them all.  Rows of no request (padding of a rounded step, behind the
// sequences' rows) come in tiles of rows without history.  The taps are given transposed, [taps x
// width], so that a tap of neighbouring channels is one load.
constexpr int NC_MAX_TAPS = 8;
constexpr int NC_ROWS = 8;

__device__ __forceinline__ float nc_value(float x, float r, float w) { return __fmul_rn(__fmul_rn(x, r), w); }

// By one warp: lanes take every 32nd element (or every 32nd pack of four), then the shuffle tree.
__device__ __forceinline__ float nc_inverse_rms(const float* __restrict__ x, int width, float eps, bool vec) {
  const int lane = threadIdx.x & 31;
  float ss = 0.f;
  if (vec) {
    for (int i = lane * 4; i < width; i += 128) {
      const float4 v = *reinterpret_cast<const float4*>(x + i);
      ss = fmaf(v.x, v.x, ss);
      ss = fmaf(v.y, v.y, ss);
      ss = fmaf(v.z, v.z, ss);
      ss = fmaf(v.w, v.w, ss);
    }
  } else {
    // The same elements per lane and the same order as the vector form.
    for (int i = lane * 4; i < width; i += 128)
      for (int e = 0; e < 4 && i + e < width; ++e) ss = fmaf(x[i + e], x[i + e], ss);
  }
  return rsqrtf(warp_sum(ss) / (float)width + eps);
}

template <typename T>
__global__ void __launch_bounds__(256)
norm_conv_kernel(const float* __restrict__ resid, long long resid_stride, int width, float eps,
                 const float* __restrict__ w, const float* __restrict__ cw_t, int taps, float* state,
                 long long state_stride, T* __restrict__ out, const int* __restrict__ q_start,
                 const int* __restrict__ q_len, const int* __restrict__ seq_slots, int num_seqs, int num_tokens,
                 int vec) {
  __shared__ float inv[NC_ROWS + 2 * NC_MAX_TAPS];
  __shared__ int seq_first[256], seq_count[256];
  allow_dependents();
  // Which tile this block has: the portions' tiles in the order of the sequences, then one tile
  // per row behind the last sequence's rows (padding).  The sequences' extents are fetched 256 at
  // a time, all at once, and then walked in shared memory.
  int seq = -1, first = 0, count = 0, tile = 0, covered = 0;
  {
    int left = blockIdx.x;
    for (int base = 0; base < num_seqs && seq < 0; base += 256) {
      const int here = min(256, num_seqs - base);
      __syncthreads();
      if ((int)threadIdx.x < here) {
        seq_first[threadIdx.x] = q_start[base + threadIdx.x];
        seq_count[threadIdx.x] = q_len[base + threadIdx.x];
      }
      __syncthreads();
      for (int s = 0; s < here && seq < 0; ++s) {
        const int n = seq_count[s];
        if (n <= 0) continue;
        const int tiles = (n + NC_ROWS - 1) / NC_ROWS;
        if (left < tiles) {
          seq = base + s;
          first = seq_first[s];
          count = n;
          tile = left;
        } else {
          left -= tiles;
        }
        covered = max(covered, seq_first[s] + n);
      }
    }
    if (seq < 0) {
      // A tile of rows without history: as if each were the first token of a portion of its own.
      first = covered;
      tile = left;
      count = num_tokens - covered;
      if (tile * NC_ROWS >= count) return;
    }
  }
  const bool lonely = seq < 0;
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, num_warps = blockDim.x >> 5;
  const int row0 = tile * NC_ROWS;                      // first row of the tile within the portion
  const int rows = min(NC_ROWS, count - row0);
  const int halo = lonely ? 0 : min(taps - 1, row0);    // rows before the tile that are in this step
  // inv[i]: row (row0 - halo + i) of the portion.
  for (int i = warp; i < halo + rows; i += num_warps) {
    const float r = nc_inverse_rms(resid + (size_t)(first + row0 - halo + i) * resid_stride, width, eps, vec != 0);
    if (lane == 0) inv[i] = r;
  }
  __syncthreads();
  const float* old_state = (seq >= 0 && taps > 1) ? state + (size_t)seq_slots[seq] * state_stride : nullptr;
  // One token of a request: its inputs from before are the whole state row, and the row after the
  // step is those entries moved up by one with the token's h behind them.
  const bool single = seq >= 0 && count == 1 && taps > 1;
  float* own_state = single ? state + (size_t)seq_slots[seq] * state_stride : nullptr;
  if (vec && (reinterpret_cast<uintptr_t>(old_state) & 15) == 0 && state_stride % 4 == 0 &&
      (reinterpret_cast<uintptr_t>(cw_t) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    // Four channels a thread: every load of a pack's taps is under way before the first product.
    const int packs = width >> 2;
    for (int idx = threadIdx.x; idx < rows * packs; idx += blockDim.x) {
      const int lr = idx / packs, i = (idx - lr * packs) << 2;
      const int row = row0 + lr;
      float4 x[NC_MAX_TAPS];
      float r[NC_MAX_TAPS];
#pragma unroll
      for (int j = 0; j < NC_MAX_TAPS; ++j) {
        if (j < taps) {
          const int src = (lonely && j < taps - 1) ? -1 : row - (taps - 1) + j;
          if (src >= 0) {
            x[j] = *reinterpret_cast<const float4*>(resid + (size_t)(first + src) * resid_stride + i);
            r[j] = inv[src - (row0 - halo)];
          } else {
            x[j] = old_state != nullptr ? *reinterpret_cast<const float4*>(old_state + (size_t)(row + j) * width + i)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
            r[j] = -1.f;  // a stored value: taken as it is
          }
        }
      }
      const float4 wi = *reinterpret_cast<const float4*>(w + i);
      float h[4] = {0.f, 0.f, 0.f, 0.f}, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < NC_MAX_TAPS; ++j) {
        if (j < taps) {
          const float4 tap = *reinterpret_cast<const float4*>(cw_t + (size_t)j * width + i);
          const float xs[4] = {x[j].x, x[j].y, x[j].z, x[j].w};
          const float ws[4] = {wi.x, wi.y, wi.z, wi.w};
          const float ts[4] = {tap.x, tap.y, tap.z, tap.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            h[c] = r[j] < 0.f ? xs[c] : nc_value(xs[c], r[j], ws[c]);
            acc[c] = fmaf(ts[c], h[c], acc[c]);
          }
        }
      }
      float result[4] = {h[0] + acc[0], h[1] + acc[1], h[2] + acc[2], h[3] + acc[3]};
      T* dst = out + (size_t)(first + row) * width + i;
#pragma unroll
      for (int c = 0; c < 4; ++c) dst[c] = from_float<T>(result[c]);
      if (single) {
#pragma unroll
        for (int j = 1; j < NC_MAX_TAPS; ++j)
          if (j < taps - 1) *reinterpret_cast<float4*>(own_state + (size_t)(j - 1) * width + i) = x[j];
        *reinterpret_cast<float4*>(own_state + (size_t)(taps - 2) * width + i) = make_float4(h[0], h[1], h[2], h[3]);
      }
    }
  } else {
    for (int idx = threadIdx.x; idx < rows * width; idx += blockDim.x) {
      const int lr = idx / width, i = idx - lr * width;
      const int row = row0 + lr;
      const float wi = w[i];
      float h = 0.f, acc = 0.f;
#pragma unroll
      for (int j = 0; j < NC_MAX_TAPS; ++j) {
        if (j < taps) {
          const int src = (lonely && j < taps - 1) ? -1 : row - (taps - 1) + j;
          if (src >= 0) h = nc_value(resid[(size_t)(first + src) * resid_stride + i], inv[src - (row0 - halo)], wi);
          else h = old_state != nullptr ? old_state[(size_t)(row + j) * width + i] : 0.f;
          acc = fmaf(cw_t[(size_t)j * width + i], h, acc);
        }
      }
      // h is now the row's own value (j = taps - 1).
      out[(size_t)(first + row) * width + i] = from_float<T>(h + acc);
      if (single) {
        for (int e = 0; e + 1 < taps - 1; ++e) own_state[(size_t)e * width + i] = own_state[(size_t)(e + 1) * width + i];
        own_state[(size_t)(taps - 2) * width + i] = h;
      }
    }
  }
  if (seq < 0 || tile != 0 || taps < 2 || single) return;
  // New state: entry e is h of portion index count - (taps - 1) + e; a negative index is the old
  // entry count + e, which lies above e, and a thread moves its own channels in rising e.
  __syncthreads();
  float* mine = state + (size_t)seq_slots[seq] * state_stride;
  const int tail0 = count - (taps - 1);                 // portion index of entry 0
  for (int e = warp; e < taps - 1; e += num_warps) {
    const int src = tail0 + e;
    if (src >= 0) {
      // A row of this tile has its statistic already (the same sum, made once).
      const float r = src < rows ? inv[src]
                                 : nc_inverse_rms(resid + (size_t)(first + src) * resid_stride, width, eps, vec != 0);
      if (lane == 0) inv[NC_ROWS + NC_MAX_TAPS + e] = r;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    // All of a channel's new entries are read before the first is written.
    float fresh[NC_MAX_TAPS];
#pragma unroll
    for (int e = 0; e < NC_MAX_TAPS - 1; ++e) {
      if (e < taps - 1) {
        const int src = tail0 + e;
        fresh[e] = src >= 0
            ? nc_value(resid[(size_t)(first + src) * resid_stride + i], inv[NC_ROWS + NC_MAX_TAPS + e], w[i])
            : mine[(size_t)(count + e) * width + i];
      }
    }
#pragma unroll
    for (int e = 0; e < NC_MAX_TAPS - 1; ++e)
      if (e < taps - 1) mine[(size_t)e * width + i] = fresh[e];
  }
}

// Two sums over a block at once; every thread gets both.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* scratch /* >= 64 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int num_warps = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  if (lane == 0) {
    scratch[warp] = a;
    scratch[32 + warp] = b;
  }
  __syncthreads();
  a = warp_sum(lane < num_warps ? scratch[lane] : 0.f);
  b = warp_sum(lane < num_warps ? scratch[32 + lane] : 0.f);
  __syncthreads();
}

__device__ __forceinline__ float sum_squares4(const float* p) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
}

// The same with sixteen bytes per access (width a multiple of the outputs' pack, every row
// 16-byte aligned): the statistics of the row and of the row before it in one pass; a portion of
// one token (decode) writes the h it has just made into the state row instead of norming the
// row a second time.
template <typename T>
__global__ void norm_shift_vec_kernel(const float* __restrict__ resid, long long resid_stride, int width, float eps,
                                      const float* __restrict__ w1, const float* __restrict__ w2,
                                      const float* __restrict__ shift, float* __restrict__ state,
                                      long long state_stride, T* __restrict__ out1, T* __restrict__ out2,
                                      const int* __restrict__ q_start, const int* __restrict__ q_len,
                                      const int* __restrict__ seq_slots, int num_seqs) {
  constexpr int N = Pack<T>::N;
  __shared__ float scratch[64];
  allow_dependents();
  const int t = blockIdx.x;
  int seq = -1, first = 0, last = 0;
  for (int s0 = 0; s0 < num_seqs; s0 += 32) {
    const int s = s0 + (threadIdx.x & 31);
    const int b = s < num_seqs ? q_start[s] : 0, n = s < num_seqs ? q_len[s] : 0;
    const unsigned hit = __ballot_sync(0xffffffffu, n > 0 && t >= b && t < b + n);
    if (hit != 0u) {
      const int src = 31 - __clz(hit);  // the last one that claims the row, as the loop form has it
      seq = s0 + src;
      first = __shfl_sync(0xffffffffu, b, src);
      last = first + __shfl_sync(0xffffffffu, n, src) - 1;
    }
  }
  grid_dependency_wait();
  const float* x = resid + (size_t)t * resid_stride;
  const bool shifted = shift != nullptr;
  const bool in_seq = shifted && seq >= 0;
  const float* prev_x = in_seq && t > first ? x - resid_stride : nullptr;
  float* own_state = in_seq && t == first ? state + (size_t)seq_slots[seq] * state_stride : nullptr;
  float ss = 0.f, ps = 0.f;
  for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
    ss += sum_squares4(x + i);
    if (prev_x != nullptr) ps += sum_squares4(prev_x + i);
  }
  block_sum2(ss, ps, scratch);
  const float r = rsqrtf(ss / (float)width + eps), prev_r = rsqrtf(ps / (float)width + eps);
  const bool state_now = own_state != nullptr && first == last;
  for (int i = threadIdx.x * N; i < width; i += blockDim.x * N) {
    float h[N], n[N], o[N];
#pragma unroll
    for (int j = 0; j < N; j += 4) {
      float xv[4], wv[4];
      load_pack(x + i + j, xv);
      load_pack(w1 + i + j, wv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        n[j + e] = xv[e] * r;
        h[j + e] = n[j + e] * wv[e];
        o[j + e] = h[j + e];
      }
      if (shifted) {
        float before[4] = {0.f, 0.f, 0.f, 0.f}, sv[4];
        if (prev_x != nullptr) {
          load_pack(prev_x + i + j, before);
#pragma unroll
          for (int e = 0; e < 4; ++e) before[e] = before[e] * prev_r * wv[e];
        } else if (own_state != nullptr) {
          load_pack(own_state + i + j, before);
        }
        load_pack(shift + i + j, sv);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j + e] = h[j + e] + (before[e] - h[j + e]) * sv[e];
      }
      if (state_now) {
        const float hv[4] = {h[j], h[j + 1], h[j + 2], h[j + 3]};
        store_pack(own_state + i + j, hv);  // read just above by this thread, by nobody else
      }
    }
    store_pack(out1 + (size_t)t * width + i, o);
    if (w2 != nullptr) {
#pragma unroll
      for (int j = 0; j < N; j += 4) {
        float wv[4];
        load_pack(w2 + i + j, wv);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j + e] = n[j + e] * wv[e];
      }
      store_pack(out2 + (size_t)t * width + i, o);
    }
  }
  if (own_state != nullptr && first != last) {
    __syncthreads();
    const float* xl = resid + (size_t)last * resid_stride;
    float ls = 0.f, unused = 0.f;
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) ls += sum_squares4(xl + i);
    block_sum2(ls, unused, scratch);
    const float lr = rsqrtf(ls / (float)width + eps);
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float xv[4], wv[4];
      load_pack(xl + i, xv);
      load_pack(w1 + i, wv);
#pragma unroll
      for (int e = 0; e < 4; ++e) xv[e] = xv[e] * lr * wv[e];
      store_pack(own_state + i, xv);
    }
  }
}

template <typename T>
__global__ void add_rows_kernel(float* __restrict__ resid, const T* __restrict__ a, const T* __restrict__ b,
                                long long count, float scale_a, float scale_b) {
  allow_dependents();
  grid_dependency_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    float v = resid[i] + scale_a * to_float(a[i]);
    if (b != nullptr) v += scale_b * to_float(b[i]);
    resid[i] = v;
  }
}

template <typename T>
__global__ void add_rows_vec_kernel(float* __restrict__ resid, const T* __restrict__ a, const T* __restrict__ b,
                                    long long packs, float scale_a, float scale_b) {
  constexpr int N = Pack<T>::N;
  allow_dependents();
  grid_dependency_wait();
  for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < packs;
       p += (long long)gridDim.x * blockDim.x) {
    const long long i = p * N;
    float av[N], bv[N];
    load_pack(a + i, av);
#pragma unroll
    for (int e = 0; e < N; ++e) av[e] *= scale_a;
    if (b != nullptr) {
      load_pack(b + i, bv);
#pragma unroll
      for (int e = 0; e < N; ++e) av[e] += scale_b * bv[e];
    }
#pragma unroll
    for (int j = 0; j < N; j += 4) {
      float xv[4];
      load_pack(resid + i + j, xv);
#pragma unroll
      for (int e = 0; e < 4; ++e) xv[e] += av[j + e];
      store_pack(resid + i + j, xv);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Differential attention, before the attention kernels.  The projection's row of token t holds
// q [H][2][dim] | k [G][2][dim] | v [G][vdim] | (further columns).  A warp takes one unit:
//   q unit (h, m): RMS norm over dim times q_norm, rotation, into qbuf[t][2 h + m][m * dim + i];
//                  the other entries of the D-wide head stay zero, so its product with the cached
//                  row [k map 0 | k map 1 | 0] is the score of map m alone
//   k unit (g, m): the same with k_norm, into k_cache[slot][g][m * dim + i]
//   v unit g     : copied into v_cache[slot][g][i]
// Rotation: dims i and i + rot / 2 (i < rot / 2) of a map are a pair that turns by the tabulated
// angle of (position, i).
template <typename T>
__global__ void diff_prepare_kernel(const T* __restrict__ proj, long long stride, T* __restrict__ qbuf,
                                    long long q_stride, const int* __restrict__ positions,
                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                    const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                    const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                    int H, int G, int dim, int vdim, int D, int rot, int max_pos,
                                    long long num_slots, int write_cache, int* status) {
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit = blockIdx.y * (blockDim.x >> 5) + warp;
  const int q_units = 2 * H, k_units = 2 * G;
  if (unit >= q_units + k_units + G) return;
  const T* row = proj + (size_t)t * stride;
  int slot = -1;
  if (unit >= q_units) {
    if (!write_cache) return;
    slot = slots[t];
    if (slot < 0) return;
    if ((long long)slot >= num_slots) {
      if (lane == 0) atomicOr(status, VX_STATUS_BAD_SLOT);
      return;
    }
  }
  if (unit >= q_units + k_units) {
    const int g = unit - q_units - k_units;
    const T* src = row + (size_t)(q_units + k_units) * dim + (size_t)g * vdim;
    T* dst = v_cache + ((size_t)slot * G + g) * D;
    for (int i = lane; i < vdim; i += 32) dst[i] = src[i];
    return;
  }
  const bool is_q = unit < q_units;
  const int u = is_q ? unit : unit - q_units;
  const int map = u & 1;
  const T* src = row + (size_t)unit * dim;  // q units first, k units right behind them
  const float* w = is_q ? q_norm : k_norm;
  int pos = positions[t];
  if (rot > 0 && (pos < 0 || pos >= max_pos)) {
    if (lane == 0 && unit == 0) atomicOr(status, VX_STATUS_BAD_POSITION);
    pos = 0;
  }
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) {
    const float v = to_float(src[i]);
    ss += v * v;
  }
  const float r = w != nullptr ? rsqrtf(warp_sum(ss) / (float)dim + eps) : 1.0f;
  T* dst = is_q ? qbuf + (size_t)t * q_stride + (size_t)unit * D + (size_t)map * dim
                : k_cache + ((size_t)slot * G + (u >> 1)) * D + (size_t)map * dim;
  const int half = rot >> 1;
  const float* c = cos_t + (size_t)pos * half;
  const float* s = sin_t + (size_t)pos * half;
  for (int i = lane; i < dim; i += 32) {
    float v = to_float(src[i]) * r * (w != nullptr ? w[i] : 1.0f);
    if (i < rot) {
      const int j = i < half ? i : i - half;
      const int other = i < half ? i + half : i - half;
      const float o = to_float(src[other]) * r * (w != nullptr ? w[other] : 1.0f);
      // (u, v) -> (u cos - v sin, v cos + u sin) for the pair (j, j + half)
      v = i < half ? v * c[j] - o * s[j] : v * c[j] + o * s[j];
    }
    dst[i] = from_float<T>(v);
  }
}

// The same with sixteen bytes per access: a unit belongs to a group of `gl` lanes (a power of two,
// at least dim / pack), so a warp takes 32 / gl units; a lane holds one pack of its unit and, in
// the rotated dims, the pack of the partner dims; every load is asked for before the group's sum.
// Wants dim, rot / 2, vdim, D and the pitches as multiples of the pack and 16-byte aligned rows.
template <typename T>
__global__ void diff_prepare_vec_kernel(const T* __restrict__ proj, long long stride, T* __restrict__ qbuf,
                                        long long q_stride, const int* __restrict__ positions,
                                        const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                        const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                        float eps, const int* __restrict__ slots, T* __restrict__ k_cache,
                                        T* __restrict__ v_cache, int H, int G, int dim, int vdim, int D, int rot,
                                        int max_pos, long long num_slots, int write_cache, int* status, int gl) {
  constexpr int N = Pack<T>::N;
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit = (blockIdx.y * (blockDim.x >> 5) + warp) * (32 / gl) + lane / gl;
  const int gi = lane % gl;
  const int q_units = 2 * H, k_units = 2 * G;
  const T* row = proj + (size_t)t * stride;
  bool active = unit < q_units + k_units + G;
  int slot = -1;
  if (active && unit >= q_units) {
    slot = write_cache ? slots[t] : -1;
    if (slot >= 0 && (long long)slot >= num_slots) {
      if (gi == 0) atomicOr(status, VX_STATUS_BAD_SLOT);
      slot = -1;
    }
    active = slot >= 0;
  }
  if (active && unit >= q_units + k_units) {
    const int g = unit - q_units - k_units;
    const T* src = row + (size_t)(q_units + k_units) * dim + (size_t)g * vdim;
    T* dst = v_cache + ((size_t)slot * G + g) * D;
    for (int i = gi * N; i < vdim; i += gl * N) {
      float v[N];
      load_pack(src + i, v);
      store_pack(dst + i, v);
    }
    active = false;
  }
  // q and k units; lanes of other units keep zeros and take part in the shuffles only.
  const bool is_q = unit < q_units;
  const int u = is_q ? unit : unit - q_units;
  const int map = u & 1;
  const int i = gi * N;
  const bool on = active && i < dim;
  const bool turned = on && i < rot;
  const int half = rot >> 1;
  const int partner = i < half ? i + half : i - half;
  const T* src = row + (size_t)unit * dim;
  const float* w = is_q ? q_norm : k_norm;
  int pos = 0;
  if (turned) {
    pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
      if (gi == 0 && unit == 0) atomicOr(status, VX_STATUS_BAD_POSITION);
      pos = 0;
    }
  }
  float x[N], o[N], wx[N], wo[N], c[N], sn[N];
#pragma unroll
  for (int e = 0; e < N; ++e) {
    x[e] = o[e] = c[e] = sn[e] = 0.f;
    wx[e] = wo[e] = 1.0f;
  }
  if (on) {
    load_pack(src + i, x);
    if (w != nullptr) {
#pragma unroll
      for (int j = 0; j < N; j += 4) {
        float part[4];
        load_pack(w + i + j, part);
#pragma unroll
        for (int e = 0; e < 4; ++e) wx[j + e] = part[e];
      }
    }
  }
  if (turned) {
    load_pack(src + partner, o);
    const int j0 = i < half ? i : i - half;
#pragma unroll
    for (int j = 0; j < N; j += 4) {
      float part[4];
      if (w != nullptr) {
        load_pack(w + partner + j, part);
#pragma unroll
        for (int e = 0; e < 4; ++e) wo[j + e] = part[e];
      }
      load_pack(cos_t + (size_t)pos * half + j0 + j, part);
#pragma unroll
      for (int e = 0; e < 4; ++e) c[j + e] = part[e];
      load_pack(sin_t + (size_t)pos * half + j0 + j, part);
#pragma unroll
      for (int e = 0; e < 4; ++e) sn[j + e] = part[e];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < N; ++e) ss += x[e] * x[e];
  for (int offset = gl >> 1; offset > 0; offset >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, offset);
  if (!on) return;
  const float r = w != nullptr ? rsqrtf(ss / (float)dim + eps) : 1.0f;
#pragma unroll
  for (int e = 0; e < N; ++e) {
    const float v = x[e] * r * wx[e];
    if (turned) {
      const float other = o[e] * r * wo[e];
      // (u, v) -> (u cos - v sin, v cos + u sin) for the pair (j, j + half)
      x[e] = i < half ? v * c[e] - other * sn[e] : v * c[e] + other * sn[e];
    } else {
      x[e] = v;
    }
  }
  T* dst = is_q ? qbuf + (size_t)t * q_stride + (size_t)unit * D + (size_t)map * dim
                : k_cache + ((size_t)slot * G + (u >> 1)) * D + (size_t)map * dim;
  store_pack(dst + i, x);
}

// After the attention kernels: attn[t][2 h + m][0 .. vdim) is map m of head h.  A warp per
// (token, head).
template <typename T>
__global__ void diff_combine_kernel(const T* __restrict__ attn, long long attn_stride, const T* __restrict__ gate,
                                    long long gate_stride, T* __restrict__ out, long long out_stride, int H,
                                    int vdim, int D, float lambda, float out_scale, float eps) {
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * (blockDim.x >> 5) + warp;
  if (h >= H) return;
  const T* a1 = attn + (size_t)t * attn_stride + (size_t)(2 * h) * D;
  const T* a2 = a1 + D;
  float ss = 0.f;
  for (int i = lane; i < vdim; i += 32) {
    const float o = to_float(a1[i]) - lambda * to_float(a2[i]);
    ss += o * o;
  }
  const float r = rsqrtf(warp_sum(ss) / (float)vdim + eps) * out_scale;
  const T* g = gate != nullptr ? gate + (size_t)t * gate_stride + (size_t)h * vdim : nullptr;
  T* dst = out + (size_t)t * out_stride + (size_t)h * vdim;
  for (int i = lane; i < vdim; i += 32) {
    float o = (to_float(a1[i]) - lambda * to_float(a2[i])) * r;
    if (g != nullptr) o *= hd_sigmoid(to_float(g[i]));
    dst[i] = from_float<T>(o);
  }
}

// The same with sixteen bytes per access (vdim, D and the pitches multiples of the pack).
template <typename T>
__global__ void diff_combine_vec_kernel(const T* __restrict__ attn, long long attn_stride, const T* __restrict__ gate,
                                        long long gate_stride, T* __restrict__ out, long long out_stride, int H,
                                        int vdim, int D, float lambda, float out_scale, float eps) {
  constexpr int N = Pack<T>::N;
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * (blockDim.x >> 5) + warp;
  if (h >= H) return;
  const T* a1 = attn + (size_t)t * attn_stride + (size_t)(2 * h) * D;
  const T* a2 = a1 + D;
  const T* g = gate != nullptr ? gate + (size_t)t * gate_stride + (size_t)h * vdim : nullptr;
  T* dst = out + (size_t)t * out_stride + (size_t)h * vdim;
  if (vdim <= 32 * N) {
    // One pack a lane: every load is asked for before the sum over the warp.
    const int i = lane * N;
    const bool on = i < vdim;
    float x[N], y[N], gv[N];
#pragma unroll
    for (int e = 0; e < N; ++e) x[e] = y[e] = gv[e] = 0.f;
    if (on) {
      load_pack(a1 + i, x);
      load_pack(a2 + i, y);
      if (g != nullptr) load_pack(g + i, gv);
    }
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < N; ++e) {
      x[e] -= lambda * y[e];
      ss += x[e] * x[e];
    }
    const float r = rsqrtf(warp_sum(ss) / (float)vdim + eps) * out_scale;
    if (on) {
#pragma unroll
      for (int e = 0; e < N; ++e) x[e] = x[e] * r * (g != nullptr ? sigmoid_for<T>(gv[e]) : 1.0f);
      store_pack(dst + i, x);
    }
    return;
  }
  float ss = 0.f;
  for (int i = lane * N; i < vdim; i += 32 * N) {
    float x[N], y[N];
    load_pack(a1 + i, x);
    load_pack(a2 + i, y);
#pragma unroll
    for (int e = 0; e < N; ++e) {
      const float o = x[e] - lambda * y[e];
      ss += o * o;
    }
  }
  const float r = rsqrtf(warp_sum(ss) / (float)vdim + eps) * out_scale;
  for (int i = lane * N; i < vdim; i += 32 * N) {
    float x[N], y[N];
    load_pack(a1 + i, x);
    load_pack(a2 + i, y);
#pragma unroll
    for (int e = 0; e < N; ++e) x[e] = (x[e] - lambda * y[e]) * r;
    if (g != nullptr) {
      load_pack(g + i, y);
#pragma unroll
      for (int e = 0; e < N; ++e) x[e] *= sigmoid_for<T>(y[e]);
    }
    store_pack(dst + i, x);
  }
}

// gate_up [tokens][2 F] (gate columns first) -> out [tokens][F].
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gate_up, long long in_stride, T* __restrict__ out,
                                   long long out_stride, int F, float limit, float alpha, float up_shift,
                                   float cubic, long long count) {
  allow_dependents();
  grid_dependency_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < count;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / F;
    const int f = (int)(idx - t * F);
    float g = to_float(gate_up[t * in_stride + f]);
    float u = to_float(gate_up[t * in_stride + F + f]);
    if (limit > 0.f) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
    }
    out[t * out_stride + f] = from_float<T>(g * hd_sigmoid(alpha * fmaf(cubic * g, g * g, g)) * (u + up_shift));
  }
}

// The same, sixteen bytes of gate and of up per thread (F and both pitches multiples of the pack).
template <typename T>
__global__ void clamped_glu_vec_kernel(const T* __restrict__ gate_up, long long in_stride, T* __restrict__ out,
                                       long long out_stride, int F, float limit, float alpha, float up_shift,
                                       float cubic) {
  constexpr int N = Pack<T>::N;
  allow_dependents();
  grid_dependency_wait();
  const T* row = gate_up + (size_t)blockIdx.y * in_stride;
  T* dst = out + (size_t)blockIdx.y * out_stride;
  for (int f = (blockIdx.x * blockDim.x + threadIdx.x) * N; f < F; f += gridDim.x * blockDim.x * N) {
    float g[N], u[N];
    load_pack(row + f, g);
    load_pack(row + F + f, u);
#pragma unroll
    for (int e = 0; e < N; ++e) {
      float gv = g[e], uv = u[e];
      if (limit > 0.f) {
        gv = fminf(gv, limit);
        uv = fminf(fmaxf(uv, -limit), limit);
      }
      g[e] = gv * sigmoid_for<T>(alpha * fmaf(cubic * gv, gv * gv, gv)) * (uv + up_shift);
    }
    store_pack(dst + f, g);
  }
}

}  // namespace vx

using namespace vx;

#define VX_BY_DTYPE(dtype, call)                  \
  if ((dtype) == VX_DTYPE_F32) {                  \
    using T = float;                              \
    call;                                         \
  } else if ((dtype) == VX_DTYPE_BF16) {          \
    using T = __nv_bfloat16;                      \
    call;                                         \
  } else {                                        \
    return (int)cudaErrorInvalidValue;            \
  }

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int row_threads(int width) {
  const int t = (width + 31) / 32 * 32;
  return t > 512 ? 512 : (t < 32 ? 32 : t);
}

VX_API int vx_norm_shift(const float* resid, long long resid_stride, int width, float eps, const float* w1,
                         const float* w2, const float* shift, float* state, long long state_stride, void* out1,
                         void* out2, int dtype, const int* q_start, const int* q_len, const int* seq_slots,
                         int num_seqs, int num_tokens, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (shift != nullptr && state == nullptr) return (int)cudaErrorInvalidValue;
  const int pack = dtype == VX_DTYPE_F32 ? 4 : 8;
  const bool vec = width % pack == 0 && resid_stride % 4 == 0 && aligned16(resid) && aligned16(w1) && aligned16(w2) &&
                   aligned16(shift) && aligned16(state) && state_stride % 4 == 0 && aligned16(out1) && aligned16(out2);
  if (vec) {
    VX_BY_DTYPE(dtype, launch_pdl(norm_shift_vec_kernel<T>, dim3(num_tokens), dim3(row_threads(width / pack)), 0, stream,
                                  resid, resid_stride, width, eps, w1, w2, shift, state, state_stride, (T*)out1,
                                  (T*)out2, q_start, q_len, seq_slots, num_seqs));
    return (int)cudaGetLastError();
  }
  VX_BY_DTYPE(dtype, launch_pdl(norm_shift_kernel<T>, dim3(num_tokens), dim3(row_threads(width)), 0, stream, resid,
                                resid_stride, width, eps, w1, w2, shift, state, state_stride, (T*)out1, (T*)out2,
                                q_start, q_len, seq_slots, num_seqs));
  return (int)cudaGetLastError();
}

VX_API int vx_norm_conv(const float* resid, long long resid_stride, int width, float eps, const float* w,
                        const float* conv_w, int taps, float* state, long long state_stride, void* out, int dtype,
                        const int* q_start, const int* q_len, const int* seq_slots, int num_seqs, int num_tokens,
                        cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (taps < 1 || taps > NC_MAX_TAPS) return -1;
  if (taps > 1 && (state == nullptr || state_stride < (long long)(taps - 1) * width)) return (int)cudaErrorInvalidValue;
  // Tiles: at most one per NC_ROWS rows, one more per sequence, and one more for the padding.
  const int blocks = (num_tokens + NC_ROWS - 1) / NC_ROWS + num_seqs + 1;
  const int vec = width % 4 == 0 && resid_stride % 4 == 0 && aligned16(resid);
  VX_BY_DTYPE(dtype, launch_pdl(norm_conv_kernel<T>, dim3(blocks), dim3(256), 0, stream, resid, resid_stride, width,
                                eps, w, conv_w, taps, state, state_stride, (T*)out, q_start, q_len, seq_slots,
                                num_seqs, num_tokens, vec));
  return (int)cudaGetLastError();
}

VX_API int vx_add_rows(float* resid, const void* a, const void* b, int dtype, long long count, float scale_a,
                       float scale_b, cudaStream_t stream) {
  if (count <= 0) return 0;
  const int pack = dtype == VX_DTYPE_F32 ? 4 : 8;
  if (count % pack == 0 && aligned16(resid) && aligned16(a) && aligned16(b)) {
    const long long packs = count / pack;
    long long vec_blocks = (packs + 255) / 256;
    if (vec_blocks > 148 * 8) vec_blocks = 148 * 8;
    VX_BY_DTYPE(dtype, launch_pdl(add_rows_vec_kernel<T>, dim3((unsigned)vec_blocks), dim3(256), 0, stream, resid,
                                  (const T*)a, (const T*)b, packs, scale_a, scale_b));
    return (int)cudaGetLastError();
  }
  long long blocks = (count + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  VX_BY_DTYPE(dtype, launch_pdl(add_rows_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, resid,
                                (const T*)a, (const T*)b, count, scale_a, scale_b));
  return (int)cudaGetLastError();
}

VX_API int vx_diff_prepare(const void* proj, int dtype, long long stride, void* qbuf, long long q_stride,
                           const int* positions, const float* cos_t, const float* sin_t, const float* q_norm,
                           const float* k_norm, float eps, const int* slots, void* k_cache, void* v_cache,
                           int num_tokens, int H, int G, int dim, int vdim, int D, int rot, int max_pos,
                           long long num_slots, int write_cache, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (2 * dim > D || vdim > D || rot > dim || (rot & 1)) return (int)cudaErrorInvalidValue;
  const int units = 2 * H + 2 * G + G;
  const int pack = dtype == VX_DTYPE_F32 ? 4 : 8;
  if (dim % pack == 0 && (rot / 2) % pack == 0 && vdim % pack == 0 && D % pack == 0 && stride % pack == 0 &&
      q_stride % pack == 0 && dim / pack <= 32 && aligned16(proj) && aligned16(qbuf) && aligned16(cos_t) &&
      aligned16(sin_t) && aligned16(q_norm) && aligned16(k_norm) && aligned16(k_cache) && aligned16(v_cache)) {
    int gl = 1;
    while (gl * pack < dim) gl *= 2;
    const int per_block = 4 * (32 / gl);
    const dim3 vec_grid(num_tokens, (units + per_block - 1) / per_block);
    VX_BY_DTYPE(dtype, launch_pdl(diff_prepare_vec_kernel<T>, vec_grid, dim3(128), 0, stream, (const T*)proj, stride,
                                  (T*)qbuf, q_stride, positions, cos_t, sin_t, q_norm, k_norm, eps, slots, (T*)k_cache,
                                  (T*)v_cache, H, G, dim, vdim, D, rot, max_pos, num_slots, write_cache, status, gl));
    return (int)cudaGetLastError();
  }
  const dim3 grid(num_tokens, (units + 3) / 4);
  VX_BY_DTYPE(dtype, launch_pdl(diff_prepare_kernel<T>, grid, dim3(128), 0, stream, (const T*)proj, stride, (T*)qbuf,
                                q_stride, positions, cos_t, sin_t, q_norm, k_norm, eps, slots, (T*)k_cache,
                                (T*)v_cache, H, G, dim, vdim, D, rot, max_pos, num_slots, write_cache, status));
  return (int)cudaGetLastError();
}

VX_API int vx_diff_combine(const void* attn, int dtype, long long attn_stride, const void* gate,
                           long long gate_stride, void* out, long long out_stride, int num_tokens, int H, int vdim,
                           int D, float lambda, float out_scale, float eps, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const dim3 grid(num_tokens, (H + 3) / 4);
  const int pack = dtype == VX_DTYPE_F32 ? 4 : 8;
  if (vdim % pack == 0 && D % pack == 0 && attn_stride % pack == 0 && gate_stride % pack == 0 &&
      out_stride % pack == 0 && aligned16(attn) && aligned16(gate) && aligned16(out)) {
    VX_BY_DTYPE(dtype, launch_pdl(diff_combine_vec_kernel<T>, grid, dim3(128), 0, stream, (const T*)attn, attn_stride,
                                  (const T*)gate, gate_stride, (T*)out, out_stride, H, vdim, D, lambda, out_scale,
                                  eps));
    return (int)cudaGetLastError();
  }
  VX_BY_DTYPE(dtype, launch_pdl(diff_combine_kernel<T>, grid, dim3(128), 0, stream, (const T*)attn, attn_stride,
                                (const T*)gate, gate_stride, (T*)out, out_stride, H, vdim, D, lambda, out_scale,
                                eps));
  return (int)cudaGetLastError();
}

VX_API int vx_clamped_glu(const void* gate_up, int dtype, long long in_stride, void* out, long long out_stride,
                          int num_tokens, int F, float limit, float alpha, float up_shift, float cubic,
                          cudaStream_t stream) {
  if (num_tokens <= 0 || F <= 0) return 0;
  const int pack = dtype == VX_DTYPE_F32 ? 4 : 8;
  if (F % pack == 0 && in_stride % pack == 0 && out_stride % pack == 0 && aligned16(gate_up) && aligned16(out) &&
      num_tokens <= 65535) {
    const int threads = 128;
    int across = (F / pack + threads - 1) / threads;
    if (across > 32) across = 32;
    VX_BY_DTYPE(dtype, launch_pdl(clamped_glu_vec_kernel<T>, dim3(across, num_tokens), dim3(threads), 0, stream,
                                  (const T*)gate_up, in_stride, (T*)out, out_stride, F, limit, alpha, up_shift, cubic));
    return (int)cudaGetLastError();
  }
  const long long count = (long long)num_tokens * F;
  long long blocks = (count + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  VX_BY_DTYPE(dtype, launch_pdl(clamped_glu_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream,
                                (const T*)gate_up, in_stride, (T*)out, out_stride, F, limit, alpha, up_shift, cubic, count));
  return (int)cudaGetLastError();
}

VX_TRACE_API(vx_heads)
