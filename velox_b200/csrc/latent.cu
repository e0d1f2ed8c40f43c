// Kernels around attention over a cached low-rank latent.
//
// The mixer caches, per token, one row [c | k_rot | 0-pad]: the normalised latent c (kv_rank
// values) and one rotated key part shared by all heads (rot_dim values).  A head's unrotated
// key is W_uk c and its value W_uv c, so with
//     q_abs[h] = W_uk[h]^T q_unrot[h]                       (kv_rank values per head)
// the score is  (q_abs[h] . c + q_rot[h] . k_rot) * scale, and the head's output is
//     W_uv[h] (sum_n p_n c_n).
// Attention itself is then multi-query attention whose single "KV head" is the cached row, with
// the same rows serving as keys and as values, and runs on the paged attention kernels.  This
// file has what comes before and after it:
//
//   latent_prepare_kernel   per token: RMS norm of the latent and interleaved-pair rotation of
//                           the shared key part, both written to the token's cache slot; the
//                           rotation of every head's q_rot into the query row [q_abs | q_rot | 0]
//   headwise_linear_kernel  out[t, h, :] = W[h] x[t, h, :] for every head, optionally times
//                           sigmoid(gate[t, h]): the absorption of W_uk into the queries and
//                           the expansion of the attention result by W_uv (FP32 pipes; the
//                           float32 path and inner sizes beyond the tensor-core form's)
//   headwise_linear_mma_kernel  the same in bfloat16 on tensor-core tiles
//
// Rotation: dims 2i and 2i + 1 of the first 2 * rot_pairs dims are a pair (u, v) ->
// (u cos a - v sin a, v cos a + u sin a), a = position * base^(-2i / (2 rot_pairs)); cos and sin
// come from float32 tables [max_pos, rot_pairs].  With `half_layout` the pair is dims i and
// i + rot_pairs instead.  Norm, rotation, sigmoid and all sums are float32.
#include "common.cuh"

namespace vx {

template <typename T>
__device__ __forceinline__ float rotated_interleaved(const T* __restrict__ x, int j, int rot_pairs,
                                                     const float* __restrict__ cos_row,
                                                     const float* __restrict__ sin_row, int half_layout = 0) {
  if (j >= 2 * rot_pairs) return to_float(x[j]);
  if (half_layout) {
    const bool second = j >= rot_pairs;
    const int i = second ? j - rot_pairs : j;
    const float u = to_float(x[i]), v = to_float(x[i + rot_pairs]);
    const float c = cos_row[i], s = sin_row[i];
    return second ? fmaf(v, c, u * s) : fmaf(u, c, -(v * s));
  }
  const int i = j >> 1;
  const float u = to_float(x[2 * i]), v = to_float(x[2 * i + 1]);
  const float c = cos_row[i], s = sin_row[i];
  return (j & 1) ? fmaf(v, c, u * s) : fmaf(u, c, -(v * s));
}

// proj [T, proj_ld]: q head h at q_off + h * (dim + R), its last R dims rotate (or, when the
// queries come from a projection of their own, in q_src [T, q_ld] at the same offset); the token's own
// latent (kr values, then R values of the shared key part) at dkv_off, or dkv_off < 0 for a layer
// that reads another layer's cache.  qa [T, H, Dp]: [kr absorbed dims (written elsewhere) | R
// rotated dims | zero pad].  cache [slots, Dp].
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ proj, long long proj_ld, const T* __restrict__ q_src,
                                      long long q_ld, int q_off, int dkv_off,
                                      const int* __restrict__ positions, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, int max_pos, int rot_pairs,
                                      const float* __restrict__ latent_w, float eps,
                                      const int* __restrict__ slots, T* __restrict__ cache, long long num_slots,
                                      T* __restrict__ qa, int H, int dim, int R, int kr, int Dp, int half_layout,
                                      int* status) {
  __shared__ float scratch[32];
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  int pos = positions[t];
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_POSITION);
    pos = 0;
  }
  const float* cos_row = cos_t + (size_t)pos * rot_pairs;
  const float* sin_row = sin_t + (size_t)pos * rot_pairs;
  const T* row = proj + (size_t)t * proj_ld;
  const T* q_row = q_src != nullptr ? q_src + (size_t)t * q_ld : row;
  const int tail = Dp - kr;
  for (int idx = threadIdx.x; idx < H * tail; idx += blockDim.x) {
    const int h = idx / tail, j = idx - h * tail;
    float v = 0.f;
    if (j < R) v = rotated_interleaved(q_row + q_off + (size_t)h * (dim + R) + dim, j, rot_pairs, cos_row, sin_row, half_layout);
    qa[((size_t)t * H + h) * Dp + kr + j] = from_float<T>(v);
  }
  if (dkv_off < 0) return;
  const T* lat = row + dkv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < kr; i += blockDim.x) {
    const float v = to_float(lat[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const long long slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_SLOT);
    return;
  }
  const float inv = 1.0f / sqrtf(ss / (float)kr + eps);
  T* dst = cache + (size_t)slot * Dp;
  for (int i = threadIdx.x; i < Dp; i += blockDim.x) {
    float v = 0.f;
    if (i < kr) v = to_float(lat[i]) * inv * latent_w[i];
    else if (i < kr + R) v = rotated_interleaved(lat + kr, i - kr, rot_pairs, cos_row, sin_row, half_layout);
    dst[i] = from_float<T>(v);
  }
}

// out[t, i] = x[t, i] / sqrt(mean_i(x[t, :n]^2) + eps) * w[i] for i < n, zero for n <= i < n_out:
// the RMS norm of a column range of a projection (a latent on the way to its second projection).
template <typename T>
__global__ void rms_rows_kernel(const T* __restrict__ x, long long x_ld, const float* __restrict__ w, float eps, int n,
                                T* __restrict__ out, long long out_ld, int n_out) {
  __shared__ float scratch[32];
  allow_dependents();
  grid_dependency_wait();
  const T* row = x + (size_t)blockIdx.x * x_ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_float(row[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
  T* dst = out + (size_t)blockIdx.x * out_ld;
  for (int i = threadIdx.x; i < n_out; i += blockDim.x)
    dst[i] = from_float<T>(i < n ? to_float(row[i]) * inv * w[i] : 0.f);
}

// out[t * out_ld + h * out_hs + n] = sum_k x[t * x_ld + h * x_hs + k] * w[(h * N + n) * K + k]
//                                    (* sigmoid(gate[t * gate_ld + h]) with a gate, or with
//                                     `gate_each` * sigmoid(gate[t * gate_ld + h * N + n]))
// One block per (tile of HL_TOKENS tokens, head); the tile's inputs are staged in shared memory
// as float32, a warp takes output n and its lanes split k, so a weight row is read once per
// block, coalesced.  Every output is summed in an order that depends on K only.
constexpr int HL_TOKENS = 8;

template <typename T>
__global__ void __launch_bounds__(256)
headwise_linear_kernel(const T* __restrict__ x, long long x_ld, int x_hs, const T* __restrict__ w,
                       T* __restrict__ out, long long out_ld, int out_hs, const T* __restrict__ gate,
                       long long gate_ld, int num_tokens, int N, int K, int gate_each) {
  extern __shared__ float xs[];  // [HL_TOKENS][K]
  allow_dependents();
  grid_dependency_wait();
  const int t0 = blockIdx.x * HL_TOKENS, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, num_warps = blockDim.x >> 5;
  for (int idx = threadIdx.x; idx < HL_TOKENS * K; idx += blockDim.x) {
    const int r = idx / K, k = idx - r * K;
    const int t = t0 + r;
    xs[idx] = t < num_tokens ? to_float(x[(size_t)t * x_ld + (size_t)h * x_hs + k]) : 0.f;
  }
  __syncthreads();
  float g[HL_TOKENS];
#pragma unroll
  for (int r = 0; r < HL_TOKENS; ++r) {
    const int t = t0 + r;
    g[r] = (gate != nullptr && !gate_each && t < num_tokens)
               ? 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_ld + h]))) : 1.0f;
  }
  for (int n = warp; n < N; n += num_warps) {
    const T* wr = w + ((size_t)h * N + n) * K;
    float acc[HL_TOKENS];
#pragma unroll
    for (int r = 0; r < HL_TOKENS; ++r) acc[r] = 0.f;
    for (int k = lane; k < K; k += 32) {
      const float wv = to_float(wr[k]);
#pragma unroll
      for (int r = 0; r < HL_TOKENS; ++r) acc[r] = fmaf(xs[r * K + k], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < HL_TOKENS; ++r) acc[r] = warp_sum(acc[r]);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < HL_TOKENS; ++r) {
        const int t = t0 + r;
        if (t < num_tokens) {
          float scale = g[r];
          if (gate != nullptr && gate_each)
            scale = 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_ld + (size_t)h * N + n])));
          out[(size_t)t * out_ld + (size_t)h * out_hs + n] = from_float<T>(acc[r] * scale);
        }
      }
    }
  }
}

// The same product on bf16 tensor-core tiles (mma.sync m16n8k16, float32 accumulators), for inner
// sizes up to HT_MAX_K: a block takes a tile of tokens of one head (16 per warp) against a range
// of outputs; inputs and the weight rows are staged in shared memory with the inner size
// zero-padded to a multiple of 16.  The work is small (two products of [T, ~100] by
// [~100, ~100] per head) and bound by its reads; what matters is that it does not run on the
// FP32 pipes when T is in the thousands.  An output's sum does not depend on T or on the tile.
constexpr int HT_MAX_K = 256;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Rows [0, rows) of a [*, K] matrix with row pitch `ld` into shared memory [*, pitch], columns
// K .. kp zeroed; 16-byte copies when `vec` says that every row starts on a 16-byte boundary and K
// is a multiple of 8.
__device__ __forceinline__ void stage_rows(__nv_bfloat16* dst, int pitch, const __nv_bfloat16* src, long long ld,
                                           int rows, int K, int kp, bool vec) {
  const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
  if (vec) {
    // Four 16-byte loads under way per thread before the first store: the copy is bound by the
    // latency of its loads, not by their number.
    const int per_row = K / 8, total = rows * per_row;
    for (int base = threadIdx.x; base < total; base += 4 * blockDim.x) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * blockDim.x;
        if (idx < total) {
          const int r = idx / per_row, c = idx - r * per_row;
          v[u] = *reinterpret_cast<const uint4*>(src + (size_t)r * ld + 8 * c);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * blockDim.x;
        if (idx < total) {
          const int r = idx / per_row, c = idx - r * per_row;
          *reinterpret_cast<uint4*>(dst + r * pitch + 8 * c) = v[u];
        }
      }
    }
    for (int idx = threadIdx.x; idx < rows * (kp - K); idx += blockDim.x) {
      const int r = idx / (kp - K), k = K + idx - r * (kp - K);
      dst[r * pitch + k] = zero;
    }
  } else {
    for (int idx = threadIdx.x; idx < rows * kp; idx += blockDim.x) {
      const int r = idx / kp, k = idx - r * kp;
      dst[r * pitch + k] = k < K ? src[(size_t)r * ld + k] : zero;
    }
  }
}

// MW x 16 tokens of one head against NC outputs (blockIdx.z picks the range of outputs); warp
// (m, n) of the MW x NW warps takes 16 tokens and NC / NW of the outputs.  Rows of the token tile
// beyond the step's tokens are not staged: what the tensor cores make of them is never stored.
template <int MW, int NW, int NC>
__global__ void __launch_bounds__(MW * NW * 32)
headwise_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, int x_hs,
                           const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long long out_ld,
                           int out_hs, const __nv_bfloat16* __restrict__ gate, long long gate_ld, int num_tokens,
                           int N, int K, int vec_x, int vec_w, int pair_store, int gate_each) {
  extern __shared__ __align__(16) unsigned char ht_smem[];
  constexpr int TOKENS = MW * 16, PER_WARP = NC / NW;
  const int kp = (K + 15) / 16 * 16, pitch = kp + 8;  // +8 bf16: rows land in different banks
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ht_smem);  // [TOKENS][pitch]
  __nv_bfloat16* ws = xs + TOKENS * pitch;                        // [NC][pitch]
  const int t0 = blockIdx.x * TOKENS, h = blockIdx.y, n0 = blockIdx.z * NC;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const int n_here = min(NC, N - n0), t_here = min(TOKENS, num_tokens - t0);
  allow_dependents();
  // The weights do not depend on the kernel before this one.
  stage_rows(ws, pitch, w + ((size_t)h * N + n0) * K, K, n_here, K, kp, vec_w != 0);
  grid_dependency_wait();
  stage_rows(xs, pitch, x + (size_t)t0 * x_ld + (size_t)h * x_hs, x_ld, t_here, K, kp, vec_x != 0);
  const int r0 = (warp % MW) * 16 + g, r1 = r0 + 8;
  const int c0 = (warp / MW) * PER_WARP;  // first output of this warp within the block's range
  float gate0 = 1.f, gate1 = 1.f;
  if (gate != nullptr && !gate_each) {
    if (r0 < t_here) gate0 = 1.0f / (1.0f + expf(-to_float(gate[(size_t)(t0 + r0) * gate_ld + h])));
    if (r1 < t_here) gate1 = 1.0f / (1.0f + expf(-to_float(gate[(size_t)(t0 + r1) * gate_ld + h])));
  }
  // One logit per output: the row's gate columns of this head, read where the output is stored.
  const __nv_bfloat16* gate_r0 = gate_each && gate != nullptr ? gate + (size_t)(t0 + r0) * gate_ld + (size_t)h * N + n0 : nullptr;
  const __nv_bfloat16* gate_r1 = gate_each && gate != nullptr ? gate + (size_t)(t0 + r1) * gate_ld + (size_t)h * N + n0 : nullptr;
  __syncthreads();
  float acc[PER_WARP / 8][4];
#pragma unroll
  for (int j = 0; j < PER_WARP / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const int tiles = max(0, min(PER_WARP, n_here - c0) + 7) / 8;
  for (int k0 = 0; k0 < kp; k0 += 16) {
    uint32_t a[4];
    a[0] = *reinterpret_cast<const uint32_t*>(xs + r0 * pitch + k0 + 2 * q);
    a[1] = *reinterpret_cast<const uint32_t*>(xs + r1 * pitch + k0 + 2 * q);
    a[2] = *reinterpret_cast<const uint32_t*>(xs + r0 * pitch + k0 + 8 + 2 * q);
    a[3] = *reinterpret_cast<const uint32_t*>(xs + r1 * pitch + k0 + 8 + 2 * q);
#pragma unroll
    for (int j = 0; j < PER_WARP / 8; ++j) {
      if (j < tiles) {
        const __nv_bfloat16* wr = ws + (c0 + j * 8 + g) * pitch + k0 + 2 * q;
        mma_bf16_16816(acc[j], a, *reinterpret_cast<const uint32_t*>(wr), *reinterpret_cast<const uint32_t*>(wr + 8));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < PER_WARP / 8; ++j) {
    if (j < tiles) {
      const int n = c0 + j * 8 + 2 * q;
      if (gate_r0 != nullptr) {
        if (r0 < t_here) {
          if (n < n_here) acc[j][0] *= 1.0f / (1.0f + expf(-to_float(gate_r0[n])));
          if (n + 1 < n_here) acc[j][1] *= 1.0f / (1.0f + expf(-to_float(gate_r0[n + 1])));
        }
        if (r1 < t_here) {
          if (n < n_here) acc[j][2] *= 1.0f / (1.0f + expf(-to_float(gate_r1[n])));
          if (n + 1 < n_here) acc[j][3] *= 1.0f / (1.0f + expf(-to_float(gate_r1[n + 1])));
        }
      }
      // Two neighbouring outputs as one 4-byte store where every row starts on an even element.
      if (r0 < t_here) {
        __nv_bfloat16* dst = out + (size_t)(t0 + r0) * out_ld + (size_t)h * out_hs + n0 + n;
        if (pair_store && n + 1 < n_here) {
          *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc[j][0] * gate0, acc[j][1] * gate0);
        } else {
          if (n < n_here) dst[0] = __float2bfloat16_rn(acc[j][0] * gate0);
          if (n + 1 < n_here) dst[1] = __float2bfloat16_rn(acc[j][1] * gate0);
        }
      }
      if (r1 < t_here) {
        __nv_bfloat16* dst = out + (size_t)(t0 + r1) * out_ld + (size_t)h * out_hs + n0 + n;
        if (pair_store && n + 1 < n_here) {
          *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc[j][2] * gate1, acc[j][3] * gate1);
        } else {
          if (n < n_here) dst[0] = __float2bfloat16_rn(acc[j][2] * gate1);
          if (n + 1 < n_here) dst[1] = __float2bfloat16_rn(acc[j][3] * gate1);
        }
      }
    }
  }
}

template <int MW, int NW, int NC>
static int launch_headwise_mma(const void* x, long long x_ld, int x_hs, const void* w, void* out, long long out_ld,
                               int out_hs, const void* gate, long long gate_ld, int num_tokens, int H, int N, int K,
                               int gate_each, cudaStream_t stream) {
  const int pitch = (K + 15) / 16 * 16 + 8;
  const size_t bytes = sizeof(__nv_bfloat16) * (size_t)(MW * 16 + NC) * pitch;
  if (bytes > 48 * 1024)
    cudaFuncSetAttribute(headwise_linear_mma_kernel<MW, NW, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  const int vec_w = (K % 8) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
  const int vec_x = (K % 8) == 0 && (x_ld % 8) == 0 && (x_hs % 8) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const int pair_store = (out_ld % 2) == 0 && (out_hs % 2) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0;
  launch_pdl(headwise_linear_mma_kernel<MW, NW, NC>, dim3((num_tokens + MW * 16 - 1) / (MW * 16), H, (N + NC - 1) / NC),
             dim3(MW * NW * 32), bytes, stream, (const __nv_bfloat16*)x, x_ld, x_hs, (const __nv_bfloat16*)w,
             (__nv_bfloat16*)out, out_ld, out_hs, (const __nv_bfloat16*)gate, gate_ld, num_tokens, N, K, vec_x, vec_w, pair_store,
             gate_each);
  return (int)cudaGetLastError();
}

}  // namespace vx

using namespace vx;

VX_API int vx_latent_prepare(const void* proj, long long proj_ld, const void* q_src, long long q_ld, int q_off,
                             int dkv_off, int dtype,
                             const int* positions, const float* cos_t, const float* sin_t, int max_pos,
                             int rot_pairs, const float* latent_w, float eps, const int* slots, void* cache,
                             long long num_slots, void* qa, int num_tokens, int H, int dim, int R, int kr, int Dp,
                             int half_layout, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || dim < 0 || R < 0 || kr <= 0 || Dp < kr + R || 2 * rot_pairs > R) return (int)cudaErrorInvalidValue;
  if (dkv_off >= 0 && (cache == nullptr || slots == nullptr || latent_w == nullptr)) return (int)cudaErrorInvalidValue;
  const int threads = 128;
  if (dtype == VX_DTYPE_F32)
    launch_pdl(latent_prepare_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, (const float*)proj, proj_ld,
               (const float*)q_src, q_ld, q_off, dkv_off, positions, cos_t, sin_t, max_pos, rot_pairs, latent_w, eps, slots, (float*)cache,
               num_slots, (float*)qa, H, dim, R, kr, Dp, half_layout, status);
  else
    launch_pdl(latent_prepare_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, stream,
               (const __nv_bfloat16*)proj, proj_ld, (const __nv_bfloat16*)q_src, q_ld, q_off, dkv_off, positions, cos_t, sin_t, max_pos, rot_pairs,
               latent_w, eps, slots, (__nv_bfloat16*)cache, num_slots, (__nv_bfloat16*)qa, H, dim, R, kr, Dp,
               half_layout, status);
  return (int)cudaGetLastError();
}

VX_API int vx_rms_rows(const void* x, long long x_ld, int dtype, const float* w, float eps, int n, void* out,
                       long long out_ld, int n_out, int num_tokens, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (n <= 0 || n_out < n) return (int)cudaErrorInvalidValue;
  const int threads = n_out >= 256 ? 256 : (n_out + 31) / 32 * 32;
  if (dtype == VX_DTYPE_F32)
    launch_pdl(rms_rows_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, (const float*)x, x_ld, w, eps, n,
               (float*)out, out_ld, n_out);
  else
    launch_pdl(rms_rows_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)x,
               x_ld, w, eps, n, (__nv_bfloat16*)out, out_ld, n_out);
  return (int)cudaGetLastError();
}

VX_API int vx_headwise_linear(const void* x, long long x_ld, int x_hs, const void* w, void* out, long long out_ld,
                              int out_hs, const void* gate, long long gate_ld, int dtype, int num_tokens, int H,
                              int N, int K, int gate_each, cudaStream_t stream) {
  if (num_tokens <= 0 || H <= 0 || N <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  if (dtype == VX_DTYPE_BF16 && K <= HT_MAX_K) {
    // Few tokens: 16 tokens a block, its four warps 16 outputs each of a range of 64, so that the
    // heads' weights are read by many blocks at once; many tokens: 64 tokens a block against 128
    // outputs.
    if (num_tokens <= 32)
      return launch_headwise_mma<1, 4, 64>(x, x_ld, x_hs, w, out, out_ld, out_hs, gate, gate_ld, num_tokens, H, N, K, gate_each, stream);
    return launch_headwise_mma<4, 1, 128>(x, x_ld, x_hs, w, out, out_ld, out_hs, gate, gate_ld, num_tokens, H, N, K, gate_each, stream);
  }
  const size_t smem = sizeof(float) * HL_TOKENS * (size_t)K;
  if (smem > 96 * 1024) return -1;
  const dim3 grid((num_tokens + HL_TOKENS - 1) / HL_TOKENS, H);
  if (dtype == VX_DTYPE_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(headwise_linear_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(headwise_linear_kernel<float>, grid, dim3(256), smem, stream, (const float*)x, x_ld, x_hs,
               (const float*)w, (float*)out, out_ld, out_hs, (const float*)gate, gate_ld, num_tokens, N, K, gate_each);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(headwise_linear_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem);
    launch_pdl(headwise_linear_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)x, x_ld,
               x_hs, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_ld, out_hs, (const __nv_bfloat16*)gate,
               gate_ld, num_tokens, N, K, gate_each);
  }
  return (int)cudaGetLastError();
}
