// Row-wise steps of decoders whose attention keeps a small latent per token: the RMS norm in groups (with the residual
// addition and a residual multiplier folded in), the short causal convolution in front of a sublayer (its last inputs
// are state of a sequence), the weighted average over depth (with the next norm folded in), the preparation of queries
// and latents for the latent attention, and the output gate.  Statistics, sums, angles and the stream are float32.
#include "common.cuh"
#include <math.h>

// ------------------------------------------------------------------------------------------
// The norm in groups of a row that lies in shared memory: out[e] = row[e] * rsqrt(mean over e's group of row^2 + eps) * w[e].
// Every thread of the block calls it; `scratch` holds 33 floats.
// ------------------------------------------------------------------------------------------
template <typename TO> __device__ __forceinline__ void store4(TO* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

template <typename TO>
__device__ __forceinline__ void group_norm_row(const float* row, int width, int groups, float eps, const void* weight, int wtype,
                                               TO* out, float* scratch) {
  const int gs = width / groups;
  if ((gs & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {      // four elements per thread (row is 16-byte aligned)
    for (int g = 0; g < groups; ++g) {
      float sq = 0.f;
      for (int e = threadIdx.x * 4; e < gs; e += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + g * gs + e);
        sq = fmaf(v.x, v.x, sq); sq = fmaf(v.y, v.y, sq); sq = fmaf(v.z, v.z, sq); sq = fmaf(v.w, v.w, sq);
      }
      const float r = rsqrtf(block_sum(sq, scratch) / (float)gs + eps);
      for (int e = threadIdx.x * 4; e < gs; e += blockDim.x * 4) {
        const int i = g * gs + e;
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        store4<TO>(out + i, v.x * r * load_as_f32(weight, wtype, i), v.y * r * load_as_f32(weight, wtype, i + 1),
                   v.z * r * load_as_f32(weight, wtype, i + 2), v.w * r * load_as_f32(weight, wtype, i + 3));
      }
    }
    return;
  }
  for (int g = 0; g < groups; ++g) {
    float sq = 0.f;
    for (int e = threadIdx.x; e < gs; e += blockDim.x) { const float v = row[g * gs + e]; sq = fmaf(v, v, sq); }
    const float r = rsqrtf(block_sum(sq, scratch) / (float)gs + eps);
    for (int e = threadIdx.x; e < gs; e += blockDim.x)
      out[g * gs + e] = from_f32<TO>(row[g * gs + e] * r * load_as_f32(weight, wtype, g * gs + e));
  }
}

// x[r] += mult * delta[r] (written back unless `rows` picks the rows); keep[r] = the updated row (optional, row stride
// keep_stride); out[b] = the norm in groups of the updated row.
template <typename TO>
__global__ void __launch_bounds__(256)
group_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, float mult, const void* __restrict__ weight, int wtype,
                     int groups, float eps, TO* __restrict__ out, const int* __restrict__ rows, float* __restrict__ keep,
                     long long keep_stride, int width, int vec) {
  extern __shared__ __align__(16) float gn_row[];
  __shared__ float scratch[33];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int b = blockIdx.x;
  const int r = rows ? rows[b] : b;
  float* xr = x + (size_t)r * width;
  if (vec) {                                           // width, keep_stride multiples of 4 and every base 16-byte aligned
    for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + e);
      if (delta) {
        const float4 d = *reinterpret_cast<const float4*>(delta + (size_t)r * width + e);
        v.x = fmaf(mult, d.x, v.x); v.y = fmaf(mult, d.y, v.y); v.z = fmaf(mult, d.z, v.z); v.w = fmaf(mult, d.w, v.w);
      }
      *reinterpret_cast<float4*>(gn_row + e) = v;
      if (delta && !rows) *reinterpret_cast<float4*>(xr + e) = v;
      if (keep) *reinterpret_cast<float4*>(keep + (size_t)r * keep_stride + e) = v;
    }
  } else {
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
      float v = xr[e];
      if (delta) v = fmaf(mult, delta[(size_t)r * width + e], v);
      gn_row[e] = v;
      if (delta && !rows) xr[e] = v;
      if (keep) keep[(size_t)r * keep_stride + e] = v;
    }
  }
  __syncthreads();
  group_norm_row<TO>(gn_row, width, groups, eps, weight, wtype, out + (size_t)b * width, scratch);
}

IFB_EXPORT int ifb_group_rmsnorm(float* x, const float* delta, float mult, const void* weight, int wtype, int groups, float eps,
                                 void* out, int otype, const int* rows, float* keep, long long keep_stride, int n, int width,
                                 cudaStream_t stream) {
  if (n <= 0) return IFB_OK;
  if (width < 1 || groups < 1 || width % groups) return IFB_ERR_SIZE;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return IFB_ERR_SIZE;
  const int vec = width % 4 == 0 && keep_stride % 4 == 0 && (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)keep) & 15) == 0;
  if (otype == IFB_BF16) {
    IFB_ALLOW_SMEM(group_rmsnorm_kernel<__nv_bfloat16>, smem);
    return ifb_launch(group_rmsnorm_kernel<__nv_bfloat16>, dim3(n), dim3(256), smem, stream, x, delta, mult, weight, wtype, groups,
                      eps, (__nv_bfloat16*)out, rows, keep, keep_stride, width, vec);
  }
  if (otype != IFB_F32) return IFB_ERR_DTYPE;
  IFB_ALLOW_SMEM(group_rmsnorm_kernel<float>, smem);
  return ifb_launch(group_rmsnorm_kernel<float>, dim3(n), dim3(256), smem, stream, x, delta, mult, weight, wtype, groups, eps,
                    (float*)out, rows, keep, keep_stride, width, vec);
}

// ------------------------------------------------------------------------------------------
// The weighted average over depth.  hist [n, slots, width] holds X_0 .. X_(depth-1) of every token.  The block's result
// X_depth = x + mult * delta is stored there, x becomes sum_j coeff[j] * X_j (j ascending, j <= depth), and `out` (optional)
// gets the norm in groups of the new x with the next norm's weight.
// ------------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256)
depth_average_kernel(float* __restrict__ x, const float* __restrict__ delta, float mult, float* __restrict__ hist, int slots,
                     int depth, const void* __restrict__ coeff, int ctype, const void* __restrict__ weight, int wtype, int groups,
                     float eps, TO* __restrict__ out, int width, int vec) {
  extern __shared__ __align__(16) float gn_row[];
  __shared__ float scratch[33];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * width;
  float* hr = hist + (size_t)t * slots * width;
  if (vec) {                                           // width a multiple of 4 and every base 16-byte aligned
    for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + e);
      if (delta) {
        const float4 d = *reinterpret_cast<const float4*>(delta + (size_t)t * width + e);
        v.x = fmaf(mult, d.x, v.x); v.y = fmaf(mult, d.y, v.y); v.z = fmaf(mult, d.z, v.z); v.w = fmaf(mult, d.w, v.w);
      }
      *reinterpret_cast<float4*>(hr + (size_t)depth * width + e) = v;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
      for (int j = 0; j < depth; ++j) {
        const float c = load_as_f32(coeff, ctype, j);
        const float4 u = *reinterpret_cast<const float4*>(hr + (size_t)j * width + e);
        acc.x = fmaf(c, u.x, acc.x); acc.y = fmaf(c, u.y, acc.y); acc.z = fmaf(c, u.z, acc.z); acc.w = fmaf(c, u.w, acc.w);
      }
      const float c = load_as_f32(coeff, ctype, depth);
      acc.x = fmaf(c, v.x, acc.x); acc.y = fmaf(c, v.y, acc.y); acc.z = fmaf(c, v.z, acc.z); acc.w = fmaf(c, v.w, acc.w);
      *reinterpret_cast<float4*>(xr + e) = acc;
      *reinterpret_cast<float4*>(gn_row + e) = acc;
    }
  } else {
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
      float v = xr[e];
      if (delta) v = fmaf(mult, delta[(size_t)t * width + e], v);
      hr[(size_t)depth * width + e] = v;
      float acc = 0.f;
      for (int j = 0; j < depth; ++j) acc = fmaf(load_as_f32(coeff, ctype, j), hr[(size_t)j * width + e], acc);
      acc = fmaf(load_as_f32(coeff, ctype, depth), v, acc);
      xr[e] = acc;
      gn_row[e] = acc;
    }
  }
  if (out == nullptr) return;
  __syncthreads();
  group_norm_row<TO>(gn_row, width, groups, eps, weight, wtype, out + (size_t)t * width, scratch);
}

IFB_EXPORT int ifb_depth_average(float* x, const float* delta, float mult, float* hist, int slots, int depth, const void* coeff,
                                 int ctype, const void* weight, int wtype, int groups, float eps, void* out, int otype, int n,
                                 int width, cudaStream_t stream) {
  if (n <= 0) return IFB_OK;
  if (width < 1 || depth < 0 || depth >= slots) return IFB_ERR_SIZE;
  if (out != nullptr && (groups < 1 || width % groups)) return IFB_ERR_SIZE;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return IFB_ERR_SIZE;
  const int vec = width % 4 == 0 && (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)hist) & 15) == 0;
  if (out == nullptr || otype == IFB_F32) {
    IFB_ALLOW_SMEM(depth_average_kernel<float>, smem);
    return ifb_launch(depth_average_kernel<float>, dim3(n), dim3(256), smem, stream, x, delta, mult, hist, slots, depth, coeff,
                      ctype, weight, wtype, groups, eps, (float*)out, width, vec);
  }
  if (otype != IFB_BF16) return IFB_ERR_DTYPE;
  IFB_ALLOW_SMEM(depth_average_kernel<__nv_bfloat16>, smem);
  return ifb_launch(depth_average_kernel<__nv_bfloat16>, dim3(n), dim3(256), smem, stream, x, delta, mult, hist, slots, depth,
                    coeff, ctype, weight, wtype, groups, eps, (__nv_bfloat16*)out, width, vec);
}

// ------------------------------------------------------------------------------------------
// out_t = h_t + sum_(j <= K) w[:, j] * h_(t - K + j), K = taps - 1, zeros before a sequence's start.  The K inputs before a
// portion come from the request's state [slots, K, width] (float32, oldest first).  A block per token.  The block of a
// portion's first token computes every token of the portion that reads the state (its first K) and then replaces the
// state by the portion's last K inputs (older ones shifted down where the portion is shorter), so that each element of the
// state is read and written by one thread only; the blocks of those other tokens do nothing.
// ------------------------------------------------------------------------------------------
constexpr int CC_MAX_TAPS = 64;
// VT > 0 (bfloat16 rows and weights, a multiple of 8 channels, 16-byte aligned, VT = taps): the tokens that read no state
// take eight channels per thread: the channels' VT x 8 weights and each tap's eight inputs are 16-byte loads.
template <typename T, int VT>
__device__ __forceinline__ void causal_conv_token(int t, const T* __restrict__ h, const void* __restrict__ weight, int wtype,
                                                  float* __restrict__ state, const int* __restrict__ state_slots,
                                                  const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                                                  const int* __restrict__ req_index, T* __restrict__ out, int width, int taps) {
  const int K = taps - 1;
  const int r = req_index[t];
  const int q0 = cu_q[r], len = cu_q[r + 1] - q0, i = t - q0;
  if (seq_lens[r] <= 0) {                              // a padding row of a recorded step: it stores and sees nothing
    for (int e = threadIdx.x; e < width; e += blockDim.x) out[(size_t)t * width + e] = h[(size_t)t * width + e];
    return;
  }
  if (i > 0 && i < K) return;                          // the first token's block computes these
  if (i >= K) {
    if constexpr (VT > 0) {
      const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(weight);
      for (int e = threadIdx.x * 8; e < width; e += blockDim.x * 8) {
        __align__(16) __nv_bfloat16 w[VT * 8];          // w[c * VT + j]
        __align__(16) __nv_bfloat16 x[VT * 8];          // x[j * 8 + c]
#pragma unroll
        for (int v = 0; v < VT; ++v) {
          *reinterpret_cast<uint4*>(w + 8 * v) = *reinterpret_cast<const uint4*>(wb + (size_t)e * VT + 8 * v);
          *reinterpret_cast<uint4*>(x + 8 * v) = *reinterpret_cast<const uint4*>(h + (size_t)(t - (VT - 1) + v) * width + e);
        }
        __align__(16) __nv_bfloat16 o[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float acc = __bfloat162float(x[(VT - 1) * 8 + c]);
#pragma unroll
          for (int j = 0; j < VT; ++j) acc = fmaf(__bfloat162float(w[c * VT + j]), __bfloat162float(x[j * 8 + c]), acc);
          o[c] = __float2bfloat16(acc);
        }
        *reinterpret_cast<uint4*>(out + (size_t)t * width + e) = *reinterpret_cast<const uint4*>(o);
      }
    } else {
      for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float acc = to_f32<T>(h[(size_t)t * width + e]);
        for (int j = 0; j <= K; ++j)
          acc = fmaf(load_as_f32(weight, wtype, (size_t)e * taps + j), to_f32<T>(h[(size_t)(t - K + j) * width + e]), acc);
        out[(size_t)t * width + e] = from_f32<T>(acc);
      }
    }
    return;
  }
  float* st = state + (size_t)state_slots[r] * (K > 0 ? K : 1) * width;
  const int head = len < K ? len : K;                  // tokens of the portion that read the state
  if constexpr (VT > 0) {
    // eight channels per thread here too (the state's rows are 16-byte aligned with the rest): the loads of a token's
    // inputs are independent of one another, and this one block is what a step of single tokens waits for
    const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(weight);
    for (int e = threadIdx.x * 8; e < width; e += blockDim.x * 8) {
      __align__(16) __nv_bfloat16 w[VT * 8];            // w[c * VT + j]
#pragma unroll
      for (int v = 0; v < VT; ++v) *reinterpret_cast<uint4*>(w + 8 * v) = *reinterpret_cast<const uint4*>(wb + (size_t)e * VT + 8 * v);
      auto input8 = [&](int x, float (&v)[8]) {         // input number x of the portion, x < 0: from the state
        if (x < 0) {
          const float4 a = *reinterpret_cast<const float4*>(st + (size_t)(K + x) * width + e);
          const float4 b = *reinterpret_cast<const float4*>(st + (size_t)(K + x) * width + e + 4);
          v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
          __align__(16) __nv_bfloat16 raw[8];
          *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(h + (size_t)(q0 + x) * width + e);
#pragma unroll
          for (int c = 0; c < 8; ++c) v[c] = __bfloat162float(raw[c]);
        }
      };
      for (int k = 0; k < head; ++k) {
        float x[VT][8];
#pragma unroll
        for (int j = 0; j < VT; ++j) input8(k - K + j, x[j]);
        __align__(16) __nv_bfloat16 o[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float acc = x[VT - 1][c];
#pragma unroll
          for (int j = 0; j < VT; ++j) acc = fmaf(__bfloat162float(w[c * VT + j]), x[j][c], acc);
          o[c] = __float2bfloat16(acc);
        }
        *reinterpret_cast<uint4*>(out + (size_t)(q0 + k) * width + e) = *reinterpret_cast<const uint4*>(o);
      }
      // the new state, ascending (see below): every place is read before a lower place's write can have reached it
      for (int k = 0; k < K; ++k) {
        float v[8];
        input8(len - K + k, v);
        *reinterpret_cast<float4*>(st + (size_t)k * width + e) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(st + (size_t)k * width + e + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
    }
  } else {
  for (int e = threadIdx.x; e < width; e += blockDim.x) {
    // input number x of the portion (x < 0: from the state, which holds inputs -K .. -1 at 0 .. K - 1)
    auto input = [&](int x) { return x < 0 ? st[(size_t)(K + x) * width + e] : to_f32<T>(h[(size_t)(q0 + x) * width + e]); };
    for (int k = 0; k < head; ++k) {
      float acc = input(k);
      for (int j = 0; j <= K; ++j) acc = fmaf(load_as_f32(weight, wtype, (size_t)e * taps + j), input(k - K + j), acc);
      out[(size_t)(q0 + k) * width + e] = from_f32<T>(acc);
    }
    // the new state: inputs len - K .. len - 1.  Place k takes input len - K + k, which is the old place len + k when that is
    // still a state's input: a place above k, so ascending k reads nothing that was written.
    for (int k = 0; k < K; ++k) st[(size_t)k * width + e] = input(len - K + k);
  }
  }
}

template <typename T, int VT>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const T* __restrict__ h, const void* __restrict__ weight, int wtype, float* __restrict__ state,
                   const int* __restrict__ state_slots, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                   const int* __restrict__ req_index, T* __restrict__ out, int width, int taps) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  causal_conv_token<T, VT>(blockIdx.x, h, weight, wtype, state, state_slots, cu_q, seq_lens, req_index, out, width, taps);
}

IFB_EXPORT int ifb_causal_conv(const void* h, int dtype, const void* weight, int wtype, float* state, const int* state_slots,
                               const int* cu_q, const int* seq_lens, const int* req_index, void* out, int tokens, int width,
                               int taps, cudaStream_t stream) {
  if (tokens <= 0) return IFB_OK;
  if (width < 1 || taps < 1 || taps > CC_MAX_TAPS) return IFB_ERR_SIZE;
  const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
  const dim3 grid((unsigned)tokens);
  if (dtype == IFB_BF16) {
    // rows that read no state go eight channels at a time where the taps are few and everything is aligned
    if (wtype == IFB_BF16 && taps >= 2 && taps <= 8 && width % 8 == 0 && width >= 256 &&
        (((uintptr_t)h | (uintptr_t)out | (uintptr_t)weight | (uintptr_t)state) & 15) == 0) {
#define CC_VEC(V)                                                                                                              \
  case V:                                                                                                                      \
    return ifb_launch(causal_conv_kernel<__nv_bfloat16, V>, grid, dim3(width >= 2048 ? 256 : 128), 0, stream,                  \
                      (const __nv_bfloat16*)h, weight, wtype, state, state_slots, cu_q, seq_lens, req_index, (__nv_bfloat16*)out, \
                      width, taps)
      switch (taps) { CC_VEC(2); CC_VEC(3); CC_VEC(4); CC_VEC(5); CC_VEC(6); CC_VEC(7); CC_VEC(8); }
#undef CC_VEC
    }
    return ifb_launch(causal_conv_kernel<__nv_bfloat16, 0>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)h, weight,
                      wtype, state, state_slots, cu_q, seq_lens, req_index, (__nv_bfloat16*)out, width, taps);
  }
  if (dtype != IFB_F32) return IFB_ERR_DTYPE;
  return ifb_launch(causal_conv_kernel<float, 0>, grid, dim3(threads), 0, stream, (const float*)h, weight, wtype, state,
                    state_slots, cu_q, seq_lens, req_index, (float*)out, width, taps);
}

// ------------------------------------------------------------------------------------------
// After the product q | down(latent, rotated key) | ... of a step (proj, float32, row stride `stride`): per token
//  * the latent: columns down_col .. + rank, divided by their root mean square, times the norm's weight, stored to its page
//    stream at slot_mapping (pages [pages, 1, page_size, rank], stored as one row per slot);
//  * the rotated key part: the next rot columns, their first `dims` entries turned by the token's angles (pair i, i + dims/2;
//    table [n, dims] holds (cos, sin) pairs), stored to its page stream;
//  * every head's unrotated query part to q_plain [heads, seg, dim] (head-major: the rows of a head are one segment of the
//    grouped product that follows) and its rotated part, turned, to q_rot [n, heads, rot] (float32).
// Block 0 also writes the segments of the grouped products: offsets[h] = h * seg and, for tiles of `tile` rows,
// tile_head[j] = j / (seg / tile).
// ------------------------------------------------------------------------------------------
template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ proj, long long stride, int heads, int dim, int rot, int rank, int down_col,
                      const void* __restrict__ norm_w, int wtype, float eps, const float* __restrict__ table, int dims,
                      TA* __restrict__ q_plain, int seg, float* __restrict__ q_rot, TC* __restrict__ latent_pages,
                      TC* __restrict__ rot_pages, const int* __restrict__ slot_mapping, int* __restrict__ offsets,
                      int* __restrict__ tile_head, int tile, int tokens, const float* __restrict__ q_rows, long long q_stride,
                      int interleaved) {
  __shared__ float scratch[33];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int t = blockIdx.x;
  if (t == 0) {
    for (int h = threadIdx.x; h <= heads; h += blockDim.x) offsets[h] = h * seg;
    if (tile_head != nullptr) {
      const int per = seg / tile;
      for (int j = threadIdx.x; j < heads * per; j += blockDim.x) tile_head[j] = j / per;
    }
  }
  const float* row = proj + (size_t)t * stride;
  const float* qrow = q_rows ? q_rows + (size_t)t * q_stride : row;        // the queries may come from a product of their own
  const float* tab = table ? table + (size_t)t * dims : nullptr;
  const int half = dims / 2;
  // queries
  const int qw = dim + rot;
  for (int i = threadIdx.x; i < heads * qw; i += blockDim.x) {
    const int h = i / qw, c = i - h * qw;
    if (c < dim) {
      q_plain[((size_t)h * seg + t) * dim + c] = from_f32<TA>(qrow[i]);
    } else {
      const int d = c - dim;
      float v = qrow[i];
      if (tab != nullptr && d < dims) {
        // the pair (u, v) becomes (u c - v s, v c + u s): entries m and m + dims/2, or 2m and 2m + 1 when interleaved
        const bool lead = interleaved ? !(d & 1) : d < half;
        const int p = interleaved ? d >> 1 : (lead ? d : d - half);
        const int other = interleaved ? (lead ? 1 : -1) : (lead ? half : -half);
        const float cs = tab[2 * p], sn = tab[2 * p + 1];
        v = lead ? v * cs - qrow[i + other] * sn : v * cs + qrow[i + other] * sn;
      }
      q_rot[((size_t)t * heads + h) * rot + d] = v;
    }
  }
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  // the latent
  const float* lat = row + down_col;
  float sq = 0.f;
  for (int e = threadIdx.x; e < rank; e += blockDim.x) sq = fmaf(lat[e], lat[e], sq);
  const float r = rsqrtf(block_sum(sq, scratch) / (float)rank + eps);
  if (slot < 0) return;
  for (int e = threadIdx.x; e < rank; e += blockDim.x)
    latent_pages[(size_t)slot * rank + e] = from_f32<TC>(lat[e] * r * load_as_f32(norm_w, wtype, e));
  // the rotated key part
  const float* kr = lat + rank;
  for (int d = threadIdx.x; d < rot; d += blockDim.x) {
    float v = kr[d];
    if (tab != nullptr && d < dims) {
      const bool lead = interleaved ? !(d & 1) : d < half;
      const int p = interleaved ? d >> 1 : (lead ? d : d - half);
      const int other = interleaved ? (lead ? 1 : -1) : (lead ? half : -half);
      const float cs = tab[2 * p], sn = tab[2 * p + 1];
      v = lead ? v * cs - kr[d + other] * sn : v * cs + kr[d + other] * sn;
    }
    rot_pages[(size_t)slot * rot + d] = from_f32<TC>(v);
  }
}

IFB_EXPORT int ifb_latent_prepare(const float* proj, long long stride, int heads, int dim, int rot, int rank, int down_col,
                                  const void* norm_w, int wtype, float eps, const float* table, int dims, void* q_plain, int atype,
                                  int seg, float* q_rot, void* latent_pages, void* rot_pages, int ctype, const int* slot_mapping,
                                  int* offsets, int* tile_head, int tile, int tokens, const float* q_rows, long long q_stride,
                                  int interleaved, cudaStream_t stream) {
  if (tokens <= 0) return IFB_OK;
  if (heads < 1 || dim < 1 || rot < 0 || rank < 1 || seg < tokens || dims < 0 || dims > rot || (dims & 1)) return IFB_ERR_SIZE;
  if (tile_head != nullptr && (tile < 1 || seg % tile)) return IFB_ERR_SIZE;
  if (atype != ctype) return IFB_ERR_DTYPE;           // queries and cache share the engine's activation dtype
#define LP_LAUNCH(TA, TC)                                                                                                        \
  return ifb_launch(latent_prepare_kernel<TA, TC>, dim3(tokens), dim3(256), 0, stream, proj, stride, heads, dim, rot, rank,      \
                    down_col, norm_w, wtype, eps, table, dims, (TA*)q_plain, seg, q_rot, (TC*)latent_pages, (TC*)rot_pages,      \
                    slot_mapping, offsets, tile_head, tile, tokens, q_rows, q_stride, interleaved)
  if (atype == IFB_BF16) LP_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (atype == IFB_F32) LP_LAUNCH(float, float);
#undef LP_LAUNCH
  return IFB_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------
// out[t, h * vdim + v] = y[h, t, v] * sigmoid(gate[t, h * vdim + v]) (gate null: no gate; per_head: gate[t, h], one number for
// the whole head): from the head-major result of a
// grouped product (float32, `seg` rows per head) to the rows the output product reads.
// ------------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256)
gate_heads_kernel(const float* __restrict__ y, int seg, const float* __restrict__ gate, long long gate_stride,
                  TO* __restrict__ out, int heads, int vdim, int per_head) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int t = blockIdx.x, width = heads * vdim;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const int h = i / vdim, v = i - h * vdim;
    float val = y[((size_t)h * seg + t) * vdim + v];
    if (gate != nullptr) val *= 1.f / (1.f + expf(-gate[(size_t)t * gate_stride + (per_head ? h : i)]));
    out[(size_t)t * width + i] = from_f32<TO>(val);
  }
}

IFB_EXPORT int ifb_gate_heads(const float* y, int seg, const float* gate, long long gate_stride, void* out, int otype, int tokens,
                              int heads, int vdim, int per_head, cudaStream_t stream) {
  if (tokens <= 0) return IFB_OK;
  if (heads < 1 || vdim < 1 || seg < tokens) return IFB_ERR_SIZE;
  if (otype == IFB_BF16)
    return ifb_launch(gate_heads_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, y, seg, gate, gate_stride,
                      (__nv_bfloat16*)out, heads, vdim, per_head);
  if (otype != IFB_F32) return IFB_ERR_DTYPE;
  return ifb_launch(gate_heads_kernel<float>, dim3(tokens), dim3(256), 0, stream, y, seg, gate, gate_stride, (float*)out, heads,
                    vdim, per_head);
}
