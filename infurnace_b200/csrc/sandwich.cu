// Pieces around the sublayers of a decoder with a norm before AND after every sublayer: the update of the residual
// stream that normalises a sublayer's result, adds it and writes the next product's input in one pass; additions of
// kept rows and of one vector to the stream; the weighted sum of mixers that run side by side; the gate of a
// per-layer token input; a soft cap on logits; and the blends of each token with the one before it that RWKV-style
// time mixing reads.  Statistics, sums and the stream are float32.  These kernels take every size.
#include "common.cuh"
#include <math.h>

// ------------------------------------------------------------------------------------------
// x[n, :] += y[n, :] / sqrt(mean(y[n, :]^2) + eps) * post[:],   y = s1 * y1 (+ s2 * y2: the weighted sum of two mixers
// that ran side by side is formed here instead of in a launch of its own; s1 = 1 without y2 leaves y1 as it is)
// out (may be null): what the next product reads, in the dtype TO:
//     next given:  x[n, :] / sqrt(mean(x[n, :]^2) + eps) * next[:]      (the next sublayer's pre-norm)
//     else         x[n, :]
// A block per row.  A row of up to RN_KEEP * RN_THREADS features stays in registers over the passes; a longer one is
// read again.
// ------------------------------------------------------------------------------------------
constexpr int RN_THREADS = 256, RN_KEEP = 8;
template <typename TO>
__global__ void __launch_bounds__(RN_THREADS)
residual_norm_update_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ y2, float s1, float s2,
                            const void* __restrict__ post, int post_dtype,
                            const void* __restrict__ next, int next_dtype, float eps, TO* __restrict__ out, int hidden) {
  __shared__ float scratch[33];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const size_t base = (size_t)blockIdx.x * hidden;
  const float* yr = y + base;
  const float* y2r = y2 ? y2 + base : nullptr;
  float* xr = x + base;
  const bool held = hidden <= RN_KEEP * RN_THREADS;
  auto term = [&](int e) { return y2r ? fmaf(s2, y2r[e], s1 * yr[e]) : s1 * yr[e]; };
  float keep[RN_KEEP];
  float ss = 0.f;
  if (held) {
#pragma unroll
    for (int j = 0; j < RN_KEEP; ++j) {
      const int e = threadIdx.x + j * RN_THREADS;
      keep[j] = e < hidden ? term(e) : 0.f;
      ss += keep[j] * keep[j];
    }
  } else {
    for (int e = threadIdx.x; e < hidden; e += RN_THREADS) { const float v = term(e); ss += v * v; }
  }
  ss = block_sum(ss, scratch);
  const float ry = 1.f / sqrtf(ss / (float)hidden + eps);
  float sx = 0.f;
  if (held) {
#pragma unroll
    for (int j = 0; j < RN_KEEP; ++j) {
      const int e = threadIdx.x + j * RN_THREADS;
      if (e < hidden) {
        keep[j] = xr[e] + keep[j] * ry * load_as_f32(post, post_dtype, e);
        xr[e] = keep[j];
        sx += keep[j] * keep[j];
      }
    }
  } else {
    for (int e = threadIdx.x; e < hidden; e += RN_THREADS) {
      const float v = xr[e] + term(e) * ry * load_as_f32(post, post_dtype, e);
      xr[e] = v;
      sx += v * v;
    }
  }
  if (!out) return;
  float rx = 1.f;
  if (next) {
    sx = block_sum(sx, scratch);
    rx = 1.f / sqrtf(sx / (float)hidden + eps);
  }
  TO* o = out + base;
  if (held) {
#pragma unroll
    for (int j = 0; j < RN_KEEP; ++j) {
      const int e = threadIdx.x + j * RN_THREADS;
      if (e < hidden) o[e] = from_f32<TO>(next ? keep[j] * rx * load_as_f32(next, next_dtype, e) : keep[j]);
    }
  } else {
    for (int e = threadIdx.x; e < hidden; e += RN_THREADS)      // a thread reads back what it wrote itself
      o[e] = from_f32<TO>(next ? xr[e] * rx * load_as_f32(next, next_dtype, e) : xr[e]);
  }
}

IFB_EXPORT int ifb_residual_norm_update(float* x, const float* y, const float* y2, float s1, float s2, const void* post, int post_dtype, const void* next,
                                        int next_dtype, float eps, void* out, int out_dtype, int n, int hidden,
                                        cudaStream_t stream) {
  if (n <= 0 || hidden <= 0) return IFB_OK;
  if ((post_dtype != IFB_F32 && post_dtype != IFB_BF16) || (next && next_dtype != IFB_F32 && next_dtype != IFB_BF16))
    return IFB_ERR_DTYPE;
  if (out && out_dtype == IFB_BF16)
    return ifb_launch(residual_norm_update_kernel<__nv_bfloat16>, dim3(n), dim3(RN_THREADS), 0, stream, x, y, y2, s1, s2, post,
                      post_dtype, next, next_dtype, eps, (__nv_bfloat16*)out, hidden);
  if (out && out_dtype != IFB_F32) return IFB_ERR_DTYPE;
  return ifb_launch(residual_norm_update_kernel<float>, dim3(n), dim3(RN_THREADS), 0, stream, x, y, y2, s1, s2, post, post_dtype,
                    next, next_dtype, eps, (float*)out, hidden);
}

// ------------------------------------------------------------------------------------------
// x[n, :] = (accumulate ? x[n, :] : 0) + rows[n, :] + vec[:]        (rows, vec: each may be null)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
add_rows_kernel(float* __restrict__ x, const float* __restrict__ rows, const void* __restrict__ vec, int vec_dtype,
                int accumulate, long long total, int hidden) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float v = accumulate ? x[i] : 0.f;
    if (rows) v += rows[i];
    if (vec) v += load_as_f32(vec, vec_dtype, (size_t)(i % hidden));
    x[i] = v;
  }
}

IFB_EXPORT int ifb_add_rows(float* x, const float* rows, const void* vec, int vec_dtype, int accumulate, int n, int hidden,
                            cudaStream_t stream) {
  if (n <= 0 || hidden <= 0) return IFB_OK;
  if (vec && vec_dtype != IFB_F32 && vec_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  const long long total = (long long)n * hidden;
  const unsigned blocks = (unsigned)min((total + 255) / 256, (long long)65535);
  return ifb_launch(add_rows_kernel, dim3(blocks), dim3(256), 0, stream, x, rows, vec, vec_dtype, accumulate, total, hidden);
}

// total[i] = (accumulate ? total[i] : 0) + scale * d[i]; copy[i] (optional, bfloat16 or float32) = the new total[i], for
// the product that reads the stream next
__global__ void __launch_bounds__(256)
scaled_sum_kernel(float* __restrict__ total, const float* __restrict__ d, float scale, int accumulate, long long count,
                  void* __restrict__ copy, int copy_dtype) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    const float v = accumulate ? fmaf(scale, d[i], total[i]) : scale * d[i];
    total[i] = v;
    if (copy != nullptr) {
      if (copy_dtype == IFB_BF16) reinterpret_cast<__nv_bfloat16*>(copy)[i] = __float2bfloat16(v);
      else reinterpret_cast<float*>(copy)[i] = v;
    }
  }
}

IFB_EXPORT int ifb_scaled_sum(float* total, const float* d, float scale, int accumulate, long long count, void* copy,
                              int copy_dtype, cudaStream_t stream) {
  if (count <= 0) return IFB_OK;
  if (copy != nullptr && copy_dtype != IFB_BF16 && copy_dtype != IFB_F32) return IFB_ERR_DTYPE;
  const unsigned blocks = (unsigned)min((count + 255) / 256, (long long)65535);
  return ifb_launch(scaled_sum_kernel, dim3(blocks), dim3(256), 0, stream, total, d, scale, accumulate, count, copy, copy_dtype);
}

// ------------------------------------------------------------------------------------------
// out[n, j] = unary(z[n, j]) * table[ids[n], offset + j]: the gate of a per-layer token input.  An id outside the
// vocabulary reads nothing (the row is zero); the embedding has recorded the fault already.
// ------------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256)
token_side_gate_kernel(const float* __restrict__ z, const void* __restrict__ table, int table_dtype, int table_width,
                       int vocab, const int* __restrict__ ids, int offset, int unary, TO* __restrict__ out, long long total,
                       int dim) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(i / dim), j = (int)(i % dim);
    const int id = ids[n];
    const float e = (id < 0 || id >= vocab) ? 0.f : load_as_f32(table, table_dtype, (size_t)id * table_width + offset + j);
    out[i] = from_f32<TO>(ifb_unary(z[i], unary) * e);
  }
}

IFB_EXPORT int ifb_token_side_gate(const float* z, const void* table, int table_dtype, int table_width, int vocab,
                                   const int* ids, int offset, int unary, void* out, int out_dtype, int n, int dim,
                                   cudaStream_t stream) {
  if (n <= 0 || dim <= 0) return IFB_OK;
  if (table_dtype != IFB_F32 && table_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  if (offset < 0 || offset + dim > table_width || unary < 0 || unary > IFB_UNARY_LAST) return IFB_ERR_ARG;
  const long long total = (long long)n * dim;
  const unsigned blocks = (unsigned)min((total + 255) / 256, (long long)65535);
  if (out_dtype == IFB_BF16)
    return ifb_launch(token_side_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, z, table, table_dtype,
                      table_width, vocab, ids, offset, unary, (__nv_bfloat16*)out, total, dim);
  if (out_dtype != IFB_F32) return IFB_ERR_DTYPE;
  return ifb_launch(token_side_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, z, table, table_dtype, table_width,
                    vocab, ids, offset, unary, (float*)out, total, dim);
}

// logits[i] = cap * tanh(logits[i] / cap)
__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ logits, float cap, long long count) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
    logits[i] = cap * tanhf(logits[i] / cap);
}

IFB_EXPORT int ifb_softcap(float* logits, float cap, long long count, cudaStream_t stream) {
  if (count <= 0) return IFB_OK;
  if (!(cap > 0.f)) return IFB_ERR_ARG;
  const unsigned blocks = (unsigned)min((count + 255) / 256, (long long)65535);
  return ifb_launch(softcap_kernel, dim3(blocks), dim3(256), 0, stream, logits, cap, count);
}

// ------------------------------------------------------------------------------------------
// Token shift.  For stream s of `streams` and token t of request r:
//     out[s][t][:] = h[t][:] + (h'[t][:] - h[t][:]) * mu[s][:]
// with h'[t] = h[t - 1] inside the request's rows of this step and, for the request's first row of the step, the row
// that the request's state slot holds (zero when the slot was granted).  The block of a request's first row also
// writes the request's last row of this step into the slot, after it has read it: the only reader and the only
// writer of a slot in a step are that one block.  A request of length 0 is padding: its rows get h itself (h' = h)
// and its slot is left alone.  A block per token.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
token_shift_mix_kernel(const T* __restrict__ h, float* __restrict__ last, const int* __restrict__ state_slots,
                       const int* __restrict__ cu_q, const int* __restrict__ seq_lens, const float* __restrict__ mu,
                       T* __restrict__ out, int tokens, int requests, int hidden, int streams) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int t = blockIdx.x;
  int lo = 0, hi = requests;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cu_q[mid] <= t) lo = mid; else hi = mid; }
  const int r = lo;
  const bool live = t < cu_q[requests] && seq_lens[r] > 0;
  const bool first = live && t == cu_q[r];
  const T* cur = h + (size_t)t * hidden;
  float* slot = live ? last + (size_t)state_slots[r] * hidden : nullptr;
  const T* tail = live ? h + (size_t)(cu_q[r + 1] - 1) * hidden : nullptr;
  for (int e = threadIdx.x; e < hidden; e += blockDim.x) {
    const float c = to_f32<T>(cur[e]);
    float p = c;
    if (first) {
      p = slot[e];
      slot[e] = to_f32<T>(tail[e]);
    } else if (live) {
      p = to_f32<T>(cur[e - hidden]);
    }
    for (int s = 0; s < streams; ++s)
      out[((size_t)s * tokens + t) * hidden + e] = from_f32<T>(fmaf(p - c, mu[(size_t)s * hidden + e], c));
  }
}

IFB_EXPORT int ifb_token_shift_mix(const void* h, int dtype, float* last, const int* state_slots, const int* cu_q,
                                   const int* seq_lens, const float* mu, void* out, int tokens, int requests, int hidden,
                                   int streams, cudaStream_t stream) {
  if (tokens <= 0 || requests <= 0 || hidden <= 0 || streams <= 0) return IFB_OK;
  const int threads = hidden >= 256 ? 256 : ((hidden + 31) / 32) * 32;
  if (dtype == IFB_BF16)
    return ifb_launch(token_shift_mix_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)h,
                      last, state_slots, cu_q, seq_lens, mu, (__nv_bfloat16*)out, tokens, requests, hidden, streams);
  if (dtype != IFB_F32) return IFB_ERR_DTYPE;
  return ifb_launch(token_shift_mix_kernel<float>, dim3(tokens), dim3(threads), 0, stream, (const float*)h, last, state_slots,
                    cu_q, seq_lens, mu, (float*)out, tokens, requests, hidden, streams);
}
