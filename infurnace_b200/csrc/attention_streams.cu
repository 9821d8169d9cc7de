// Softmax attention whose values carry positions, over page streams that may differ in width.
//
// (1) rotary_store: per token, the q and k heads are rotated on their first rot_dims entries by the token's angles,
// each value head is divided by its root mean square (optional) and rotated over its whole width by the token's
// angles (optional); q goes to a row buffer, k and v into their page streams at the token's slot.  Where a model has no
// value projection the values are the key heads as projected, before their rotation.  The angles come
// as a table of (cos, sin) pairs per token, float32.  A rotation pairs entry m with m + dims/2, or 2m with 2m + 1
// when interleaved; the pair (u, v) becomes (u c - v s, v c + u s).
//
// (2) paged_attention_streams: one warp per (query token, query head); float32 scores, softmax weights and sums,
// whatever the storage.  A query at position p reads the keys at positions first .. p from the pages of its request,
// first = max(0, p - window + 1) with a window, else 0.  After the division by the softmax sum the head's output is
// rotated BACK by the query token's angles (optional): (u, v) becomes (u c + v s, v c - u s).
//
// Head sizes up to 256 for keys and for values, any page size, any grouping.
#include "common.cuh"
#include <math.h>

#define AS_MAX_D 256

// element j of a head after the rotation of its first `dims` entries; x: the head's entries (float32, in shared or
// global memory), tab: the token's (cos, sin) pairs, sign +1 forward, -1 back; gain multiplies both entries first
__device__ __forceinline__ float as_rotated(const float* x, int j, int dims, int interleaved, const float* tab, float sign,
                                            float gain) {
  if (j >= dims) return x[j] * gain;
  const int half = dims >> 1;
  int m, partner;
  bool lead;
  if (interleaved) { m = j >> 1; lead = !(j & 1); partner = j ^ 1; }
  else { lead = j < half; m = lead ? j : j - half; partner = lead ? j + half : j - half; }
  const float c = tab[2 * m], s = tab[2 * m + 1] * sign;
  const float a = x[j] * gain, b = x[partner] * gain;
  return lead ? a * c - b * s : a * c + b * s;
}

template <typename T>
__global__ void __launch_bounds__(128)
rotary_store_kernel(const float* __restrict__ qkv, int ld, int H, int G, int d, int dv, const float* __restrict__ qk_table,
                    int rot_dims, int interleaved, int v_norm, float v_eps, const float* __restrict__ v_table, int v_interleaved,
                    T* __restrict__ q_out, T* __restrict__ k_pages, long long k_page_stride, T* __restrict__ v_pages,
                    long long v_page_stride, const int* __restrict__ slot_mapping, int page_size, int v_from_k) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int n = blockIdx.x;
  const float* row = qkv + (size_t)n * ld;
  const int slot = slot_mapping ? slot_mapping[n] : -1;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  const float* qt = qk_table ? qk_table + (size_t)n * rot_dims : nullptr;
  const int dims = qt ? rot_dims : 0;
  for (int idx = threadIdx.x; idx < (H + G) * d; idx += blockDim.x) {
    const int head = idx / d, j = idx % d;
    const float y = as_rotated(row + (size_t)head * d, j, dims, interleaved, qt, 1.f, 1.f);
    if (head < H) q_out[(size_t)n * H * d + idx] = from_f32<T>(y);
    else if (slot >= 0)
      k_pages[(size_t)page * k_page_stride + ((size_t)(head - H) * page_size + off) * d + j] = from_f32<T>(y);
  }
  if (slot < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const float* vt = v_table ? v_table + (size_t)n * dv : nullptr;
  for (int g = warp; g < G; g += warps) {
    // v_from_k: the row holds no values; a value head is the key head as projected, before its rotation (dv == d)
    const float* v = v_from_k ? row + (size_t)(H + g) * d : row + (size_t)(H + G) * d + (size_t)g * dv;
    float gain = 1.f;
    if (v_norm) {
      float ss = 0.f;
      for (int j = lane; j < dv; j += 32) ss += v[j] * v[j];
      gain = 1.f / sqrtf(warp_sum(ss) / (float)dv + v_eps);
    }
    T* dst = v_pages + (size_t)page * v_page_stride + ((size_t)g * page_size + off) * dv;
    for (int j = lane; j < dv; j += 32) dst[j] = from_f32<T>(as_rotated(v, j, vt ? dv : 0, v_interleaved, vt, 1.f, gain));
  }
}

IFB_EXPORT int ifb_rotary_store(const float* qkv, int ld, int H, int G, int d, int dv, const float* qk_table, int rot_dims,
                                int interleaved, int v_norm, float v_eps, const float* v_table, int v_interleaved, void* q_out,
                                int dtype, void* k_pages, long long k_page_stride, void* v_pages, long long v_page_stride,
                                const int* slot_mapping, int page_size, int n, int v_from_k, cudaStream_t stream) {
  if (n <= 0) return IFB_OK;
  if (H < 1 || G < 1 || d < 1 || dv < 1 || page_size < 1 || (v_from_k && dv != d)) return IFB_ERR_SIZE;
  if ((qk_table && (rot_dims < 2 || rot_dims % 2 || rot_dims > d)) || (v_table && dv % 2)) return IFB_ERR_ARG;
  if (dtype == IFB_BF16)
    return ifb_launch(rotary_store_kernel<__nv_bfloat16>, dim3(n), dim3(128), 0, stream, qkv, ld, H, G, d, dv, qk_table, rot_dims,
                      interleaved, v_norm, v_eps, v_table, v_interleaved, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages,
                      k_page_stride, (__nv_bfloat16*)v_pages, v_page_stride, slot_mapping, page_size, v_from_k);
  if (dtype != IFB_F32) return IFB_ERR_DTYPE;
  return ifb_launch(rotary_store_kernel<float>, dim3(n), dim3(128), 0, stream, qkv, ld, H, G, d, dv, qk_table, rot_dims, interleaved,
                    v_norm, v_eps, v_table, v_interleaved, (float*)q_out, (float*)k_pages, k_page_stride, (float*)v_pages,
                    v_page_stride, slot_mapping, page_size, v_from_k);
}

// rows[n][head][:] are rotated in place by the token's angles, forward (sign 1) or back (sign -1), over `dims` entries
template <typename T>
__global__ void __launch_bounds__(128)
rotate_rows_kernel(T* __restrict__ rows, const float* __restrict__ table, int heads, int d, int dims, int interleaved, float sign) {
  extern __shared__ float sm[];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int n = blockIdx.x;
  T* row = rows + (size_t)n * heads * d;
  for (int i = threadIdx.x; i < heads * d; i += blockDim.x) sm[i] = to_f32<T>(row[i]);
  __syncthreads();
  const float* tab = table + (size_t)n * dims;
  for (int i = threadIdx.x; i < heads * d; i += blockDim.x)
    row[i] = from_f32<T>(as_rotated(sm + (i / d) * d, i % d, dims, interleaved, tab, sign, 1.f));
}

IFB_EXPORT int ifb_rotate_rows(void* rows, int dtype, const float* table, int n, int heads, int d, int dims, int interleaved,
                               int back, cudaStream_t stream) {
  if (n <= 0) return IFB_OK;
  if (heads < 1 || d < 1 || dims < 2 || dims % 2 || dims > d) return IFB_ERR_ARG;
  const size_t smem = (size_t)heads * d * sizeof(float);
  if (smem > 200 * 1024) return IFB_ERR_SIZE;
  const float sign = back ? -1.f : 1.f;
  if (dtype == IFB_BF16) {
    IFB_ALLOW_SMEM(rotate_rows_kernel<__nv_bfloat16>, smem);
    return ifb_launch(rotate_rows_kernel<__nv_bfloat16>, dim3(n), dim3(128), smem, stream, (__nv_bfloat16*)rows, table, heads, d, dims,
                      interleaved, sign);
  }
  if (dtype != IFB_F32) return IFB_ERR_DTYPE;
  IFB_ALLOW_SMEM(rotate_rows_kernel<float>, smem);
  return ifb_launch(rotate_rows_kernel<float>, dim3(n), dim3(128), smem, stream, (float*)rows, table, heads, d, dims, interleaved, sign);
}

template <typename T>
__global__ void __launch_bounds__(128)
paged_attention_streams_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, long long k_page_stride,
                               const T* __restrict__ v_pages, long long v_page_stride, const int* __restrict__ block_tables,
                               int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_lens, T* __restrict__ out,
                               int n_tokens, int n_req, int H, int G, int d, int dv, int page_size, float scale, int window,
                               const float* __restrict__ out_table, int out_interleaved) {
  extern __shared__ float sm[];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * warps + warp;
  if (item >= (long long)n_tokens * H) return;
  const int tok = (int)(item / H), h = (int)(item % H);
  const int kvh = h / (H / G);
  int lo = 0, hi = n_req;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cu_q[mid] <= tok) lo = mid; else hi = mid; }
  const int r = lo;
  T* o = out + ((size_t)tok * H + h) * dv;
  const int q_len = cu_q[r + 1] - cu_q[r];
  const int p = tok < cu_q[n_req] ? seq_lens[r] - q_len + (tok - cu_q[r]) : -1;
  if (p < 0) { for (int i = lane; i < dv; i += 32) o[i] = from_f32<T>(0.f); return; }      // padding rows
  const int first = window > 0 ? max(0, p - window + 1) : 0;
  float* qs = sm + (size_t)warp * (d + dv);
  float* os = qs + d;
  const T* qp = q + ((size_t)tok * H + h) * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_f32<T>(qp[i]);
  __syncwarp();
  const int* bt = block_tables + (size_t)r * bt_stride;
  float m = -INFINITY, l = 0.f;
  float acc[AS_MAX_D / 32];
#pragma unroll
  for (int c = 0; c < AS_MAX_D / 32; ++c) acc[c] = 0.f;
  for (int kb = first; kb <= p; kb += 32) {
    const int key = kb + lane;
    const bool valid = key <= p;
    float s = -INFINITY;
    if (valid) {
      const int page = bt[key / page_size];
      const T* kp = k_pages + (size_t)page * k_page_stride + ((size_t)kvh * page_size + key % page_size) * d;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32<T>(kp[i]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float pj = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int c = 0; c < AS_MAX_D / 32; ++c) acc[c] *= corr;
    const int count = min(32, p - kb + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const int kj = kb + jj;
      const int page = bt[kj / page_size];
      const T* vp = v_pages + (size_t)page * v_page_stride + ((size_t)kvh * page_size + kj % page_size) * dv;
#pragma unroll
      for (int c = 0; c < AS_MAX_D / 32; ++c) {
        const int e = lane + 32 * c;
        if (e < dv) acc[c] = fmaf(pv, to_f32<T>(vp[e]), acc[c]);
      }
    }
    m = m_new;
  }
  const float inv = 1.f / l;
  if (!out_table) {
#pragma unroll
    for (int c = 0; c < AS_MAX_D / 32; ++c) {
      const int e = lane + 32 * c;
      if (e < dv) o[e] = from_f32<T>(acc[c] * inv);
    }
    return;
  }
#pragma unroll
  for (int c = 0; c < AS_MAX_D / 32; ++c) {
    const int e = lane + 32 * c;
    if (e < dv) os[e] = acc[c] * inv;
  }
  __syncwarp();
  const float* tab = out_table + (size_t)tok * dv;
  for (int e = lane; e < dv; e += 32) o[e] = from_f32<T>(as_rotated(os, e, dv, out_interleaved, tab, -1.f, 1.f));
}

IFB_EXPORT int ifb_paged_attention_streams(const void* q, int dtype, const void* k_pages, long long k_page_stride,
                                           const void* v_pages, long long v_page_stride, const int* block_tables, int bt_stride,
                                           const int* cu_q, const int* seq_lens, void* out, int n_tokens, int n_req, int H, int G,
                                           int d, int dv, int page_size, float scale, int window, const float* out_table,
                                           int out_interleaved, cudaStream_t stream) {
  if (n_tokens <= 0 || n_req <= 0) return IFB_OK;
  if (d < 1 || d > AS_MAX_D || dv < 1 || dv > AS_MAX_D) return IFB_ERR_SIZE;
  if (G < 1 || H % G || page_size < 1 || window < 0 || (out_table && dv % 2)) return IFB_ERR_ARG;
  const int warps = 4;
  const long long items = (long long)n_tokens * H;
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  const size_t smem = (size_t)warps * (d + dv) * sizeof(float);
  if (dtype == IFB_F32)
    return ifb_launch(paged_attention_streams_kernel<float>, dim3(blocks), dim3(warps * 32), smem, stream, (const float*)q,
                      (const float*)k_pages, k_page_stride, (const float*)v_pages, v_page_stride, block_tables, bt_stride, cu_q,
                      seq_lens, (float*)out, n_tokens, n_req, H, G, d, dv, page_size, scale, window, out_table, out_interleaved);
  if (dtype == IFB_BF16)
    return ifb_launch(paged_attention_streams_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, stream,
                      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, k_page_stride, (const __nv_bfloat16*)v_pages,
                      v_page_stride, block_tables, bt_stride, cu_q, seq_lens, (__nv_bfloat16*)out, n_tokens, n_req, H, G, d, dv,
                      page_size, scale, window, out_table, out_interleaved);
  return IFB_ERR_DTYPE;
}
