// Attention over cached latents, in the absorbed form: with k_h = UK_h c and v_h = UV_h c, the score q_h . k_h equals
// (UK_h^T q_h) . c, and the weighted sum of values equals UV_h applied to the weighted sum of latents.  So all heads of a
// token attend over the same rows c_j (plus one small rotated key part shared by the heads), and neither keys nor values
// are ever formed for the context.  Scores, softmax weights and sums are float32.
//
// q_lat [heads, seg, rank] float32 (head-major, `seg` rows per head), q_rot [n, heads, rot] float32, latent pages
// [pages, 1, page_size, rank] and rotated-key pages [pages, 1, page_size, rot] in the cache's dtype.  Position i sees j <= i,
// with a window only i - j < window.  sink [heads] (optional): exp(sink_h) joins the softmax's denominator and carries no
// value, which is the running softmax started at maximum sink_h with sum 1.  out [heads, seg, rank]: the weighted sum of
// latents per head, for the grouped product with UV that follows.
#include "common.cuh"
#include <math.h>

constexpr int LA_WARPS = 4;      // (token, head) pairs per block, a warp each
constexpr int LA_KEYS = 4;       // keys whose scores a warp forms together

template <typename TC, typename TO, int PER>      // PER: latent entries per lane (rank <= 32 * PER)
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot, int seg, const TC* __restrict__ lat_pages,
                        const TC* __restrict__ rot_pages, const int* __restrict__ block_tables, int table_stride, int page_size,
                        const int* __restrict__ cu_q, const int* __restrict__ seq_lens, const int* __restrict__ req_index,
                        const void* __restrict__ sink, int stype, TO* __restrict__ out, int tokens, int heads, int rank, int rot,
                        float scale, int window) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long pair = (long long)blockIdx.x * LA_WARPS + (threadIdx.x >> 5);
  if (pair >= (long long)tokens * heads) return;
  const int t = (int)(pair / heads), h = (int)(pair - (long long)t * heads);
  const int r = req_index[t];
  const int q0 = cu_q[r], q1 = cu_q[r + 1], L = seq_lens[r];
  TO* o = out + ((size_t)h * seg + t) * rank;
  if (L <= 0) {
    for (int e = lane; e < rank; e += 32) o[e] = from_f32<TO>(0.f);
    return;
  }
  const int p = L - (q1 - q0) + (t - q0);
  const int first = window > 0 ? max(0, p - window + 1) : 0;
  float q[PER], acc[PER];
  const float* ql = q_lat + ((size_t)h * seg + t) * rank;
#pragma unroll
  for (int k = 0; k < PER; ++k) { const int e = lane + 32 * k; q[k] = e < rank ? ql[e] : 0.f; acc[k] = 0.f; }
  const float* qr = q_rot + ((size_t)t * heads + h) * rot;
  float m = -INFINITY, l = 0.f;
  if (sink != nullptr) { m = load_as_f32(sink, stype, h); l = 1.f; }
  const int* table = block_tables + (size_t)r * table_stride;
  for (int j0 = first; j0 <= p; j0 += LA_KEYS) {
    float s[LA_KEYS];
    const TC* rows[LA_KEYS];
#pragma unroll
    for (int u = 0; u < LA_KEYS; ++u) {
      const int j = j0 + u;
      s[u] = 0.f;
      rows[u] = nullptr;
      if (j <= p) {
        const size_t slot = (size_t)table[j / page_size] * page_size + j % page_size;
        rows[u] = lat_pages + slot * rank;
#pragma unroll
        for (int k = 0; k < PER; ++k) { const int e = lane + 32 * k; if (e < rank) s[u] = fmaf(q[k], to_f32<TC>(rows[u][e]), s[u]); }
        const TC* kr = rot_pages + slot * rot;
        for (int d = lane; d < rot; d += 32) s[u] = fmaf(qr[d], to_f32<TC>(kr[d]), s[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < LA_KEYS; ++u) s[u] = warp_sum(s[u]) * scale;
#pragma unroll
    for (int u = 0; u < LA_KEYS; ++u) {
      if (rows[u] == nullptr) continue;
      const float m_new = fmaxf(m, s[u]);
      const float corr = expf(m - m_new), w = expf(s[u] - m_new);      // exp(-inf) = 0 at the first key without a sink
      l = fmaf(l, corr, w);
#pragma unroll
      for (int k = 0; k < PER; ++k) { const int e = lane + 32 * k; if (e < rank) acc[k] = fmaf(acc[k], corr, w * to_f32<TC>(rows[u][e])); }
      m = m_new;
    }
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int k = 0; k < PER; ++k) { const int e = lane + 32 * k; if (e < rank) o[e] = from_f32<TO>(acc[k] * inv); }
}

template <typename TC, typename TO>
static int la_launch(int per, dim3 grid, cudaStream_t stream, const float* q_lat, const float* q_rot, int seg, const void* lat_pages,
                     const void* rot_pages, const int* block_tables, int table_stride, int page_size, const int* cu_q,
                     const int* seq_lens, const int* req_index, const void* sink, int stype, void* out, int tokens, int heads, int rank,
                     int rot, float scale, int window) {
#define LA_CASE(P)                                                                                                              \
  return ifb_launch(latent_attention_kernel<TC, TO, P>, grid, dim3(LA_WARPS * 32), 0, stream, q_lat, q_rot, seg,                \
                    (const TC*)lat_pages, (const TC*)rot_pages, block_tables, table_stride, page_size, cu_q, seq_lens, req_index,  \
                    sink, stype, (TO*)out, tokens, heads, rank, rot, scale, window)
  if (per <= 2) LA_CASE(2);
  if (per <= 4) LA_CASE(4);
  if (per <= 8) LA_CASE(8);
  if (per <= 16) LA_CASE(16);
  LA_CASE(32);
#undef LA_CASE
}

IFB_EXPORT int ifb_latent_attention(const float* q_lat, const float* q_rot, int seg, const void* lat_pages, const void* rot_pages,
                                    int ctype, const int* block_tables, int table_stride, int page_size, const int* cu_q,
                                    const int* seq_lens, const int* req_index, const void* sink, int stype, void* out, int otype,
                                    int tokens, int heads, int rank, int rot, float scale, int window, cudaStream_t stream) {
  if (tokens <= 0) return IFB_OK;
  if (heads < 1 || rank < 1 || rank > 1024 || rot < 0 || page_size < 1 || seg < tokens || window < 0) return IFB_ERR_SIZE;
  const long long pairs = (long long)tokens * heads;
  const dim3 grid((unsigned)((pairs + LA_WARPS - 1) / LA_WARPS));
  const int per = (rank + 31) / 32;
  if (ctype == IFB_BF16 && otype == IFB_BF16)
    return la_launch<__nv_bfloat16, __nv_bfloat16>(per, grid, stream, q_lat, q_rot, seg, lat_pages, rot_pages, block_tables,
                                                   table_stride, page_size, cu_q, seq_lens, req_index, sink, stype, out, tokens, heads,
                                                   rank, rot, scale, window);
  if (ctype == IFB_F32 && otype == IFB_F32)
    return la_launch<float, float>(per, grid, stream, q_lat, q_rot, seg, lat_pages, rot_pages, block_tables, table_stride, page_size,
                                   cu_q, seq_lens, req_index, sink, stype, out, tokens, heads, rank, rot, scale, window);
  return IFB_ERR_DTYPE;
}
