// The recurrent block around a real-gated linear recurrent unit (RG-LRU), after its two input projections:
//
// (1) rglru_conv: u_t = conv_b + sum_(j <= K) w[:, j] * xin_(t - K + j), K = taps - 1, xin = x_raw + x_bias, per channel over
// each request's tokens in order, zeros before a sequence's start.  The K inputs before a portion come from the request's
// state [slots, max(K, 1), width] (float32, oldest first), which then takes the portion's last K inputs.  u is written
// twice: token-major in float32 (the recurrence reads it) and block-major [blocks, seg, width / blocks] in the products'
// dtype (the block-diagonal gate products read it as a grouped product, a block being what an expert is there); with two
// terms a block's row is twice as long and holds every number's rounding and then what each rounding left out, so that a
// product against the gate matrix repeated along k sees 16 bits of every number.
//
// (2) rglru_scan: per channel of a float32 state, r = sigmoid(gr + a_bias), i = sigmoid(gi + i_bias) from the gate products'
// float32 results (block-major rows of [r | i]), log a = -scale * r * softplus(lam), a = exp(log a),
// S <- a S + sqrt(1 - a^2) * i * u, out = S * gelu_tanh(y_raw + y_bias).  A thread owns a (request, channel) and walks the
// request's tokens of the step from the slot's state, eight tokens' numbers formed ahead of the chain.  Long portions run
// in three launches: every (token, channel) pair's decay and input term side by side, left where the pair's raw gates were;
// then, over chunks of 32 tokens side by side, every chunk's map S -> A S + B from zero (the slot's state is set aside);
// then each chunk folds the maps of the chunks before its own onto that state, walks its tokens and writes the outputs (the
// last chunk of a request writes the state).  The two forms differ by rounding only.  Everything here is float32 arithmetic.
#include "common.cuh"
#include <math.h>

// ------------------------------------------------------------------------------------------ the convolution
// A block is (eight tokens, or one in a small step; slice of 128 * V channels) and takes its tokens one after another; a thread
// owns V neighbouring channels (V = 4 where widths and addresses
// allow 16-byte accesses, else 1).
template <int V> struct RgVec { float v[V]; };
template <int V> __device__ __forceinline__ RgVec<V> rg_load(const float* p) {
  RgVec<V> r;
  if constexpr (V == 4) { const float4 f = *reinterpret_cast<const float4*>(p); r.v[0] = f.x; r.v[1] = f.y; r.v[2] = f.z; r.v[3] = f.w; }
  else r.v[0] = *p;
  return r;
}
template <int V> __device__ __forceinline__ void rg_store(float* p, const RgVec<V>& r) {
  if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  else *p = r.v[0];
}
template <int V> __device__ __forceinline__ void rg_store(__nv_bfloat16* p, const RgVec<V>& r) {
  if constexpr (V == 4) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(r.v[0], r.v[1]), hi = __floats2bfloat162_rn(r.v[2], r.v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  } else *p = __float2bfloat16(r.v[0]);
}

constexpr int RC_TOKENS = 8;        // tokens a block of a large step walks: the start of a block costs a chain of small loads
template <typename TB, int V>
__global__ void __launch_bounds__(128)
rglru_conv_kernel(const float* __restrict__ proj, long long ld, int x_col, const float* __restrict__ x_bias,
                  const float* __restrict__ conv_w, const float* __restrict__ conv_b, float* __restrict__ state,
                  const int* __restrict__ state_slots, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                  const int* __restrict__ req_index, float* __restrict__ u, TB* __restrict__ ub, int seg, int blocks,
                  int* __restrict__ offsets, int* __restrict__ tile_block, int tile, int width, int taps, int tokens, int per_block, int terms) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  if (blockIdx.x == 0 && blockIdx.y == 0) {
    for (int b = threadIdx.x; b <= blocks; b += blockDim.x) offsets[b] = b * seg;
    if (tile_block != nullptr) {
      const int per = seg / tile;
      for (int j = threadIdx.x; j < blocks * per; j += blockDim.x) tile_block[j] = j / per;
    }
  }
  const int e = (blockIdx.y * blockDim.x + threadIdx.x) * V;      // this thread's first channel
  if (e >= width) return;
  const int bs = width / blocks;
  const RgVec<V> xb = rg_load<V>(x_bias + e), cb = rg_load<V>(conv_b + e);
  const int t_end = min(tokens, ((int)blockIdx.x + 1) * per_block);
  for (int t = blockIdx.x * per_block; t < t_end; ++t) {
  const int r = req_index[t];
  const int q0 = cu_q[r], len = cu_q[r + 1] - q0, i = t - q0;
  // a row of a block holds bs numbers, or (terms == 2) 2 bs: every number's rounding to TB and then what each rounding left out
  const int rowlen = terms * bs;
  TB* ub_e = ub + ((size_t)(e / bs) * seg) * rowlen + e % bs;      // + row * rowlen: the V channels lie in one block (bs % V == 0)
  if (seq_lens[r] <= 0) {                              // a padding row of a recorded step: it stores and sees nothing
    RgVec<V> z;
#pragma unroll
    for (int v = 0; v < V; ++v) z.v[v] = 0.f;
    rg_store<V>(u + (size_t)t * width + e, z);
    rg_store<V>(ub_e + (size_t)t * rowlen, z);
    if (terms == 2) rg_store<V>(ub_e + (size_t)t * rowlen + bs, z);
    continue;
  }
  const int K = taps - 1, Kp = K > 0 ? K : 1;
  if (i > 0 && i < K) continue;                        // the thread that has the portion's first token computes these
  float* st = state + (size_t)state_slots[r] * Kp * width + e;
  const float* xr = proj + x_col + e;
  // input idx of the portion (negative: from the state)
  auto input = [&](int idx) -> RgVec<V> {
    if (idx < 0) return rg_load<V>(st + (size_t)(K + idx) * width);
    RgVec<V> x = rg_load<V>(xr + (size_t)(q0 + idx) * ld);
#pragma unroll
    for (int v = 0; v < V; ++v) x.v[v] += xb.v[v];
    return x;
  };
  auto token = [&](int ii) {
    RgVec<V> acc = cb;
    for (int j = 0; j <= K; ++j) {
      const RgVec<V> x = input(ii - K + j);
#pragma unroll
      for (int v = 0; v < V; ++v) acc.v[v] = fmaf(__ldg(conv_w + (size_t)(e + v) * taps + j), x.v[v], acc.v[v]);
    }
    rg_store<V>(u + (size_t)(q0 + ii) * width + e, acc);
    rg_store<V>(ub_e + (size_t)(q0 + ii) * rowlen, acc);
    if (terms == 2) {
      RgVec<V> rest;
#pragma unroll
      for (int v = 0; v < V; ++v) rest.v[v] = acc.v[v] - to_f32<TB>(from_f32<TB>(acc.v[v]));
      rg_store<V>(ub_e + (size_t)(q0 + ii) * rowlen + bs, rest);
    }
  };
  if (i >= K) {                                        // reads this step's rows only
    token(i);
    continue;
  }
  // i == 0 and K > 0: the tokens that read the state, then the state's replacement; a channel is one thread's throughout
  const int lim = len < K ? len : K;
  for (int ii = 0; ii < lim; ++ii) token(ii);
  for (int k = 0; k < K; ++k) {                        // new entry k is the input at portion index len - K + k
    const int src = len - K + k;
    rg_store<V>(st + (size_t)k * width, src >= 0 ? input(src) : rg_load<V>(st + (size_t)(k + len) * width));
  }
  }
}

IFB_EXPORT int ifb_rglru_conv(const float* proj, long long ld, int x_col, const float* x_bias, const float* conv_w,
                              const float* conv_b, float* state, const int* state_slots, const int* cu_q, const int* seq_lens,
                              const int* req_index, float* u, void* ub, int ub_dtype, int seg, int blocks, int* offsets,
                              int* tile_block, int tile, int n, int width, int taps, int terms, cudaStream_t stream) {
  if (n <= 0) return IFB_OK;
  if (terms != 1 && terms != 2) return IFB_ERR_ARG;
  if (width < 1 || blocks < 1 || width % blocks || taps < 1 || seg < n || x_col < 0 || x_col + width > ld) return IFB_ERR_SIZE;
  if (tile_block != nullptr && (tile < 1 || seg % tile)) return IFB_ERR_SIZE;
  const bool vec = (width / blocks) % 4 == 0 && ld % 4 == 0 && x_col % 4 == 0 &&
                   (((uintptr_t)proj | (uintptr_t)x_bias | (uintptr_t)conv_b | (uintptr_t)state | (uintptr_t)u | (uintptr_t)ub) & 15) == 0;
#define RC_LAUNCH(TB, V)                                                                                                          \
  {                                                                                                                               \
    const int ys = (width + 128 * V - 1) / (128 * V);                                                                             \
    const int per = (long long)n * ys >= 4096 ? RC_TOKENS : 1;          /* a small step keeps a block per token */                \
    return ifb_launch(rglru_conv_kernel<TB, V>, dim3((n + per - 1) / per, ys), dim3(128), 0, stream, proj, ld, x_col, x_bias,      \
                      conv_w, conv_b, state, state_slots, cu_q, seq_lens, req_index, u, (TB*)ub, seg, blocks, offsets, tile_block, \
                      tile, width, taps, n, per, terms);                                                                                 \
  }
  if (ub_dtype == IFB_BF16) { if (vec) RC_LAUNCH(__nv_bfloat16, 4); RC_LAUNCH(__nv_bfloat16, 1); }
  if (ub_dtype != IFB_F32) return IFB_ERR_DTYPE;
  if (vec) RC_LAUNCH(float, 4);
  RC_LAUNCH(float, 1);
#undef RC_LAUNCH
}

// ------------------------------------------------------------------------------------------ the recurrence
constexpr int RG_CHUNK = 32;
constexpr int RG_AHEAD = 8;        // tokens whose numbers are formed before the chain takes them
constexpr int RG_THREADS = 128;

struct RgArgs {
  float* gates; int seg, bs;               // [blocks * seg, 2 bs]: row b * seg + t holds r | i of block b
  const float* a_bias; const float* i_bias; const float* lam; float scale;
  const float* u;                          // [n, width]
  const float* proj; long long ld; int y_col; const float* y_bias;
  int width;
};

__device__ __forceinline__ float rg_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float rg_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float rg_gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// the token's decay a and input term sqrt(1 - a^2) * i * u for channel e = (b, c)
__device__ __forceinline__ void rg_token(const RgArgs& g, int t, int e, int b, int c, float sp, float& a, float& in) {
  const float* row = g.gates + ((size_t)b * g.seg + t) * (2 * g.bs);
  const float r = rg_sigmoid(row[c] + g.a_bias[e]);
  const float i = rg_sigmoid(row[g.bs + c] + g.i_bias[e]);
  const float loga = -g.scale * r * sp;
  a = expf(loga);
  in = sqrtf(fmaxf(-expm1f(2.f * loga), 0.f)) * i * g.u[(size_t)t * g.width + e];
}

// The chunked form's first launch: every (token, channel) pair's decay and input term, side by side, left where the pair's
// raw gates were (each pair is one thread's).
__global__ void __launch_bounds__(RG_THREADS)
rglru_terms_kernel(RgArgs g, int tokens) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int e = blockIdx.x * RG_THREADS + threadIdx.x;
  if (e >= g.width) return;
  const int b = e / g.bs, c = e - b * g.bs;
  const float sp = rg_softplus(g.lam[e]);
  const int t0 = blockIdx.y * RG_AHEAD;
  float a[RG_AHEAD], in[RG_AHEAD];
#pragma unroll
  for (int j = 0; j < RG_AHEAD; ++j)
    if (t0 + j < tokens) rg_token(g, t0 + j, e, b, c, sp, a[j], in[j]);
#pragma unroll
  for (int j = 0; j < RG_AHEAD; ++j)
    if (t0 + j < tokens) {
      float* row = g.gates + ((size_t)b * g.seg + t0 + j) * (2 * g.bs);
      row[c] = a[j];
      row[g.bs + c] = in[j];
    }
}

// MODE 0: a thread walks all tokens of (request, channel) from the slot's state and writes it back.
// MODE 1: a thread forms the map of (chunk, channel) from zero out of the decays and input terms that rglru_terms_kernel
//         left in the gates' place; chunk 0 of a request sets the slot's state aside.
// MODE 2: a thread folds the earlier chunks' maps onto the state set aside, walks its chunk, writes outputs (and the state
//         after the request's last chunk).
// scratch: [requests][width] states set aside, then [chunk slots][2][width] maps; chunk slots are numbered request by
// request, ceil(len / RG_CHUNK) each.
template <typename TO, int MODE>
__global__ void __launch_bounds__(RG_THREADS)
rglru_scan_kernel(RgArgs g, float* __restrict__ state, const int* __restrict__ state_slots, const int* __restrict__ cu_q,
                  const int* __restrict__ seq_lens, TO* __restrict__ out, float* __restrict__ scratch, int requests) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int e = blockIdx.y * RG_THREADS + threadIdx.x;
  int r, first_chunk = 0, chunk = 0;
  if (MODE == 0) {
    r = blockIdx.x;
  } else {
    int acc = 0;
    for (r = 0; r < requests; ++r) {
      const int cnt = (cu_q[r + 1] - cu_q[r] + RG_CHUNK - 1) / RG_CHUNK;
      if ((int)blockIdx.x < acc + cnt) break;
      acc += cnt;
    }
    if (r >= requests) return;
    first_chunk = acc;
    chunk = blockIdx.x - acc;
  }
  if (e >= g.width) return;
  const int q0 = cu_q[r], len = cu_q[r + 1] - q0;
  const int lo = MODE == 0 ? 0 : chunk * RG_CHUNK, hi = MODE == 0 ? len : min(len, lo + RG_CHUNK);
  if (seq_lens[r] <= 0) {                              // a padding row: no state, zeros out
    if (MODE != 1)
      for (int t = q0 + lo; t < q0 + hi; ++t) out[(size_t)t * g.width + e] = from_f32<TO>(0.f);
    return;
  }
  const int b = e / g.bs, c = e - b * g.bs;
  const float sp = rg_softplus(g.lam[e]);
  float* st = state + (size_t)state_slots[r] * g.width + e;
  float* aside = scratch + (size_t)r * g.width + e;
  float* maps = scratch + (size_t)requests * g.width;
  if (MODE == 1) {
    if (chunk == 0) *aside = *st;
    float A = 1.f, B = 0.f;
    for (int t = q0 + lo; t < q0 + hi; t += RG_AHEAD) {
      float a[RG_AHEAD], in[RG_AHEAD];
#pragma unroll
      for (int j = 0; j < RG_AHEAD; ++j) {
        a[j] = 1.f; in[j] = 0.f;
        if (t + j < q0 + hi) {
          const float* row = g.gates + ((size_t)b * g.seg + t + j) * (2 * g.bs);
          a[j] = row[c]; in[j] = row[g.bs + c];
        }
      }
#pragma unroll
      for (int j = 0; j < RG_AHEAD; ++j) { A *= a[j]; B = fmaf(a[j], B, in[j]); }
    }
    maps[((size_t)(first_chunk + chunk) * 2) * g.width + e] = A;
    maps[((size_t)(first_chunk + chunk) * 2 + 1) * g.width + e] = B;
    return;
  }
  float S = MODE == 0 ? *st : *aside;
  if (MODE == 2) {
#pragma unroll 8
    for (int k = 0; k < chunk; ++k)
      S = fmaf(maps[((size_t)(first_chunk + k) * 2) * g.width + e], S, maps[((size_t)(first_chunk + k) * 2 + 1) * g.width + e]);
  }
  const float yb = g.y_bias[e];
  for (int t = q0 + lo; t < q0 + hi; t += RG_AHEAD) {
    float a[RG_AHEAD], in[RG_AHEAD], y[RG_AHEAD];
#pragma unroll
    for (int j = 0; j < RG_AHEAD; ++j) {
      a[j] = 1.f; in[j] = 0.f; y[j] = 0.f;
      if (t + j < q0 + hi) {
        if (MODE == 2) {
          const float* row = g.gates + ((size_t)b * g.seg + t + j) * (2 * g.bs);
          a[j] = row[c]; in[j] = row[g.bs + c];
        } else {
          rg_token(g, t + j, e, b, c, sp, a[j], in[j]);
        }
        y[j] = rg_gelu_tanh(g.proj[(size_t)(t + j) * g.ld + g.y_col + e] + yb);
      }
    }
#pragma unroll
    for (int j = 0; j < RG_AHEAD; ++j) {
      S = fmaf(a[j], S, in[j]);
      if (t + j < q0 + hi) out[(size_t)(t + j) * g.width + e] = from_f32<TO>(S * y[j]);
    }
  }
  if (MODE == 0 || hi == len) *st = S;
}

IFB_EXPORT long long ifb_rglru_scratch_floats(int n, int requests, int width) {
  const long long chunks = (long long)(n + RG_CHUNK - 1) / RG_CHUNK + requests;
  return ((long long)requests + 2 * chunks) * width;
}

template <typename TO>
static int rg_launch(const RgArgs& g, float* state, const int* state_slots, const int* cu_q, const int* seq_lens, TO* out,
                     float* scratch, int requests, int n, cudaStream_t stream) {
  const unsigned ey = (unsigned)((g.width + RG_THREADS - 1) / RG_THREADS);
  if (scratch == nullptr)
    return ifb_launch(rglru_scan_kernel<TO, 0>, dim3(requests, ey), dim3(RG_THREADS), 0, stream, g, state, state_slots, cu_q,
                      seq_lens, out, scratch, requests);
  const unsigned chunks = (unsigned)((n + RG_CHUNK - 1) / RG_CHUNK + requests);
  int rc = ifb_launch(rglru_terms_kernel, dim3(ey, (unsigned)((n + RG_AHEAD - 1) / RG_AHEAD)), dim3(RG_THREADS), 0, stream, g, n);
  if (rc != IFB_OK) return rc;
  rc = ifb_launch(rglru_scan_kernel<TO, 1>, dim3(chunks, ey), dim3(RG_THREADS), 0, stream, g, state, state_slots, cu_q,
                            seq_lens, out, scratch, requests);
  if (rc != IFB_OK) return rc;
  return ifb_launch(rglru_scan_kernel<TO, 2>, dim3(chunks, ey), dim3(RG_THREADS), 0, stream, g, state, state_slots, cu_q, seq_lens,
                    out, scratch, requests);
}

// scratch null: the one-launch walk; else the chunked form (ifb_rglru_scratch_floats floats)
IFB_EXPORT int ifb_rglru_scan(float* gates, int seg, int blocks, const float* a_bias, const float* i_bias, const float* lam,
                              float scale, const float* u, const float* proj, long long ld, int y_col, const float* y_bias,
                              float* state, const int* state_slots, const int* cu_q, const int* seq_lens, void* out, int out_dtype,
                              float* scratch, int requests, int n, int width, cudaStream_t stream) {
  if (n <= 0 || requests <= 0) return IFB_OK;
  if (width < 1 || blocks < 1 || width % blocks || seg < n || y_col < 0 || y_col + width > ld) return IFB_ERR_SIZE;
  const RgArgs g{gates, seg, width / blocks, a_bias, i_bias, lam, scale, u, proj, ld, y_col, y_bias, width};
  if (out_dtype == IFB_BF16)
    return rg_launch<__nv_bfloat16>(g, state, state_slots, cu_q, seq_lens, (__nv_bfloat16*)out, scratch, requests, n, stream);
  if (out_dtype != IFB_F32) return IFB_ERR_DTYPE;
  return rg_launch<float>(g, state, state_slots, cu_q, seq_lens, (float*)out, scratch, requests, n, stream);
}
