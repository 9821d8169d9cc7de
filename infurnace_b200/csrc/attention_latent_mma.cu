// Attention over cached latents on tensor cores (bfloat16 operands, float32 scores, softmax and sums), the absorbed form of
// attention_latent.cu: every head of a token attends over the same rows [latent | rotated key part], so the (token, head)
// pairs of a request are the rows of one product against those rows, and the weighted sum is taken over the latent itself.
//
// A CTA takes 64 consecutive rows rho = (token - first token of the step) * heads + head of one request (16 per warp) and
// walks the keys they see in tiles of 64, two tiles in flight (16-byte cp.async, rows padded by 16 bytes so that ldmatrix
// meets no bank conflict).  Scores S = Q K^T by mma.sync m16n8k16 over the latent's and the rotated part's columns; mask
// (causal, window), running maximum and sum in the base-2 domain; the weights, rounded to bfloat16, are the left operand
// of O += P C over the latent's columns, which the same shared-memory rows give through ldmatrix.trans.  A sink starts a
// row's maximum at the sink and its sum at 1.  With `splits` > 1 (few rows and a long context: decode) the keys of a CTA's
// rows are divided among that many CTAs, which write unnormalised sums with their maximum and denominator, and a second
// kernel merges them (the sink joins there).
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;
constexpr int LM_ROWS = 64, LM_KEYS = 64, LM_THREADS = 128;

__device__ __forceinline__ uint32_t lm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lm_cp16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;                   // 0: zeros are written and src is not read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(lm_smem(dst)), "l"(src), "r"(sz));
}
__device__ __forceinline__ void lm_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void lm_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void lm_ldm(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(lm_smem(p)));
}
__device__ __forceinline__ void lm_ldm_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(lm_smem(p)));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// what the rounding of (lo, hi) to bfloat16 left out, itself rounded to bfloat16: the second term of a two-term weight
__device__ __forceinline__ uint32_t lm_pack_rest(float lo, float hi) {
  const float2 f = __bfloat1622float2(__floats2bfloat162_rn(lo, hi));
  return lm_pack(lo - f.x, hi - f.y);
}
// 2^x of a weight that is rounded to bfloat16 next: the approximation's error is far below that rounding
__device__ __forceinline__ float lm_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
constexpr float LM_LOG2E = 1.4426950408889634f;

// Scratch of the split form, per (request, row tile, split): 64 rows of RANK sums, then 64 maxima, then 64 denominators.
__host__ __device__ inline size_t lm_part_floats(int rank_pad) { return (size_t)LM_ROWS * (rank_pad + 2); }

// RANK: columns of the latent in shared memory (the latent's width rounded up; the rest zeros).  ROTP: the rotated part's
// columns there, known when the kernel is compiled (row length, offsets of every ldmatrix and the trip counts are then
// constants), or -1: the argument rot_pad says.
template <int RANK, int ROTP>
__global__ void __launch_bounds__(LM_THREADS, RANK <= 64 ? 4 : RANK <= 128 ? 3 : 2)
latent_attention_mma_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot, int seg, const bf16* __restrict__ lat_pages,
                            const bf16* __restrict__ rot_pages, const int* __restrict__ block_tables, int table_stride, int page_size,
                            const int* __restrict__ cu_q, const int* __restrict__ seq_lens, const void* __restrict__ sink, int stype,
                            bf16* __restrict__ out, float* __restrict__ part, int heads, int rank, int rot, int rot_pad,
                            float scale, int window, int splits, int terms) {
  extern __shared__ __align__(16) unsigned char lm_raw[];
  if (ROTP >= 0) rot_pad = ROTP;
  const int KD = RANK + rot_pad, LD = KD + 8;      // columns of a row, and its length in shared memory
  bf16* Qs = reinterpret_cast<bf16*>(lm_raw);
  bf16* Ks = Qs + (size_t)LM_ROWS * LD;            // two stages of LM_KEYS rows
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int r = blockIdx.y, split = blockIdx.z, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q0 = cu_q[r], nq = cu_q[r + 1] - q0, L = seq_lens[r];
  // the last rows of a request see the most keys: they start first, so that the grid's tail is made of short CTAs
  const int tile_x = gridDim.x - 1 - blockIdx.x;
  const int nrows = nq * heads, row0 = tile_x * LM_ROWS;
  if (row0 >= nrows) return;
  if (L <= 0) {                                    // a padding request of a recorded step: zeros
    if (split == 0)
      for (int i = tid; i < min(LM_ROWS, nrows - row0) * rank; i += LM_THREADS) {
        const int rho = row0 + i / rank;
        out[((size_t)(rho % heads) * seg + q0 + rho / heads) * rank + i % rank] = __float2bfloat16(0.f);
      }
    return;                                        // (the merge kernel skips such a request by its length)
  }
  const int p_first = L - nq;
  const int p_lo = p_first + row0 / heads, p_hi = p_first + min(nrows - 1, row0 + LM_ROWS - 1) / heads;
  const int k_lo = window > 0 ? max(0, p_lo - window + 1) : 0;
  int kb = k_lo, ke = p_hi;
  if (splits > 1) {
    const int per = ((p_hi - k_lo + splits) / splits + LM_KEYS - 1) / LM_KEYS * LM_KEYS;
    kb = k_lo + split * per;
    ke = min(p_hi, kb + per - 1);
  }
  float* my_part = part ? part + ((size_t)(r * gridDim.x + tile_x) * splits + split) * lm_part_floats(RANK) : nullptr;
  const int* table = block_tables + (size_t)r * table_stride;
  // two threads per key: one look at the block table per thread and tile (made one tile ahead, so that no copy waits for
  // it), then 16-byte pieces of the row alternately
  const int my_key = tid >> 1;
  auto page_of = [&](int tile0) {
    const int j = tile0 + my_key;
    return j >= kb && j <= ke ? table[j / page_size] : 0;
  };
  auto load_tile = [&](int tile0, int stage, int page) {
    const int j = tile0 + my_key;
    bf16* dst = Ks + ((size_t)stage * LM_KEYS + my_key) * LD;
    const bool live = j >= kb && j <= ke;
    const size_t slot = live ? (size_t)page * page_size + j % page_size : 0;
    const bf16* lat = lat_pages + slot * rank;
    const bf16* rk = rot_pages + slot * rot;
    for (int c = (tid & 1) * 8; c < KD; c += 16) {
      const bool in_lat = c < rank, in_rot = c >= RANK && c - RANK < rot;
      lm_cp16(dst + c, in_lat ? lat + c : in_rot ? rk + (c - RANK) : lat_pages, live && (in_lat || in_rot));
    }
  };
  float o[RANK / 8][4];
#pragma unroll
  for (int n = 0; n < RANK / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  // per thread two rows: lane / 4 and lane / 4 + 8 of the warp's sixteen
  const int rowA = row0 + warp * 16 + (lane >> 2), rowB = rowA + 8;
  const int pA = rowA < nrows ? p_first + rowA / heads : -1, pB = rowB < nrows ? p_first + rowB / heads : -1;
  const int loA = window > 0 ? pA - window + 1 : 0, loB = window > 0 ? pB - window + 1 : 0;
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
  if (sink != nullptr && splits == 1) {
    // the four lanes that share a row hold parts of its sum: the sink's 1 stands on one of them
    if (pA >= 0) { mA = load_as_f32(sink, stype, rowA % heads) * LM_LOG2E; lA = (lane & 3) == 0 ? 1.f : 0.f; }
    if (pB >= 0) { mB = load_as_f32(sink, stype, rowB % heads) * LM_LOG2E; lB = (lane & 3) == 0 ? 1.f : 0.f; }
  }
  const bool warp_live = row0 + warp * 16 < nrows;
  const float sc = scale * LM_LOG2E;
  const int ntiles = ke >= kb ? (ke - kb) / LM_KEYS + 1 : 0;
  if (ntiles > 0) load_tile(kb, 0, page_of(kb));
  lm_commit();
  // ---- the rows' queries: [latent-space part | rotated part], bfloat16; two threads per row, four columns (16 bytes of
  // float32) at a time, while the first tile of keys is on its way
  {
    const int row = tid >> 1, rho = row0 + row;
    const bool live = rho < nrows;
    const int t = live ? q0 + rho / heads : 0, h = live ? rho % heads : 0;
    const float* ql = q_lat + ((size_t)h * seg + t) * rank;
    const float* qr = q_rot + ((size_t)t * heads + h) * rot;
    bf16* dst = Qs + (size_t)row * LD;
#pragma unroll 6
    for (int c = (tid & 1) * 4; c < KD; c += 8) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live && c < rank) v = *reinterpret_cast<const float4*>(ql + c);
      else if (live && c >= RANK && c - RANK < rot) v = *reinterpret_cast<const float4*>(qr + (c - RANK));
      *reinterpret_cast<uint2*>(dst + c) = make_uint2(lm_pack(v.x, v.y), lm_pack(v.z, v.w));
    }
  }
  int page_next = ntiles > 1 ? page_of(kb + LM_KEYS) : 0;
  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) load_tile(kb + (it + 1) * LM_KEYS, (it + 1) & 1, page_next);
    lm_commit();
    if (it + 2 < ntiles) page_next = page_of(kb + (it + 2) * LM_KEYS);
    lm_wait<1>();
    __syncthreads();
    const int tile0 = kb + it * LM_KEYS;
    const bf16* Kt = Ks + (size_t)(it & 1) * LM_KEYS * LD;
    // rows of this warp that see nothing of the tile skip it (the tile lies after them, or before their window)
    const int w_hi = p_first + min(nrows - 1, row0 + warp * 16 + 15) / heads, w_lo_row = p_first + (row0 + warp * 16) / heads;
    const bool useful = warp_live && tile0 <= w_hi && (window == 0 || tile0 + LM_KEYS - 1 > w_lo_row - window);
    if (useful) {
      float s[LM_KEYS / 8][4];
#pragma unroll
      for (int n = 0; n < LM_KEYS / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll(ROTP >= 0 ? (RANK + (ROTP >= 0 ? ROTP : 0)) / 16 : 1)
      for (int kk = 0; kk < KD / 16; ++kk) {
        uint32_t a[4];
        lm_ldm(a, Qs + (size_t)(warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < LM_KEYS / 16; ++np) {
          uint32_t b[4];
          lm_ldm(b, Kt + (size_t)(np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
          lm_mma(s[2 * np], a, b[0], b[1]);
          lm_mma(s[2 * np + 1], a, b[2], b[3]);
        }
      }
      float mxA = -INFINITY, mxB = -INFINITY;
      // a tile that every row of the warp sees whole (no row ends inside it, no window starts inside it, none of its keys
      // belongs to another split or lies beyond the rows) needs no mask
      const bool whole = row0 + warp * 16 + 15 < nrows && tile0 + LM_KEYS - 1 <= min(w_lo_row, ke) && tile0 >= kb &&
                         (window == 0 || tile0 >= w_hi - window + 1);
      if (whole) {
#pragma unroll
        for (int n = 0; n < LM_KEYS / 8; ++n) {
          s[n][0] *= sc; s[n][1] *= sc; s[n][2] *= sc; s[n][3] *= sc;
          mxA = fmaxf(mxA, fmaxf(s[n][0], s[n][1]));
          mxB = fmaxf(mxB, fmaxf(s[n][2], s[n][3]));
        }
      } else {
#pragma unroll
        for (int n = 0; n < LM_KEYS / 8; ++n) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int key = tile0 + n * 8 + (lane & 3) * 2 + (c & 1);
            const bool second = c >= 2;
            const int p = second ? pB : pA, lo = second ? loB : loA;
            const bool see = key <= p && key >= lo && key >= kb && key <= ke;
            const float v = see ? s[n][c] * sc : -INFINITY;
            s[n][c] = v;
            if (second) mxB = fmaxf(mxB, v); else mxA = fmaxf(mxA, v);
          }
        }
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1)); mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1)); mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
      const float baseA = nA == -INFINITY ? 0.f : nA, baseB = nB == -INFINITY ? 0.f : nB;      // a row that has seen nothing yet
      const float cA = exp2f(mA - baseA), cB = exp2f(mB - baseB);
      mA = nA; mB = nB;
      float sumA = 0.f, sumB = 0.f;
#pragma unroll
      for (int n = 0; n < LM_KEYS / 8; ++n) {
        s[n][0] = lm_ex2(s[n][0] - baseA); s[n][1] = lm_ex2(s[n][1] - baseA);
        s[n][2] = lm_ex2(s[n][2] - baseB); s[n][3] = lm_ex2(s[n][3] - baseB);
        sumA += s[n][0] + s[n][1];
        sumB += s[n][2] + s[n][3];
      }
      lA = fmaf(lA, cA, sumA);
      lB = fmaf(lB, cB, sumB);
      if (__any_sync(0xffffffffu, cA != 1.f || cB != 1.f)) {      // else no row's maximum moved: the sums stay as they are
#pragma unroll
        for (int n = 0; n < RANK / 8; ++n) { o[n][0] *= cA; o[n][1] *= cA; o[n][2] *= cB; o[n][3] *= cB; }
      }
#pragma unroll
      for (int ks = 0; ks < LM_KEYS / 16; ++ks) {
        uint32_t a[4] = {lm_pack(s[2 * ks][0], s[2 * ks][1]), lm_pack(s[2 * ks][2], s[2 * ks][3]),
                         lm_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]), lm_pack(s[2 * ks + 1][2], s[2 * ks + 1][3])};
        // terms == 2: a weight is the sum of two bfloat16 numbers (16 bits of its float32 value) and the sum takes two products
        uint32_t a2[4] = {0u, 0u, 0u, 0u};
        if (terms == 2) {
          a2[0] = lm_pack_rest(s[2 * ks][0], s[2 * ks][1]); a2[1] = lm_pack_rest(s[2 * ks][2], s[2 * ks][3]);
          a2[2] = lm_pack_rest(s[2 * ks + 1][0], s[2 * ks + 1][1]); a2[3] = lm_pack_rest(s[2 * ks + 1][2], s[2 * ks + 1][3]);
        }
#pragma unroll
        for (int np = 0; np < RANK / 16; ++np) {
          uint32_t b[4];
          lm_ldm_t(b, Kt + (size_t)(ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + np * 16 + (lane >> 4) * 8);
          lm_mma(o[2 * np], a, b[0], b[1]);
          lm_mma(o[2 * np + 1], a, b[2], b[3]);
          if (terms == 2) {
            lm_mma(o[2 * np], a2, b[0], b[1]);
            lm_mma(o[2 * np + 1], a2, b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();                               // the stage is free for the load after next
  }
  lm_wait<0>();
  lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int rho = half ? rowB : rowA;
    if (rho >= nrows) continue;
    const float l = half ? lB : lA, m = half ? mB : mA;
    if (splits == 1) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = out + ((size_t)(rho % heads) * seg + q0 + rho / heads) * rank;
#pragma unroll
      for (int n = 0; n < RANK / 8; ++n) {
        const int c = n * 8 + (lane & 3) * 2;
        if (c < rank) *reinterpret_cast<uint32_t*>(dst + c) = lm_pack(o[n][2 * half] * inv, o[n][2 * half + 1] * inv);
      }
    } else {
      const int row = rho - row0;
      float* dst = my_part + (size_t)row * RANK;
#pragma unroll
      for (int n = 0; n < RANK / 8; ++n) {
        const int c = n * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(dst + c) = make_float2(o[n][2 * half], o[n][2 * half + 1]);
      }
      if ((lane & 3) == 0) {
        my_part[(size_t)LM_ROWS * RANK + row] = m;
        my_part[(size_t)LM_ROWS * RANK + LM_ROWS + row] = l;
      }
    }
  }
}

// The split form's second step, a block per row: the maximum over the splits (and the sink), every split's weight
// 2^(m_z - m), the denominator, and the weighted sums' quotient.  The first warp forms the weights (at most 32 splits).
template <int RANK>
__global__ void __launch_bounds__(LM_THREADS)
latent_attention_merge_kernel(const float* __restrict__ part, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                              const void* __restrict__ sink, int stype, bf16* __restrict__ out, int seg, int heads, int rank,
                              int splits, int tiles) {
  __shared__ float wz[32];
  __shared__ float inv_l;
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int r = blockIdx.y, rho = blockIdx.x, lane = threadIdx.x & 31;
  const int q0 = cu_q[r], nrows = (cu_q[r + 1] - q0) * heads;
  if (rho >= nrows || seq_lens[r] <= 0) return;
  const int tile = rho / LM_ROWS, row = rho - tile * LM_ROWS, h = rho % heads;
  const size_t PF = lm_part_floats(RANK);
  const float* base = part + (size_t)(r * tiles + tile) * splits * PF;
  if (threadIdx.x < 32) {
    const float s2 = sink != nullptr ? load_as_f32(sink, stype, h) * LM_LOG2E : -INFINITY;
    const float mz = lane < splits ? base[lane * PF + (size_t)LM_ROWS * RANK + row] : -INFINITY;
    const float lz = lane < splits ? base[lane * PF + (size_t)LM_ROWS * RANK + LM_ROWS + row] : 0.f;
    const float m = fmaxf(warp_max(mz), s2);
    const float w = mz == -INFINITY ? 0.f : exp2f(mz - m);
    float l = warp_sum(lz * w);
    if (sink != nullptr) l += exp2f(s2 - m);
    wz[lane] = w;
    if (lane == 0) inv_l = l > 0.f ? 1.f / l : 0.f;
  }
  __syncthreads();
  bf16* dst = out + ((size_t)h * seg + q0 + rho / heads) * rank;
  for (int c = threadIdx.x; c < rank; c += LM_THREADS) {
    float acc = 0.f;
#pragma unroll 8
    for (int z = 0; z < splits; ++z) acc = fmaf(base[z * PF + (size_t)row * RANK + c], wz[z], acc);
    dst[c] = __float2bfloat16(acc * inv_l);
  }
}

static int lm_rank_pad(int rank) { return rank <= 32 ? 32 : rank <= 64 ? 64 : rank <= 128 ? 128 : 256; }

// Floats of scratch that `splits` > 1 needs for a step of `requests` requests of at most `max_q_len` tokens.
IFB_EXPORT long long ifb_latent_attention_mma_scratch_floats(int requests, int max_q_len, int heads, int rank, int splits) {
  if (splits <= 1) return 0;
  const long long tiles = ((long long)max_q_len * heads + LM_ROWS - 1) / LM_ROWS;
  return (long long)requests * tiles * splits * (long long)lm_part_floats(lm_rank_pad(rank));
}

template <int RANK, int ROTP>
static int lm_launch(const float* q_lat, const float* q_rot, int seg, const void* lat_pages, const void* rot_pages, const int* block_tables,
                     int table_stride, int page_size, const int* cu_q, const int* seq_lens, const void* sink, int stype, void* out,
                     float* part, int requests, int max_q_len, int heads, int rank, int rot, float scale, int window, int splits,
                     int terms, cudaStream_t stream) {
  const int rot_pad = (rot + 15) / 16 * 16, LD = RANK + rot_pad + 8;
  const size_t smem = (size_t)(LM_ROWS + 2 * LM_KEYS) * LD * sizeof(bf16);
  if (smem > 220 * 1024) return IFB_ERR_SIZE;
  IFB_ALLOW_SMEM((latent_attention_mma_kernel<RANK, ROTP>), smem);
  const dim3 grid((unsigned)(((long long)max_q_len * heads + LM_ROWS - 1) / LM_ROWS), (unsigned)requests, (unsigned)splits);
  int rc = ifb_launch(latent_attention_mma_kernel<RANK, ROTP>, grid, dim3(LM_THREADS), smem, stream, q_lat, q_rot, seg, (const bf16*)lat_pages,
                      (const bf16*)rot_pages, block_tables, table_stride, page_size, cu_q, seq_lens, sink, stype, (bf16*)out, part, heads,
                      rank, rot, rot_pad, scale, window, splits, terms);
  if (rc != IFB_OK || splits <= 1) return rc;
  return ifb_launch(latent_attention_merge_kernel<RANK>, dim3((unsigned)(max_q_len * heads), grid.y), dim3(LM_THREADS), 0, stream,
                    (const float*)part, cu_q, seq_lens, sink, stype, (bf16*)out, seg, heads, rank, splits, (int)grid.x);
}

// bfloat16 pages and outputs; rank and rot multiples of 8, rank at most 256.
IFB_EXPORT int ifb_latent_attention_mma(const float* q_lat, const float* q_rot, int seg, const void* lat_pages, const void* rot_pages,
                                        const int* block_tables, int table_stride, int page_size, const int* cu_q, const int* seq_lens,
                                        const void* sink, int stype, void* out, float* part, int requests, int max_q_len, int heads,
                                        int rank, int rot, float scale, int window, int splits, int terms, cudaStream_t stream) {
  if (requests <= 0 || max_q_len <= 0) return IFB_OK;
  if (terms != 1 && terms != 2) return IFB_ERR_ARG;
  if (heads < 1 || rank < 8 || rank > 256 || rank % 8 || rot < 0 || rot % 8 || page_size < 1 || window < 0 || splits < 1 || splits > 32 ||
      (splits > 1 && part == nullptr) || (((uintptr_t)q_lat | (uintptr_t)q_rot) & 15))      // queries are read 16 bytes at a time
    return IFB_ERR_SIZE;
#define LM_ARGS                                                                                                                \
  q_lat, q_rot, seg, lat_pages, rot_pages, block_tables, table_stride, page_size, cu_q, seq_lens, sink, stype, out, part, requests, \
      max_q_len, heads, rank, rot, scale, window, splits, terms, stream
  // the usual widths of a rotated part have kernels of their own; any other width runs the one that reads it at run time
#define LM_CASE(P)                                            \
  switch ((rot + 15) / 16 * 16) {                             \
    case 0: return lm_launch<P, 0>(LM_ARGS);                  \
    case 16: return lm_launch<P, 16>(LM_ARGS);                \
    case 32: return lm_launch<P, 32>(LM_ARGS);                \
    case 64: return lm_launch<P, 64>(LM_ARGS);                \
    default: return lm_launch<P, -1>(LM_ARGS);                \
  }
  switch (lm_rank_pad(rank)) {
    case 32: return lm_launch<32, -1>(LM_ARGS);
    case 64: LM_CASE(64);
    case 128: LM_CASE(128);
    default: LM_CASE(256);
  }
#undef LM_CASE
#undef LM_ARGS
}
