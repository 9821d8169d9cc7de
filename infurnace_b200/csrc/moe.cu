// A mixture of experts on the device, with no step that the host has to wait for: the router's choice, the list of
// (token, choice) pairs by expert, the experts' products as grouped launches over that list, and the weighted sum.
// Router arithmetic, the softmax over the chosen logits and the final sum are float32; the grouped product
// multiplies in float32 whatever the storage (each output element is one thread's sum over k in ascending order, so
// a row's result does not depend on which other rows share its tile).  These kernels take every size.
#include "common.cuh"
#include <math.h>

// ------------------------------------------------------------------------------------------
// ids[n][j], j < top: the indices of row n's `top` largest scores, largest first, the lower index among equals.
// mode 0: the scores are the logits, and gates[n][j] is the softmax over the chosen logits only.  mode 1: the scores are
// the softmax over all experts, only experts of the `keep` groups (of `groups` equal groups of neighbours) whose best score
// is largest can be chosen, and gates[n][j] = score * wscale, not renormalised.  mode 2: the scores are sigmoid(logit) per
// expert (the order of the logits is the order of the scores), gates[n][j] = score * wscale.  A row of logits has `stride` entries, of
// which the first `experts` are the router's.  A warp per row; a lane holds the logits e = lane, lane + 32, ... (up to
// MR_PER_LANE * 32 experts); lane j keeps the j-th chosen score (up to 32 choices).
// ------------------------------------------------------------------------------------------
constexpr int MR_PER_LANE = 8;
struct MrMode { int stride, mode, groups, keep; float wscale; };
__device__ __forceinline__ void mr_route_row(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ gates,
                                             int row, int experts, int top, int lane, MrMode md) {
  float val[MR_PER_LANE];
#pragma unroll
  for (int j = 0; j < MR_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    val[j] = e < experts ? logits[(size_t)row * md.stride + e] : -INFINITY;
    if (val[j] != val[j]) val[j] = -INFINITY;          // a NaN is never chosen before a number
  }
  if (md.mode == 1) {
    float mx = -INFINITY, tot = 0.f;
#pragma unroll
    for (int j = 0; j < MR_PER_LANE; ++j) mx = fmaxf(mx, val[j]);
    mx = warp_max(mx);
#pragma unroll
    for (int j = 0; j < MR_PER_LANE; ++j) { val[j] = lane + 32 * j < experts ? expf(val[j] - mx) : 0.f; tot += val[j]; }
    tot = warp_sum(tot);
#pragma unroll
    for (int j = 0; j < MR_PER_LANE; ++j) val[j] = lane + 32 * j < experts ? val[j] / tot : -INFINITY;
    if (md.groups > 1 && md.keep < md.groups) {
      const int gsz = experts / md.groups;
      float gbest[MR_PER_LANE];                         // lane holds the best score of groups lane, lane + 32, ...
#pragma unroll
      for (int j = 0; j < MR_PER_LANE; ++j) gbest[j] = -INFINITY;
      for (int g = 0; g < md.groups; ++g) {
        float b = -INFINITY;
#pragma unroll
        for (int j = 0; j < MR_PER_LANE; ++j) { const int e = lane + 32 * j; if (e < experts && e / gsz == g) b = fmaxf(b, val[j]); }
        b = warp_max(b);
#pragma unroll
        for (int j = 0; j < MR_PER_LANE; ++j) if ((g & 31) == lane && (g >> 5) == j) gbest[j] = b;
      }
      unsigned kept = 0;                                // bit j: this lane's j-th group is kept
      for (int t = 0; t < md.keep; ++t) {
        float best = -INFINITY;
        int best_g = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < MR_PER_LANE; ++j) {
          const int g = lane + 32 * j;
          if (g < md.groups && !((kept >> j) & 1u) && (gbest[j] > best || (gbest[j] == best && g < best_g))) { best = gbest[j]; best_g = g; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
          if (ob > best || (ob == best && og < best_g)) { best = ob; best_g = og; }
        }
        if ((best_g & 31) == lane && best_g < md.groups) kept |= 1u << (best_g >> 5);
      }
#pragma unroll
      for (int j = 0; j < MR_PER_LANE; ++j) {
        const int e = lane + 32 * j, g = e < experts ? e / gsz : 0;
        const unsigned bits = __shfl_sync(0xffffffffu, kept, g & 31);
        if (e < experts && !((bits >> (g >> 5)) & 1u)) val[j] = -INFINITY;
      }
    }
  }
  unsigned taken = 0;                                   // bit j: this lane's j-th logit is chosen already
  float first = 0.f, mine = -INFINITY, sum = 0.f;       // lane j < top keeps the j-th chosen logit
  for (int t = 0; t < top; ++t) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MR_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < experts && !((taken >> j) & 1u) && (val[j] > best || (val[j] == best && e < best_e))) { best = val[j]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if ((best_e & 31) == lane && best_e < experts) taken |= 1u << (best_e >> 5);
    if (t == 0) first = best;
    if (lane == t) mine = best;
    if (lane == 0) ids[(size_t)row * top + t] = best_e < experts ? best_e : 0;
  }
  if (md.mode == 1) {
    if (lane < top) gates[(size_t)row * top + lane] = mine * md.wscale;
    return;
  }
  if (md.mode == 2) {
    if (lane < top) gates[(size_t)row * top + lane] = md.wscale / (1.f + expf(-mine));
    return;
  }
  const float p = lane < top ? expf(mine - first) : 0.f;
  sum = warp_sum(p);
  if (lane < top) gates[(size_t)row * top + lane] = p / sum;
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ gates, int rows, int experts,
                 int top, MrMode md) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  mr_route_row(logits, ids, gates, row, experts, top, lane, md);
}

// The router and the pair list of a step of few rows (decode) in one launch: one block routes the rows, a warp each in
// turn, then a thread per expert counts its pairs, finds its offset and lists them in ascending pair number.
constexpr int MS_THREADS = 256;
__global__ void __launch_bounds__(MS_THREADS)
moe_route_plan_small_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ gates, int rows, int experts,
                            int top, int* __restrict__ offsets, int* __restrict__ perm, int* __restrict__ pos, MrMode md) {
  __shared__ int cnt[MS_THREADS];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = warp; row < rows; row += MS_THREADS / 32) mr_route_row(logits, ids, gates, row, experts, top, lane, md);
  __syncthreads();                                 // the block's own writes of ids are visible to it
  const int e = threadIdx.x, pairs = rows * top;
  int mine = 0;
  if (e < experts)
    for (int i = 0; i < pairs; ++i) mine += ids[i] == e ? 1 : 0;
  cnt[threadIdx.x] = mine;
  __syncthreads();
  if (e >= experts) return;
  int place = 0;
  for (int j = 0; j < e; ++j) place += cnt[j];
  offsets[e] = place;
  if (e == experts - 1) offsets[experts] = place + mine;
  for (int i = 0; i < pairs && mine > 0; ++i)
    if (ids[i] == e) { perm[place] = i; pos[i] = place; ++place; }
}

static bool mr_mode_ok(const MrMode& md, int experts) {
  return md.stride >= experts && md.mode >= 0 && md.mode <= 2 && md.groups >= 1 && md.keep >= 1 && md.keep <= md.groups &&
         experts % md.groups == 0;
}

IFB_EXPORT int ifb_moe_route_plan_small(const float* logits, int* ids, float* gates, int rows, int experts, int top, int* offsets,
                                        int* perm, int* pos, int stride, int mode, int groups, int keep, float wscale,
                                        cudaStream_t stream) {
  if (rows <= 0) return IFB_OK;
  if (experts < 1 || experts > MS_THREADS || top < 1 || top > experts || top > 32 || (long long)rows * top > 4096) return IFB_ERR_SIZE;
  const MrMode md{stride, mode, groups, keep, wscale};
  if (!mr_mode_ok(md, experts)) return IFB_ERR_ARG;
  return ifb_launch(moe_route_plan_small_kernel, dim3(1), dim3(MS_THREADS), 0, stream, logits, ids, gates, rows, experts, top,
                    offsets, perm, pos, md);
}

IFB_EXPORT int ifb_moe_route(const float* logits, int* ids, float* gates, int rows, int experts, int top, int stride, int mode,
                             int groups, int keep, float wscale, cudaStream_t stream) {
  if (rows <= 0) return IFB_OK;
  if (experts < 1 || experts > 32 * MR_PER_LANE || top < 1 || top > experts || top > 32) return IFB_ERR_SIZE;
  const MrMode md{stride, mode, groups, keep, wscale};
  if (!mr_mode_ok(md, experts)) return IFB_ERR_ARG;
  return ifb_launch(moe_route_kernel, dim3((rows + 3) / 4), dim3(128), 0, stream, logits, ids, gates, rows, experts, top, md);
}

// ------------------------------------------------------------------------------------------
// The pairs (row, choice), numbered row * top + choice, listed by expert in ascending pair number: expert e's places
// in `perm` are offsets[e] .. offsets[e + 1]; pos[pair] is the pair's place.  A block per expert: it counts the pairs
// of lower experts (its offset), then walks the pairs in order, a block-wide prefix sum placing its own.
// ------------------------------------------------------------------------------------------
constexpr int MP_THREADS = 256;
__global__ void __launch_bounds__(MP_THREADS)
moe_plan_kernel(const int* __restrict__ ids, int pairs, int experts, int* __restrict__ offsets, int* __restrict__ perm,
                int* __restrict__ pos) {
  __shared__ int warp_tot[MP_THREADS / 32];
  __shared__ int lower_s;
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int lower = 0;
  for (int i = threadIdx.x; i < pairs; i += MP_THREADS) { const int id = ids[i]; lower += (id >= 0 && id < e) ? 1 : 0; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lower += __shfl_xor_sync(0xffffffffu, lower, o);
  if (lane == 0) warp_tot[warp] = lower;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < MP_THREADS / 32; ++w) s += warp_tot[w];
    lower_s = s;
  }
  __syncthreads();
  int base = lower_s;
  if (threadIdx.x == 0) offsets[e] = base;
  for (int i0 = 0; i0 < pairs; i0 += MP_THREADS) {
    const int i = i0 + threadIdx.x;
    const bool hit = i < pairs && ids[i] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    __syncthreads();                                 // the totals of the round before have been read
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < MP_THREADS / 32; ++w) { const int c = warp_tot[w]; if (w < warp) before += c; total += c; }
    if (hit) {
      const int place = base + before + __popc(ballot & ((1u << lane) - 1u));
      perm[place] = i;
      pos[i] = place;
    }
    base += total;
  }
  if (e == experts - 1 && threadIdx.x == 0) offsets[experts] = base;
}

IFB_EXPORT int ifb_moe_plan(const int* ids, int pairs, int experts, int* offsets, int* perm, int* pos, cudaStream_t stream) {
  if (experts < 1) return IFB_ERR_SIZE;
  if (pairs < 0) return IFB_ERR_ARG;
  return ifb_launch(moe_plan_kernel, dim3(experts), dim3(MP_THREADS), 0, stream, ids, pairs, experts, offsets, perm, pos);
}

// ------------------------------------------------------------------------------------------
// The pair list with every expert's segment padded to a multiple of `pad` places (the row tile of the tcgen05 grouped
// product, which needs an expert's rows contiguous and tiles that do not straddle experts): offsets[e] is the segment's
// padded start, perm[place] = -1 in the padding, tile_expert[t] the expert of tile t of `pad` places, -1 for the tiles
// after the last segment (tiles_total of them exist).  A block per expert; each counts all experts' pairs itself.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(MP_THREADS)
moe_plan_padded_kernel(const int* __restrict__ ids, int pairs, int experts, int pad, int* __restrict__ offsets,
                       int* __restrict__ perm, int* __restrict__ pos, int* __restrict__ tile_expert, int tiles_total) {
  __shared__ int hist[256];
  __shared__ int warp_tot[MP_THREADS / 32];
  __shared__ int seg[3];                 // start, count, padded count of this block's expert
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 256; i += MP_THREADS) hist[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += MP_THREADS) { const int id = ids[i]; if (id >= 0 && id < experts) atomicAdd(&hist[id], 1); }
  __syncthreads();
  if (threadIdx.x == 0) {
    int start = 0;
    for (int j = 0; j < e; ++j) start += (hist[j] + pad - 1) / pad * pad;
    seg[0] = start; seg[1] = hist[e]; seg[2] = (hist[e] + pad - 1) / pad * pad;
    offsets[e] = start;
    if (e == experts - 1) offsets[experts] = start + seg[2];
  }
  __syncthreads();
  const int start = seg[0], count = seg[1], padded = seg[2];
  for (int i = start + count + threadIdx.x; i < start + padded; i += MP_THREADS) perm[i] = -1;
  for (int t = start / pad + threadIdx.x; t < (start + padded) / pad; t += MP_THREADS) tile_expert[t] = e;
  if (e == experts - 1)
    for (int t = (start + padded) / pad + threadIdx.x; t < tiles_total; t += MP_THREADS) tile_expert[t] = -1;
  int base = start;
  for (int i0 = 0; i0 < pairs; i0 += MP_THREADS) {
    const int i = i0 + threadIdx.x;
    const bool hit = i < pairs && ids[i] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    __syncthreads();
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < MP_THREADS / 32; ++w) { const int c = warp_tot[w]; if (w < warp) before += c; total += c; }
    if (hit) {
      const int place = base + before + __popc(ballot & ((1u << lane) - 1u));
      perm[place] = i;
      pos[i] = place;
    }
    base += total;
  }
}

IFB_EXPORT int ifb_moe_plan_padded(const int* ids, int pairs, int experts, int pad, int* offsets, int* perm, int* pos,
                                   int* tile_expert, int tiles_total, cudaStream_t stream) {
  if (experts < 1 || experts > 256 || pad < 1) return IFB_ERR_SIZE;
  if (pairs < 0 || (long long)tiles_total * pad < (long long)pairs + (long long)experts * (pad - 1)) return IFB_ERR_ARG;
  return ifb_launch(moe_plan_padded_kernel, dim3(experts), dim3(MP_THREADS), 0, stream, ids, pairs, experts, pad, offsets, perm, pos,
                    tile_expert, tiles_total);
}

// out[place][:] = x[perm[place] / top][:], zeros where perm[place] < 0; places of unused tiles are left alone.
// bfloat16 rows of k elements, k a multiple of 8; a block per place.
__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ perm, int top, const int* __restrict__ tile_expert,
                       int pad, uint4* __restrict__ out, int k8) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int place = blockIdx.x;
  if (tile_expert[place / pad] < 0) return;
  const int p = perm[place];
  uint4* dst = out + (size_t)place * k8;
  if (p < 0) {
    for (int i = threadIdx.x; i < k8; i += blockDim.x) dst[i] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const uint4* src = x + (size_t)(p / top) * k8;
  for (int i = threadIdx.x; i < k8; i += blockDim.x) dst[i] = src[i];
}

IFB_EXPORT int ifb_moe_gather_rows(const void* x, const int* perm, int top, const int* tile_expert, int pad, void* out, int places,
                                   int k, cudaStream_t stream) {
  if (places <= 0) return IFB_OK;
  if (k < 8 || k % 8 || top < 1 || pad < 1) return IFB_ERR_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)out & 15)) return IFB_ERR_ALIGN;
  return ifb_launch(moe_gather_rows_kernel, dim3(places), dim3(128), 0, stream, (const uint4*)x, perm, top, tile_expert, pad,
                    (uint4*)out, k / 8);
}

// out[place][:] = gates[perm[place]] * x[perm[place] / top][:] in out's dtype (the product in float32, rounded once): what an
// expert reads when its weight multiplies its input.  Zeros where perm[place] < 0; with tile_expert, places of unused tiles
// are left alone.  Any dtype and width; bfloat16 rows of a multiple of 8 elements go 16 bytes at a time.
template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_scaled_kernel(const T* __restrict__ x, const int* __restrict__ perm, int top, const float* __restrict__ gates,
                         const int* __restrict__ tile_expert, int pad, T* __restrict__ out, int k, int vec) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int place = blockIdx.x;
  if (tile_expert != nullptr && tile_expert[place / pad] < 0) return;
  const int p = perm[place];
  T* dst = out + (size_t)place * k;
  if (p < 0) {
    for (int i = threadIdx.x; i < k; i += blockDim.x) dst[i] = from_f32<T>(0.f);
    return;
  }
  const float g = gates[p];
  const T* src = x + (size_t)(p / top) * k;
  if constexpr (sizeof(T) == 2) {
    if (vec) {
      for (int i = threadIdx.x * 8; i < k; i += blockDim.x * 8) {
        uint4 raw = *reinterpret_cast<const uint4*>(src + i);
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
          h2[j] = __floats2bfloat162_rn(f.x * g, f.y * g);
        }
        *reinterpret_cast<uint4*>(dst + i) = raw;
      }
      return;
    }
  }
  for (int i = threadIdx.x; i < k; i += blockDim.x) dst[i] = from_f32<T>(to_f32<T>(src[i]) * g);
}

IFB_EXPORT int ifb_moe_gather_scaled(const void* x, int dtype, const int* perm, int top, const float* gates, const int* tile_expert,
                                     int pad, void* out, int places, int k, cudaStream_t stream) {
  if (places <= 0) return IFB_OK;
  if (k < 1 || top < 1 || pad < 1) return IFB_ERR_SIZE;
  const int vec = k % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0;
  if (dtype == IFB_BF16)
    return ifb_launch(moe_gather_scaled_kernel<__nv_bfloat16>, dim3(places), dim3(128), 0, stream, (const __nv_bfloat16*)x, perm, top,
                      gates, tile_expert, pad, (__nv_bfloat16*)out, k, vec);
  if (dtype != IFB_F32) return IFB_ERR_DTYPE;
  return ifb_launch(moe_gather_scaled_kernel<float>, dim3(places), dim3(128), 0, stream, (const float*)x, perm, top, gates,
                    tile_expert, pad, (float*)out, k, 0);
}

// ------------------------------------------------------------------------------------------
// The grouped product.  Row i of `out` belongs to the expert e with offsets[e] <= i < offsets[e + 1] and is
//     x[src(i)] w[e]^T,   src(i) = perm[i] / top (perm null: i),   w [experts][o_w][k]
// GATED: w[e] holds o gate rows and then o up rows, and out[i][j] = silu(gate_j) * up_j.  A block is a tile of ML_ROWS
// rows of one expert by ML_COLS outputs; block row y is the y-th tile in the order of the experts (each expert's rows
// are tiled on their own; block rows beyond the last tile return).  A thread owns 2 rows x 4 outputs.
// ------------------------------------------------------------------------------------------
constexpr int ML_ROWS = 32, ML_COLS = 64, ML_K = 32, ML_THREADS = 256;
template <typename TA, typename TW, typename TO, bool GATED>
__global__ void __launch_bounds__(ML_THREADS)
moe_linear_kernel(const TA* __restrict__ x, const TW* __restrict__ w, const int* __restrict__ offsets,
                  const int* __restrict__ perm, int top, TO* __restrict__ out, int experts, int o, int k) {
  __shared__ float As[ML_ROWS][ML_K + 1];
  __shared__ float Ws[(GATED ? 2 : 1) * ML_COLS][ML_K + 1];
  __shared__ int src[ML_ROWS];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  int e = 0, row0 = 0, row1 = 0, tile = blockIdx.y;
  bool found = false;
  for (; e < experts; ++e) {
    const int a = offsets[e], b = offsets[e + 1];
    const int tiles = (b - a + ML_ROWS - 1) / ML_ROWS;
    if (tile < tiles) { row0 = a + tile * ML_ROWS; row1 = min(b, row0 + ML_ROWS); found = true; break; }
    tile -= tiles;
  }
  if (!found) return;
  const int col0 = blockIdx.x * ML_COLS;
  const int o_w = GATED ? 2 * o : o;
  const TW* we = w + (size_t)e * o_w * k;
  if (threadIdx.x < ML_ROWS) {
    const int i = row0 + threadIdx.x;
    src[threadIdx.x] = i < row1 ? (perm ? perm[i] / top : i) : -1;
  }
  __syncthreads();
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;       // rows 2 ty, 2 ty + 1; outputs 4 tx .. 4 tx + 3
  float acc[2][4] = {}, up[2][4] = {};
  for (int k0 = 0; k0 < k; k0 += ML_K) {
    for (int idx = threadIdx.x; idx < ML_ROWS * ML_K; idx += ML_THREADS) {
      const int r = idx / ML_K, kk = idx % ML_K;
      const int s = src[r];
      As[r][kk] = (s >= 0 && k0 + kk < k) ? to_f32<TA>(x[(size_t)s * k + k0 + kk]) : 0.f;
    }
    for (int idx = threadIdx.x; idx < (GATED ? 2 : 1) * ML_COLS * ML_K; idx += ML_THREADS) {
      const int c = idx / ML_K, kk = idx % ML_K;
      const int half = c / ML_COLS, cc = c % ML_COLS;
      const int feat = col0 + cc;
      Ws[c][kk] = (feat < o && k0 + kk < k) ? to_f32<TW>(we[((size_t)half * o + feat) * k + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < ML_K; ++kk) {
      const float a0 = As[2 * ty][kk], a1 = As[2 * ty + 1][kk];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float wv = Ws[4 * tx + j][kk];
        acc[0][j] = fmaf(a0, wv, acc[0][j]);
        acc[1][j] = fmaf(a1, wv, acc[1][j]);
        if (GATED) {
          const float uv = Ws[ML_COLS + 4 * tx + j][kk];
          up[0][j] = fmaf(a0, uv, up[0][j]);
          up[1][j] = fmaf(a1, uv, up[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + 2 * ty + i;
    if (row >= row1) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int feat = col0 + 4 * tx + j;
      if (feat >= o) continue;
      float y = acc[i][j];
      if (GATED) y = y / (1.f + expf(-y)) * up[i][j];
      out[(size_t)row * o + feat] = from_f32<TO>(y);
    }
  }
}

// ------------------------------------------------------------------------------------------
// The grouped product on tensor cores (bfloat16 operands, float32 accumulation): mma.sync m16n8k16.  A CTA of four
// warps is a tile of MM_ROWS rows of one expert by MM_COLS outputs (GATED: the gate and the up column of each output,
// so that the activation is the epilogue); warp w owns rows 32 w .. 32 w + 31 of the tile, so that a weight fragment
// read from shared memory serves two blocks of rows.  The k range is walked in steps of MM_K through three stages of
// shared memory filled by 16-byte asynchronous copies (rows gathered through the pair list; rows and columns beyond
// the tile, and k beyond the end, are filled with zeros), fragments come out of shared memory by ldmatrix from rows
// padded to 80 bytes (no bank conflicts).  A row's result depends on its own
// operands only, whatever else shares its tile.  k must be a multiple of 8.
// ------------------------------------------------------------------------------------------
constexpr int MM_ROWS = 128, MM_COLS = 64, MM_K = 32, MM_PAD = 8, MM_THREADS = 128, MM_STAGES = 3;
constexpr int MM_LD = MM_K + MM_PAD;

__device__ __forceinline__ void mm_cp16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void mm_ldmatrix4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mm_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool GATED> constexpr size_t mm_smem_bytes() {
  return (size_t)MM_STAGES * (MM_ROWS + (GATED ? 2 : 1) * MM_COLS) * MM_LD * sizeof(__nv_bfloat16) + MM_ROWS * sizeof(int);
}

template <typename TO, bool GATED>
__global__ void __launch_bounds__(MM_THREADS)
moe_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const int* __restrict__ offsets,
                      const int* __restrict__ perm, int top, TO* __restrict__ out, int experts, int o, int k) {
  constexpr int WR = (GATED ? 2 : 1) * MM_COLS;              // weight rows of a tile
  extern __shared__ __align__(16) unsigned char mm_raw[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(mm_raw);                  // [STAGES][MM_ROWS][MM_LD]
  __nv_bfloat16* Ws = As + (size_t)MM_STAGES * MM_ROWS * MM_LD;                  // [STAGES][WR][MM_LD]
  int* src = reinterpret_cast<int*>(Ws + (size_t)MM_STAGES * WR * MM_LD);        // [MM_ROWS]
  ifb_pdl_wait();
  ifb_pdl_trigger();
  int e = 0, row0 = 0, row1 = 0, tile = blockIdx.y;
  bool found = false;
  for (; e < experts; ++e) {
    const int a = offsets[e], b = offsets[e + 1];
    const int tiles = (b - a + MM_ROWS - 1) / MM_ROWS;
    if (tile < tiles) { row0 = a + tile * MM_ROWS; row1 = min(b, row0 + MM_ROWS); found = true; break; }
    tile -= tiles;
  }
  if (!found) return;
  const int col0 = blockIdx.x * MM_COLS;
  const int o_w = GATED ? 2 * o : o;
  const __nv_bfloat16* we = w + (size_t)e * o_w * k;
  for (int r = threadIdx.x; r < MM_ROWS; r += MM_THREADS) {
    const int i = row0 + r;
    src[r] = i < row1 ? (perm ? perm[i] / top : i) : -1;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // warp w owns rows 32 w .. 32 w + 31 of the tile, as two blocks of 16; a block beyond the expert's rows is not multiplied
  const bool live0 = row0 + 32 * warp < row1, live1 = row0 + 32 * warp + 16 < row1;
  auto fill = [&](int stage, int k0) {
    __nv_bfloat16* A = As + (size_t)stage * MM_ROWS * MM_LD;
    __nv_bfloat16* W = Ws + (size_t)stage * WR * MM_LD;
    for (int idx = threadIdx.x; idx < MM_ROWS * (MM_K / 8); idx += MM_THREADS) {
      const int r = idx / (MM_K / 8), c = (idx % (MM_K / 8)) * 8;
      const int s = src[r];
      const bool ok = s >= 0 && k0 + c < k;
      mm_cp16(A + r * MM_LD + c, ok ? x + (size_t)s * k + k0 + c : x, ok);
    }
    for (int idx = threadIdx.x; idx < WR * (MM_K / 8); idx += MM_THREADS) {
      const int r = idx / (MM_K / 8), c = (idx % (MM_K / 8)) * 8;
      const int half = r / MM_COLS, feat = col0 + r % MM_COLS;
      const bool ok = feat < o && k0 + c < k;
      mm_cp16(W + r * MM_LD + c, ok ? we + ((size_t)half * o + feat) * k + k0 + c : we, ok);
    }
  };
  float acc[2][MM_COLS / 8][4] = {}, up[GATED ? 2 : 1][GATED ? MM_COLS / 8 : 1][4] = {};
  const int steps = (k + MM_K - 1) / MM_K;
  for (int p = 0; p < MM_STAGES - 1; ++p) {
    if (p < steps) fill(p, p * MM_K);
    asm volatile("cp.async.commit_group;\n" ::);
  }
  for (int st = 0; st < steps; ++st) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(MM_STAGES - 2));      // stage st has landed
    __syncthreads();                                                       // ... for everyone, and everyone is done with stage st - 1
    if (st + MM_STAGES - 1 < steps) fill((st + MM_STAGES - 1) % MM_STAGES, (st + MM_STAGES - 1) * MM_K);
    asm volatile("cp.async.commit_group;\n" ::);
    if (!live0) continue;
    const __nv_bfloat16* A = As + (size_t)(st % MM_STAGES) * MM_ROWS * MM_LD;
    const __nv_bfloat16* W = Ws + (size_t)(st % MM_STAGES) * WR * MM_LD;
#pragma unroll
    for (int kk = 0; kk < MM_K; kk += 16) {
      unsigned a0[4], a1[4] = {0u, 0u, 0u, 0u};
      mm_ldmatrix4(a0[0], a0[1], a0[2], a0[3], A + (32 * warp + (lane & 15)) * MM_LD + kk + (lane >> 4) * 8);
      if (live1) mm_ldmatrix4(a1[0], a1[1], a1[2], a1[3], A + (32 * warp + 16 + (lane & 15)) * MM_LD + kk + (lane >> 4) * 8);
#pragma unroll
      for (int nt = 0; nt < MM_COLS / 8; nt += 2) {
        unsigned b0, b1, b2, b3;
        const int brow = nt * 8 + (lane & 7) + (lane >> 4) * 8, bcol = kk + ((lane >> 3) & 1) * 8;
        mm_ldmatrix4(b0, b1, b2, b3, W + brow * MM_LD + bcol);
        mm_mma(acc[0][nt], a0, b0, b1);
        mm_mma(acc[0][nt + 1], a0, b2, b3);
        if (live1) { mm_mma(acc[1][nt], a1, b0, b1); mm_mma(acc[1][nt + 1], a1, b2, b3); }
        if (GATED) {
          mm_ldmatrix4(b0, b1, b2, b3, W + (MM_COLS + brow) * MM_LD + bcol);
          mm_mma(up[0][nt], a0, b0, b1);
          mm_mma(up[0][nt + 1], a0, b2, b3);
          if (live1) { mm_mma(up[GATED ? 1 : 0][nt], a1, b0, b1); mm_mma(up[GATED ? 1 : 0][nt + 1], a1, b2, b3); }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  if (!live0) return;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
    for (int nt = 0; nt < MM_COLS / 8; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = row0 + 32 * warp + 16 * blk + g + (i >> 1) * 8, feat = col0 + nt * 8 + 2 * t + (i & 1);
        if (row >= row1 || feat >= o) continue;
        float y = acc[blk][nt][i];
        if (GATED) y = y / (1.f + expf(-y)) * up[GATED ? blk : 0][GATED ? nt : 0][i];
        out[(size_t)row * o + feat] = from_f32<TO>(y);
      }
    }
  }
}

// The same product for steps of few rows (decode): tiles of SK_ROWS rows, so that the step is the experts' weights
// streamed once; the four warps of a CTA split the tile's 64 outputs, the k range goes through four stages of 128, which
// keeps about a hundred kilobytes of weights in flight per CTA (a CTA of the wide form waits on 16 KB at a time).
constexpr int MM_SKINNY_MAX_ROWS = 256;      // rows of a step up to which the few-rows form runs
constexpr int SK_ROWS = 16, SK_COLS = 64, SK_K = 128, SK_STAGES = 4, SK_LD = SK_K + 8, SK_THREADS = 128;

template <bool GATED> constexpr size_t sk_smem_bytes() {
  return (size_t)SK_STAGES * (SK_ROWS + (GATED ? 2 : 1) * SK_COLS) * SK_LD * sizeof(__nv_bfloat16) + SK_ROWS * sizeof(int);
}

template <typename TO, bool GATED>
__global__ void __launch_bounds__(SK_THREADS)
moe_linear_mma_skinny_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const int* __restrict__ offsets,
                             const int* __restrict__ perm, int top, TO* __restrict__ out, int experts, int o, int k) {
  constexpr int WR = (GATED ? 2 : 1) * SK_COLS;
  extern __shared__ __align__(16) unsigned char mm_raw[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(mm_raw);                  // [STAGES][SK_ROWS][SK_LD]
  __nv_bfloat16* Ws = As + (size_t)SK_STAGES * SK_ROWS * SK_LD;                  // [STAGES][WR][SK_LD]
  int* src = reinterpret_cast<int*>(Ws + (size_t)SK_STAGES * WR * SK_LD);        // [SK_ROWS]
  ifb_pdl_wait();
  ifb_pdl_trigger();
  int e = 0, row0 = 0, row1 = 0, tile = blockIdx.y;
  bool found = false;
  for (; e < experts; ++e) {
    const int a = offsets[e], b = offsets[e + 1];
    const int tiles = (b - a + SK_ROWS - 1) / SK_ROWS;
    if (tile < tiles) { row0 = a + tile * SK_ROWS; row1 = min(b, row0 + SK_ROWS); found = true; break; }
    tile -= tiles;
  }
  if (!found) return;
  const int col0 = blockIdx.x * SK_COLS;
  const int o_w = GATED ? 2 * o : o;
  const __nv_bfloat16* we = w + (size_t)e * o_w * k;
  if (threadIdx.x < SK_ROWS) {
    const int i = row0 + threadIdx.x;
    src[threadIdx.x] = i < row1 ? (perm ? perm[i] / top : i) : -1;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto fill = [&](int stage, int k0) {
    __nv_bfloat16* A = As + (size_t)stage * SK_ROWS * SK_LD;
    __nv_bfloat16* W = Ws + (size_t)stage * WR * SK_LD;
    for (int idx = threadIdx.x; idx < SK_ROWS * (SK_K / 8); idx += SK_THREADS) {
      const int r = idx / (SK_K / 8), c = (idx % (SK_K / 8)) * 8;
      const int s = src[r];
      const bool ok = s >= 0 && k0 + c < k;
      mm_cp16(A + r * SK_LD + c, ok ? x + (size_t)s * k + k0 + c : x, ok);
    }
    for (int idx = threadIdx.x; idx < WR * (SK_K / 8); idx += SK_THREADS) {
      const int r = idx / (SK_K / 8), c = (idx % (SK_K / 8)) * 8;
      const int half = r / SK_COLS, feat = col0 + r % SK_COLS;
      const bool ok = feat < o && k0 + c < k;
      mm_cp16(W + r * SK_LD + c, ok ? we + ((size_t)half * o + feat) * k + k0 + c : we, ok);
    }
  };
  float acc[2][4] = {}, up[2][4] = {};
  const int steps = (k + SK_K - 1) / SK_K;
  for (int p = 0; p < SK_STAGES - 1; ++p) {
    if (p < steps) fill(p, p * SK_K);
    asm volatile("cp.async.commit_group;\n" ::);
  }
  for (int st = 0; st < steps; ++st) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(SK_STAGES - 2));
    __syncthreads();
    if (st + SK_STAGES - 1 < steps) fill((st + SK_STAGES - 1) % SK_STAGES, (st + SK_STAGES - 1) * SK_K);
    asm volatile("cp.async.commit_group;\n" ::);
    const __nv_bfloat16* A = As + (size_t)(st % SK_STAGES) * SK_ROWS * SK_LD;
    const __nv_bfloat16* W = Ws + (size_t)(st % SK_STAGES) * WR * SK_LD;
#pragma unroll
    for (int kk = 0; kk < SK_K; kk += 16) {
      unsigned a[4], b0, b1, b2, b3;
      mm_ldmatrix4(a[0], a[1], a[2], a[3], A + (lane & 15) * SK_LD + kk + (lane >> 4) * 8);
      const int brow = 16 * warp + (lane & 7) + (lane >> 4) * 8, bcol = kk + ((lane >> 3) & 1) * 8;
      mm_ldmatrix4(b0, b1, b2, b3, W + brow * SK_LD + bcol);
      mm_mma(acc[0], a, b0, b1);
      mm_mma(acc[1], a, b2, b3);
      if (GATED) {
        mm_ldmatrix4(b0, b1, b2, b3, W + (SK_COLS + brow) * SK_LD + bcol);
        mm_mma(up[0], a, b0, b1);
        mm_mma(up[1], a, b2, b3);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = row0 + g + (i >> 1) * 8, feat = col0 + 16 * warp + nt * 8 + 2 * t + (i & 1);
      if (row >= row1 || feat >= o) continue;
      float y = acc[nt][i];
      if (GATED) y = y / (1.f + expf(-y)) * up[nt][i];
      out[(size_t)row * o + feat] = from_f32<TO>(y);
    }
  }
}

template <typename TO>
static int sk_launch(const void* x, const void* w, const int* offsets, const int* perm, int top, void* out, int rows, int experts,
                     int o, int k, int gated, cudaStream_t s) {
  dim3 grid((o + SK_COLS - 1) / SK_COLS, (rows + SK_ROWS - 1) / SK_ROWS + experts);
  if (gated) {
    IFB_ALLOW_SMEM((moe_linear_mma_skinny_kernel<TO, true>), sk_smem_bytes<true>());
    return ifb_launch(moe_linear_mma_skinny_kernel<TO, true>, grid, dim3(SK_THREADS), sk_smem_bytes<true>(), s,
                      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, offsets, perm, top, (TO*)out, experts, o, k);
  }
  IFB_ALLOW_SMEM((moe_linear_mma_skinny_kernel<TO, false>), sk_smem_bytes<false>());
  return ifb_launch(moe_linear_mma_skinny_kernel<TO, false>, grid, dim3(SK_THREADS), sk_smem_bytes<false>(), s,
                    (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, offsets, perm, top, (TO*)out, experts, o, k);
}

template <typename TO>
static int mm_launch(const void* x, const void* w, const int* offsets, const int* perm, int top, void* out, int rows, int experts,
                     int o, int k, int gated, cudaStream_t s) {
  dim3 grid((o + MM_COLS - 1) / MM_COLS, (rows + MM_ROWS - 1) / MM_ROWS + experts);
  if (grid.y > 65535) return IFB_ERR_SIZE;
  if (gated) {
    IFB_ALLOW_SMEM((moe_linear_mma_kernel<TO, true>), mm_smem_bytes<true>());
    return ifb_launch(moe_linear_mma_kernel<TO, true>, grid, dim3(MM_THREADS), mm_smem_bytes<true>(), s, (const __nv_bfloat16*)x,
                      (const __nv_bfloat16*)w, offsets, perm, top, (TO*)out, experts, o, k);
  }
  IFB_ALLOW_SMEM((moe_linear_mma_kernel<TO, false>), mm_smem_bytes<false>());
  return ifb_launch(moe_linear_mma_kernel<TO, false>, grid, dim3(MM_THREADS), mm_smem_bytes<false>(), s, (const __nv_bfloat16*)x,
                    (const __nv_bfloat16*)w, offsets, perm, top, (TO*)out, experts, o, k);
}

template <typename TA, typename TW, typename TO>
static int ml_launch(const void* x, const void* w, const int* offsets, const int* perm, int top, void* out, int rows, int experts,
                     int o, int k, int gated, cudaStream_t s) {
  dim3 grid((o + ML_COLS - 1) / ML_COLS, (rows + ML_ROWS - 1) / ML_ROWS + experts);
  if (grid.y > 65535) return IFB_ERR_SIZE;
  if (gated)
    return ifb_launch(moe_linear_kernel<TA, TW, TO, true>, grid, dim3(ML_THREADS), 0, s, (const TA*)x, (const TW*)w, offsets, perm,
                      top, (TO*)out, experts, o, k);
  return ifb_launch(moe_linear_kernel<TA, TW, TO, false>, grid, dim3(ML_THREADS), 0, s, (const TA*)x, (const TW*)w, offsets, perm,
                    top, (TO*)out, experts, o, k);
}

// x and w: float32 or bfloat16, in any mix; out: float32 or bfloat16.  rows: the number of rows of `out` (the pairs);
// o: outputs per row (with gated, w holds 2 o rows per expert).  tensor_cores: bfloat16 x and w with k a multiple of 8
// run the mma.sync kernel; everything else, and everything when it is 0, runs the plain kernel.
IFB_EXPORT int ifb_moe_linear(const void* x, int x_dtype, const void* w, int w_dtype, const int* offsets, const int* perm, int top,
                              void* out, int out_dtype, int rows, int experts, int o, int k, int gated, int tensor_cores,
                              cudaStream_t stream) {
  if (rows <= 0 || o <= 0) return IFB_OK;
  if (experts < 1 || k < 1 || top < 1) return IFB_ERR_SIZE;
  if (tensor_cores && x_dtype == IFB_BF16 && w_dtype == IFB_BF16 && k % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0)) {
    const bool few = rows <= MM_SKINNY_MAX_ROWS;          // a step of few rows: tiles of 16 rows and a deep pipeline
    if (out_dtype == IFB_F32)
      return few ? sk_launch<float>(x, w, offsets, perm, top, out, rows, experts, o, k, gated, stream)
                 : mm_launch<float>(x, w, offsets, perm, top, out, rows, experts, o, k, gated, stream);
    if (out_dtype == IFB_BF16)
      return few ? sk_launch<__nv_bfloat16>(x, w, offsets, perm, top, out, rows, experts, o, k, gated, stream)
                 : mm_launch<__nv_bfloat16>(x, w, offsets, perm, top, out, rows, experts, o, k, gated, stream);
    return IFB_ERR_DTYPE;
  }
#define ML_CASE(XD, WD, OD, TA, TW, TO)                                                                      \
  if (x_dtype == XD && w_dtype == WD && out_dtype == OD)                                                     \
    return ml_launch<TA, TW, TO>(x, w, offsets, perm, top, out, rows, experts, o, k, gated, stream);
  ML_CASE(IFB_F32, IFB_F32, IFB_F32, float, float, float)
  ML_CASE(IFB_BF16, IFB_BF16, IFB_F32, __nv_bfloat16, __nv_bfloat16, float)
  ML_CASE(IFB_BF16, IFB_BF16, IFB_BF16, __nv_bfloat16, __nv_bfloat16, __nv_bfloat16)
  ML_CASE(IFB_BF16, IFB_F32, IFB_F32, __nv_bfloat16, float, float)
  ML_CASE(IFB_BF16, IFB_F32, IFB_BF16, __nv_bfloat16, float, __nv_bfloat16)
  ML_CASE(IFB_F32, IFB_BF16, IFB_F32, float, __nv_bfloat16, float)
#undef ML_CASE
  return IFB_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------
// out[n][f] = sum_j gates[n][j] * y[pos[n * top + j]][f], j ascending, float32 (gates null: every weight is 1, for experts whose
// weight went into what they read); then, with `shared` (the result of an
// expert that every row runs), + g * shared[n][f], g = sigmoid(shared_logit[n * logit_stride]) or 1 without a logit.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos, const float* __restrict__ gates,
                   float* __restrict__ out, int top, int width, const float* __restrict__ shared,
                   const float* __restrict__ shared_logit, int logit_stride) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int n = blockIdx.x;
  float g = 1.f;
  if (shared != nullptr && shared_logit != nullptr) g = 1.f / (1.f + expf(-shared_logit[(size_t)n * logit_stride]));
  for (int f = threadIdx.x; f < width; f += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j)
      acc = fmaf(gates ? gates[(size_t)n * top + j] : 1.f, y[(size_t)pos[(size_t)n * top + j] * width + f], acc);
    if (shared != nullptr) acc = fmaf(g, shared[(size_t)n * width + f], acc);
    out[(size_t)n * width + f] = acc;
  }
}

IFB_EXPORT int ifb_moe_combine(const float* y, const int* pos, const float* gates, float* out, int rows, int top, int width,
                               const float* shared, const float* shared_logit, int logit_stride, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return IFB_OK;
  if (top < 1) return IFB_ERR_SIZE;
  return ifb_launch(moe_combine_kernel, dim3(rows), dim3(256), 0, stream, y, pos, gates, out, top, width, shared, shared_logit,
                    logit_stride);
}
