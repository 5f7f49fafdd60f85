// Chapter router: fp32 mean-pool, router GEMV, softmax, prefix mask, exact top-k with the total
// order (value descending, chapter id ascending), weight renormalisation, shared-chapter prefix,
// load-balance / auxiliary / z losses and entropy -- and the backward of all of it.
//
// All kernels here are bandwidth or latency bound (the router is ~5e7 FLOPs); reductions are
// done in a fixed order so results do not depend on scheduling.
#include <math.h>

#include "moc_common.cuh"

namespace moc {
namespace {

constexpr int kPoolSplits = 32;       // sequence splits of the mean-pool
constexpr int kSelectThreads = 1024;  // one CTA per batch row in the select / dlogits kernels
constexpr int kLossChunk = 256;       // chapters per CTA in the loss kernels
constexpr int kLogitsPerWarp = 1;    // chapters per warp in the logits / d_w kernels
constexpr int kDpChunk = 16;          // chapters per CTA in the d_pooled kernel

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// ---- block reductions (fixed order) ----------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  if (warp == 0) {
    t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// ---- forward ---------------------------------------------------------------------------------
// partial[b][split][c] = sum over the split's positions of h[b, t, c]
template <typename T>
__global__ void pool_partial_kernel(const T* __restrict__ h, float* __restrict__ partial, int L, int d) {
  const int b = blockIdx.x, sp = blockIdx.y;
  const int rows_per = (L + kPoolSplits - 1) / kPoolSplits;
  const int t0 = sp * rows_per;
  const int t1 = min(L, t0 + rows_per);
  const T* base = h + (static_cast<long long>(b) * L) * d;
  float* dst = partial + (static_cast<long long>(b) * kPoolSplits + sp) * d;
  if (sizeof(T) == 2 && (d & 7) == 0 && (reinterpret_cast<uintptr_t>(h) & 15) == 0) {
    // bf16 rows in 16-byte pieces: eight columns per thread, four independent row loads in flight
    for (int c8 = threadIdx.x; c8 < (d >> 3); c8 += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      const uint4* col = reinterpret_cast<const uint4*>(base) + c8;
      const long long stride = d >> 3;
      int t = t0;
      for (; t + 4 <= t1; t += 4) {
        uint4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = col[(t + i) * stride];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] += __uint_as_float(w[j] << 16);
            acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
          }
        }
      }
      for (; t < t1; ++t) {
        const uint4 v = col[t * stride];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += __uint_as_float(w[j] << 16);
          acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[c8 * 8 + j] = acc[j];
    }
    return;
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int t = t0; t < t1; ++t) acc += to_f32(base[static_cast<long long>(t) * d + c]);
    dst[c] = acc;
  }
}
__global__ void pool_finish_kernel(const float* __restrict__ partial, float* __restrict__ pooled, int L, int d,
                                   int total) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int b = i / d, c = i - b * d;
  float acc = 0.f;
  for (int sp = 0; sp < kPoolSplits; ++sp) acc += partial[(static_cast<long long>(b) * kPoolSplits + sp) * d + c];
  pooled[i] = acc / static_cast<float>(L);
}

// pooled[b, c] = sum_t pos_weight[t] * h[b, t, c]: the sequence-rolling pooling of the reference collapses to one
// coefficient per position (the average over t of the rolling-window means is linear in h).  Same split layout
// as the plain mean: partial sums per (batch row, sequence split), then a fixed-order sum over the splits.
template <typename T>
__global__ void pool_weighted_partial_kernel(const T* __restrict__ h, const float* __restrict__ pos_weight,
                                             float* __restrict__ partial, int L, int d) {
  const int b = blockIdx.x, sp = blockIdx.y;
  const int rows_per = (L + kPoolSplits - 1) / kPoolSplits;
  const int t0 = sp * rows_per;
  const int t1 = min(L, t0 + rows_per);
  const T* base = h + (static_cast<long long>(b) * L) * d;
  float* dst = partial + (static_cast<long long>(b) * kPoolSplits + sp) * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int t = t0; t < t1; ++t) acc = fmaf(pos_weight[t], to_f32(base[static_cast<long long>(t) * d + c]), acc);
    dst[c] = acc;
  }
}
__global__ void pool_weighted_finish_kernel(const float* __restrict__ partial, float* __restrict__ pooled, int d,
                                            int total) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int b = i / d, c = i - b * d;
  float acc = 0.f;
  for (int sp = 0; sp < kPoolSplits; ++sp) acc += partial[(static_cast<long long>(b) * kPoolSplits + sp) * d + c];
  pooled[i] = acc;
}
// d_h[b, t, :] (+)= pos_weight[t] * d_pooled[b, :]
template <typename T>
__global__ void pool_weighted_bwd_kernel(const float* __restrict__ d_pooled, const float* __restrict__ pos_weight,
                                         T* __restrict__ d_h, int L, int d, long long total, int accumulate) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / d;
    const int c = static_cast<int>(i - row * d);
    const int b = static_cast<int>(row / L), t = static_cast<int>(row - static_cast<long long>(b) * L);
    float v = d_pooled[static_cast<long long>(b) * d + c] * pos_weight[t];
    if (accumulate) v += to_f32(d_h[i]);
    if constexpr (sizeof(T) == 4) d_h[i] = v; else d_h[i] = __float2bfloat16(v);
  }
}

// logits[b,c] = <pooled[b,:], w[c,:]> + bias[c]; one warp per chapter, 8 batch rows per pass
__global__ void logits_kernel(const float* __restrict__ pooled, const float* __restrict__ w,
                              const float* __restrict__ bias, float* __restrict__ logits, int B, int d, int C) {
  extern __shared__ float sp[];   // [8][d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool vec = (d & 3) == 0;
  // the first chapter's weight row is requested before the pooled states are staged, so both fetches overlap
  float4 wpre[8];
  const bool pre = vec && d <= 1024 && kLogitsPerWarp == 1;
  if (pre) {
    const int c = blockIdx.x * (blockDim.x >> 5) + warp;
    const float4* w4 = reinterpret_cast<const float4*>(w + static_cast<long long>(c < C ? c : 0) * d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = lane + 32 * i;
      wpre[i] = (k < d / 4) ? w4[k] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  for (int b0 = 0; b0 < B; b0 += 8) {
    const int nb = min(8, B - b0);
    __syncthreads();
    for (int i = threadIdx.x; i < nb * d; i += blockDim.x) sp[i] = pooled[static_cast<long long>(b0) * d + i];
    __syncthreads();
    for (int cc = 0; cc < kLogitsPerWarp; ++cc) {
      const int c = (blockIdx.x * (blockDim.x >> 5) + warp) * kLogitsPerWarp + cc;
      if (c >= C) break;
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      const float* wr = w + static_cast<long long>(c) * d;
      if (vec && d <= 1024) {
        // the whole weight row is requested before any arithmetic: 8 independent 16-byte loads per lane
        const float4* w4 = reinterpret_cast<const float4*>(wr);
        float4 wv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int k = lane + 32 * i;
          wv[i] = pre ? wpre[i] : ((k < d / 4) ? w4[k] : make_float4(0.f, 0.f, 0.f, 0.f));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int k = lane + 32 * i;
          if (k < d / 4) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (j < nb) {
                const float4 pv = reinterpret_cast<const float4*>(sp + j * d)[k];
                acc[j] = fmaf(wv[i].x, pv.x, fmaf(wv[i].y, pv.y, fmaf(wv[i].z, pv.z, fmaf(wv[i].w, pv.w, acc[j]))));
              }
          }
        }
      } else if (vec) {
        const float4* w4 = reinterpret_cast<const float4*>(wr);
        for (int k = lane; k < d / 4; k += 32) {
          const float4 wv = w4[k];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < nb) {
              const float4 pv = reinterpret_cast<const float4*>(sp + j * d)[k];
              acc[j] = fmaf(wv.x, pv.x, fmaf(wv.y, pv.y, fmaf(wv.z, pv.z, fmaf(wv.w, pv.w, acc[j]))));
            }
        }
      } else {
        for (int k = lane; k < d; k += 32) {
          const float wv = wr[k];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < nb) acc[j] = fmaf(wv, sp[j * d + k], acc[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < nb) {
          const float s = warp_sum(acc[j]);
          if (lane == 0) logits[static_cast<long long>(b0 + j) * C + c] = s + (bias ? bias[c] : 0.f);
        }
      }
    }
  }
}

// One CTA per batch row: softmax, prefix mask + renormalise, exact top-k, weights, shared prefix.
__global__ void __launch_bounds__(kSelectThreads)
select_kernel(const float* __restrict__ logits, float* __restrict__ probs, long long* __restrict__ idx,
              float* __restrict__ weights, int* __restrict__ comb_idx, float* __restrict__ comb_w,
              float* __restrict__ row_stats, int C, int k_sel, int S, float rho) {
  extern __shared__ float sm[];            // [C] masked probabilities, then selection scratch
  float* pt = sm;                          // p~
  uint32_t* sel_key = reinterpret_cast<uint32_t*>(sm + C);   // [k_sel]
  int* sel_idx = reinterpret_cast<int*>(sel_key + k_sel);    // [k_sel]
  __shared__ float red[33];
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_krem, s_count, s_ties;

  const int b = blockIdx.x;
  const float* z = logits + static_cast<long long>(b) * C;
  float* p = probs + static_cast<long long>(b) * C;

  float m = -INFINITY;
  for (int c = threadIdx.x; c < C; c += blockDim.x) m = fmaxf(m, z[c]);
  m = block_max(m, red);
  float s = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float e = expf(z[c] - m);
    pt[c] = e;
    s += e;
  }
  const float denom = block_sum(s, red);
  float ms = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float pv = pt[c] / denom;
    p[c] = pv;
    const float pm = (c < S) ? 0.f : pv;
    pt[c] = pm;
    ms += pm;
  }
  const float masked_mass = block_sum(ms, red);
  if (S > 0) {
    const float dn = fmaxf(masked_mass, 1e-12f);
    for (int c = threadIdx.x; c < C; c += blockDim.x) pt[c] = pt[c] / dn;
  }
  __syncthreads();

  float topk_mass = 0.f, comb_mass = static_cast<float>(S);
  if (k_sel > 0) {
    // radix select on the fp32 bit pattern (non-negative values order like unsigned integers)
    if (threadIdx.x == 0) { s_prefix = 0u; s_krem = k_sel; }
    uint32_t mask = 0u;
    for (int pass = 3; pass >= 0; --pass) {
      for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const uint32_t key = __float_as_uint(pt[c]);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> (8 * pass)) & 255u], 1);
      }
      __syncthreads();
      if (threadIdx.x < 32) {
        // warp 0 finds, from the top bin down, the bin in which the running count reaches s_krem
        const int lane = threadIdx.x;
        int h8[8], sl = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) { h8[i] = hist[lane * 8 + i]; sl += h8[i]; }
        int incl = sl;                       // inclusive suffix sum over lanes lane..31
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_down_sync(0xffffffffu, incl, o);
          if (lane + o < 32) incl += t;
        }
        const int above = incl - sl;         // elements in bins owned by higher lanes
        const int rem0 = s_krem;
        const bool mine = (above < rem0) && (rem0 <= incl);
        const unsigned who = __ballot_sync(0xffffffffu, mine);
        // all remaining elements sit in bin 0 of lane 0 when no lane qualifies (cannot happen while rem0 <= count)
        const int owner = who ? (31 - __clz(who)) : 0;
        if (lane == owner) {
          int rem = rem0 - above, i = 7;
          for (; i > 0; --i) {
            if (h8[i] >= rem) break;
            rem -= h8[i];
          }
          s_krem = rem;
          s_prefix = prefix | (static_cast<uint32_t>(lane * 8 + i) << (8 * pass));
          s_ties = h8[i];
        }
      }
      mask |= 0xFFu << (8 * pass);
      __syncthreads();
    }
    const uint32_t thr = s_prefix;     // bit pattern of the k-th largest value
    const int need_ties = s_krem;      // how many entries equal to it are selected
    const int have_ties = s_ties;
    if (threadIdx.x == 0) s_count = 0;
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      const uint32_t key = __float_as_uint(pt[c]);
      if (key > thr || (key == thr && have_ties == need_ties)) {
        const int pos = atomicAdd(&s_count, 1);
        if (pos < k_sel) { sel_key[pos] = key; sel_idx[pos] = c; }
      }
    }
    __syncthreads();
    if (have_ties != need_ties && threadIdx.x == 0) {
      int pos = s_count, taken = 0;            // more ties than slots: lowest chapter ids win
      for (int c = 0; c < C && taken < need_ties; ++c) {
        if (__float_as_uint(pt[c]) == thr) {
          if (pos < k_sel) { sel_key[pos] = thr; sel_idx[pos] = c; }
          ++pos; ++taken;
        }
      }
    }
    __syncthreads();
    // rank sort of the k selected entries: value descending, chapter id ascending (shared memory)
    float* srt_w = sm;                         // p~ is no longer needed: reuse its first 2k words
    int* srt_i = reinterpret_cast<int*>(sm + k_sel);
    uint32_t kt_reg[1]; int it_reg[1]; int rk_reg[1];
    {
      const int t = threadIdx.x;
      if (t < k_sel) {
        const uint32_t kt = sel_key[t];
        const int it = sel_idx[t];
        int rank = 0;
        for (int j = 0; j < k_sel; ++j) {
          const uint32_t kj = sel_key[j];
          rank += (kj > kt) || (kj == kt && sel_idx[j] < it);
        }
        kt_reg[0] = kt; it_reg[0] = it; rk_reg[0] = rank;
      }
    }
    __syncthreads();
    if (threadIdx.x < k_sel) { srt_w[rk_reg[0]] = __uint_as_float(kt_reg[0]); srt_i[rk_reg[0]] = it_reg[0]; }
    __syncthreads();
    float part = 0.f;
    for (int j = threadIdx.x; j < k_sel; j += blockDim.x) part += srt_w[j];
    topk_mass = block_sum(part, red);
    const float dn = fmaxf(topk_mass, 1e-12f);
    long long* out_idx = idx + static_cast<long long>(b) * k_sel;
    float* out_w = weights + static_cast<long long>(b) * k_sel;
    float cpart = 0.f;
    for (int j = threadIdx.x; j < k_sel; j += blockDim.x) {
      const float wj = srt_w[j] / dn;
      srt_w[j] = wj;
      out_w[j] = wj;
      out_idx[j] = srt_i[j];
      cpart += wj * rho;
    }
    comb_mass = static_cast<float>(S) + block_sum(cpart, red);
  }
  // shared prefix + renormalised combined weights (only meaningful when S > 0; with S == 0 the
  // combined lists are the routed lists unchanged)
  const int kc = S + k_sel;
  for (int j = threadIdx.x; j < kc; j += blockDim.x) {
    int ci; float u;
    if (j < S) { ci = j; u = 1.f; }
    else { ci = reinterpret_cast<int*>(sm + k_sel)[j - S]; u = sm[j - S] * (S > 0 ? rho : 1.f); }
    comb_idx[static_cast<long long>(b) * kc + j] = ci;
    comb_w[static_cast<long long>(b) * kc + j] = (S > 0) ? u / fmaxf(comb_mass, 1e-12f) : u;
  }
  if (threadIdx.x == 0) {
    float* rs = row_stats + static_cast<long long>(b) * 4;
    rs[0] = m + logf(denom);
    rs[1] = masked_mass;
    rs[2] = topk_mass;
    rs[3] = comb_mass;
  }
}

// Per chapter chunk: f, mean p^2, and partial sums of the three chapter-separable loss terms.
__global__ void loss_partial_kernel(const float* __restrict__ probs, const long long* __restrict__ idx,
                                    float* __restrict__ chapter_stats, float* __restrict__ partial,
                                    int B, int C, int k_sel) {
  __shared__ int cnt[kLossChunk];
  __shared__ float red[33];
  const int c0 = blockIdx.x * kLossChunk;
  for (int i = threadIdx.x; i < kLossChunk; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  const long long n_idx = static_cast<long long>(B) * k_sel;
  for (long long i = threadIdx.x; i < n_idx; i += blockDim.x) {
    const int c = static_cast<int>(idx[i]) - c0;
    if (c >= 0 && c < kLossChunk) atomicAdd(&cnt[c], 1);
  }
  __syncthreads();
  float lb = 0.f, aux = 0.f, ent = 0.f;
  const int c = c0 + threadIdx.x;
  if (threadIdx.x < kLossChunk && c < C) {
    float ps = 0.f, p2 = 0.f, e = 0.f;
    for (int b = 0; b < B; ++b) {
      const float pv = probs[static_cast<long long>(b) * C + c];
      ps += pv;
      p2 += pv * pv;
      e += pv * logf(fmaxf(pv, 1e-12f));
    }
    const float f = static_cast<float>(cnt[threadIdx.x]) / static_cast<float>(B);
    const float P = ps / static_cast<float>(B);
    const float q = p2 / static_cast<float>(B);
    chapter_stats[c] = f;
    chapter_stats[C + c] = q;
    lb = f * P;
    const float dv = q - 1.f / static_cast<float>(C);
    aux = dv * dv;
    ent = e;
  }
  lb = block_sum(lb, red);
  aux = block_sum(aux, red);
  ent = block_sum(ent, red);
  if (threadIdx.x == 0) {
    partial[blockIdx.x * 3 + 0] = lb;
    partial[blockIdx.x * 3 + 1] = aux;
    partial[blockIdx.x * 3 + 2] = ent;
  }
}
// The same statistics for many routing rows (token-level routing: B = batch * seq): the rows are cut into `splits`
// ranges, every (chapter chunk, range) CTA leaves {sum p, sum p^2, sum p log p, count} per chapter, and a second kernel
// adds the ranges in order before the non-linear terms are formed.
__global__ void loss_rows_partial_kernel(const float* __restrict__ probs, const long long* __restrict__ idx,
                                         float* __restrict__ part, int B, int C, int k_sel, int rows_per_split) {
  __shared__ int cnt[kLossChunk];
  const int c0 = blockIdx.x * kLossChunk;
  const int r0 = blockIdx.y * rows_per_split, r1 = min(B, r0 + rows_per_split);
  cnt[threadIdx.x] = 0;
  __syncthreads();
  for (long long i = static_cast<long long>(r0) * k_sel + threadIdx.x; i < static_cast<long long>(r1) * k_sel;
       i += blockDim.x) {
    const int c = static_cast<int>(idx[i]) - c0;
    if (c >= 0 && c < kLossChunk) atomicAdd(&cnt[c], 1);
  }
  __syncthreads();
  const int c = c0 + threadIdx.x;
  if (c >= C) return;
  float ps = 0.f, p2 = 0.f, e = 0.f;
  for (int b = r0; b < r1; ++b) {
    const float pv = probs[static_cast<long long>(b) * C + c];
    ps += pv;
    p2 += pv * pv;
    e += pv * logf(fmaxf(pv, 1e-12f));
  }
  float4* dst = reinterpret_cast<float4*>(part) + static_cast<long long>(blockIdx.y) * C + c;
  *dst = make_float4(ps, p2, e, static_cast<float>(cnt[threadIdx.x]));
}
__global__ void loss_rows_finish_kernel(const float* __restrict__ part, float* __restrict__ chapter_stats,
                                        float* __restrict__ partial, int B, int C, int splits) {
  __shared__ float red[33];
  const int c = blockIdx.x * kLossChunk + threadIdx.x;
  float lb = 0.f, aux = 0.f, ent = 0.f;
  if (c < C) {
    float ps = 0.f, p2 = 0.f, e = 0.f, n = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
      const float4 v = reinterpret_cast<const float4*>(part)[static_cast<long long>(sp) * C + c];
      ps += v.x; p2 += v.y; e += v.z; n += v.w;
    }
    const float f = n / static_cast<float>(B);
    const float P = ps / static_cast<float>(B);
    const float q = p2 / static_cast<float>(B);
    chapter_stats[c] = f;
    chapter_stats[C + c] = q;
    lb = f * P;
    const float dv = q - 1.f / static_cast<float>(C);
    aux = dv * dv;
    ent = e;
  }
  lb = block_sum(lb, red);
  aux = block_sum(aux, red);
  ent = block_sum(ent, red);
  if (threadIdx.x == 0) {
    partial[blockIdx.x * 3 + 0] = lb;
    partial[blockIdx.x * 3 + 1] = aux;
    partial[blockIdx.x * 3 + 2] = ent;
  }
}
__global__ void loss_finish_kernel(const float* __restrict__ partial, const float* __restrict__ row_stats,
                                   float* __restrict__ losses, int nblk, int B, int C) {
  // one warp; every lane sums a strided share in a fixed order, then a fixed-order shuffle tree
  if (blockIdx.x != 0 || threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  float lb = 0.f, aux = 0.f, ent = 0.f, z = 0.f;
  for (int i = lane; i < nblk; i += 32) { lb += partial[i * 3]; aux += partial[i * 3 + 1]; ent += partial[i * 3 + 2]; }
  for (int b = lane; b < B; b += 32) { const float l = row_stats[static_cast<long long>(b) * 4]; z += l * l; }
  lb = warp_sum(lb); aux = warp_sum(aux); ent = warp_sum(ent); z = warp_sum(z);
  if (lane == 0) {
    losses[0] = static_cast<float>(C) * lb;
    losses[1] = aux / static_cast<float>(C);
    losses[2] = z / static_cast<float>(B);
    losses[3] = -ent / static_cast<float>(B);
  }
}

// logits[r, c] += bias[c]
__global__ void add_bias_kernel(float* __restrict__ logits, const float* __restrict__ bias, long long total, int C) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    logits[i] += bias[static_cast<int>(i % C)];
}
// dst[r, c] = bias[c] + sum_t src[r, t * ld + c], smallest term (highest t) first
__global__ void sum_terms_kernel(const float* __restrict__ src, const float* __restrict__ bias,
                                 float* __restrict__ dst, long long rows, int cols, int ld, int terms) {
  const long long total = rows * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols;
    const int c = static_cast<int>(i - r * cols);
    const float* p = src + r * static_cast<long long>(ld) * terms + c;
    float acc = 0.f;
    for (int t = terms - 1; t >= 0; --t) acc += p[static_cast<long long>(t) * ld];
    dst[i] = bias != nullptr ? acc + bias[c] : acc;
  }
}
// out[c] = sum_r x[r, c]: one CTA per 32 columns, 8 row groups, fixed-order sums
__global__ void col_sum_kernel(const float* __restrict__ x, float* __restrict__ out, long long rows, int cols) {
  __shared__ float part[8][32];
  const int c = blockIdx.x * 32 + (threadIdx.x & 31), g = threadIdx.x >> 5;
  float acc = 0.f;
  if (c < cols)
    for (long long r = g; r < rows; r += 8) acc += x[r * cols + c];
  part[g][threadIdx.x & 31] = acc;
  __syncthreads();
  if (g == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += part[i][threadIdx.x];
    out[c] = t;
  }
}

// ---- backward --------------------------------------------------------------------------------
// One CTA per batch row: gradient of everything downstream of the logits.
__global__ void __launch_bounds__(kSelectThreads)
dlogits_kernel(const float* __restrict__ probs, const long long* __restrict__ idx,
               const float* __restrict__ weights, const float* __restrict__ comb_w,
               const float* __restrict__ row_stats, const float* __restrict__ chapter_stats,
               const float* __restrict__ d_weights, const float* __restrict__ d_comb_w,
               const float* __restrict__ d_losses, float* __restrict__ d_logits,
               int B, int C, int k_sel, int S, float rho) {
  extern __shared__ float dp[];   // [C]
  __shared__ float red[33];
  __shared__ float s_dv[1024];    // k_sel <= 1024
  __shared__ float s_scal[2];
  const int b = blockIdx.x;
  const float* p = probs + static_cast<long long>(b) * C;
  const float lse = row_stats[b * 4 + 0], s_mass = row_stats[b * 4 + 1];
  const float v_mass = row_stats[b * 4 + 2], u_mass = row_stats[b * 4 + 3];
  const float g_lb = d_losses ? d_losses[0] : 0.f, g_aux = d_losses ? d_losses[1] : 0.f;
  const float g_z = d_losses ? d_losses[2] : 0.f, g_ent = d_losses ? d_losses[3] : 0.f;
  const int kc = S + k_sel;

  // (a)+(b): gradients of the k selected (unnormalised) masked probabilities v_j
  __shared__ float s_w[1024];
  float dotu_p = 0.f;
  if (d_comb_w != nullptr && S > 0)
    for (int i = threadIdx.x; i < kc; i += blockDim.x)
      dotu_p += d_comb_w[static_cast<long long>(b) * kc + i] * comb_w[static_cast<long long>(b) * kc + i];
  const float dotu = block_sum(dotu_p, red);
  float dotw_p = 0.f;
  for (int j = threadIdx.x; j < k_sel; j += blockDim.x) {
    float dw = d_weights ? d_weights[static_cast<long long>(b) * k_sel + j] : 0.f;
    if (d_comb_w != nullptr) {
      const float dcu = d_comb_w[static_cast<long long>(b) * kc + S + j];
      if (S > 0) dw += rho * ((u_mass >= 1e-12f) ? (dcu - dotu) / u_mass : dcu / 1e-12f);
      else dw += dcu;
    }
    const float wj = weights[static_cast<long long>(b) * k_sel + j];
    s_dv[j] = dw;
    s_w[j] = wj;
    dotw_p += dw * wj;
  }
  const float dotw = block_sum(dotw_p, red);
  float a_p = 0.f;
  for (int j = threadIdx.x; j < k_sel; j += blockDim.x) {
    const float dv = (v_mass >= 1e-12f) ? (s_dv[j] - dotw) / v_mass : s_dv[j] / 1e-12f;
    s_dv[j] = dv;
    a_p += dv * (s_w[j] * fmaxf(v_mass, 1e-12f));   // v_j
  }
  const float a_tot = block_sum(a_p, red);
  if (threadIdx.x == 0) s_scal[0] = a_tot;
  __syncthreads();
  const float A = s_scal[0];
  const bool renorm = (S > 0);
  const float inv_s = renorm ? ((s_mass >= 1e-12f) ? 1.f / s_mass : 1e12f) : 1.f;
  const float dense = (renorm && s_mass >= 1e-12f) ? -A * inv_s : 0.f;
  const float invB = 1.f / static_cast<float>(B), invC = 1.f / static_cast<float>(C);
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float pv = p[c];
    float g = (c >= S) ? dense : 0.f;
    g += g_lb * static_cast<float>(C) * chapter_stats[c] * invB;
    g += g_aux * (2.f * invC) * (chapter_stats[C + c] - invC) * (2.f * pv * invB);
    g += g_ent * (-invB) * (logf(fmaxf(pv, 1e-12f)) + (pv > 1e-12f ? 1.f : 0.f));
    dp[c] = g;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < k_sel; j += blockDim.x) {
    const int c = static_cast<int>(idx[static_cast<long long>(b) * k_sel + j]);
    dp[c] += s_dv[j] * inv_s;    // chapter ids in one row are distinct
  }
  __syncthreads();
  float dot = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) dot += dp[c] * p[c];
  dot = block_sum(dot, red);
  const float zc = g_z * 2.f * lse * invB;
  for (int c = threadIdx.x; c < C; c += blockDim.x)
    d_logits[static_cast<long long>(b) * C + c] = p[c] * (dp[c] - dot + zc);
}

// d_w[c,:] = sum_b d_logits[b,c] * pooled[b,:]; d_bias[c] = sum_b d_logits[b,c]; one warp per chapter,
// 8 batch rows of `pooled` staged in shared memory per pass
__global__ void dweight_kernel(const float* __restrict__ d_logits, const float* __restrict__ pooled,
                               float* __restrict__ d_w, float* __restrict__ d_bias, int B, int d, int C) {
  extern __shared__ float sp[];   // [8][d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c_first = (blockIdx.x * (blockDim.x >> 5) + warp) * kLogitsPerWarp;
  float bsum[kLogitsPerWarp];
#pragma unroll
  for (int cc = 0; cc < kLogitsPerWarp; ++cc) bsum[cc] = 0.f;
  for (int b0 = 0; b0 < B; b0 += 8) {
    const int nb = min(8, B - b0);
    __syncthreads();
    // rows past the batch are zero-filled: they are multiplied by dz = 0 below, and 0 x stale NaN would be NaN
    for (int i = threadIdx.x; i < 8 * d; i += blockDim.x)
      sp[i] = (i < nb * d) ? pooled[static_cast<long long>(b0) * d + i] : 0.f;
    __syncthreads();
#pragma unroll
    for (int cc = 0; cc < kLogitsPerWarp; ++cc) {
      const int c = c_first + cc;
      if (c >= C) break;
      float dz[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dz[j] = j < nb ? d_logits[static_cast<long long>(b0 + j) * C + c] : 0.f;
        bsum[cc] += dz[j];
      }
      float* dst = d_w + static_cast<long long>(c) * d;
      for (int k = lane; k < d; k += 32) {
        float acc = (b0 == 0) ? 0.f : dst[k];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(dz[j], sp[j * d + k], acc);
        dst[k] = acc;
      }
    }
  }
#pragma unroll
  for (int cc = 0; cc < kLogitsPerWarp; ++cc)
    if (c_first + cc < C && lane == 0 && d_bias) d_bias[c_first + cc] = bsum[cc];
}

// partial[chunk][b][k] = sum over the chunk's chapters of d_logits[b,c] * w[c,k]
__global__ void dpooled_partial_kernel(const float* __restrict__ d_logits, const float* __restrict__ w,
                                       float* __restrict__ partial, int B, int d, int C) {
  __shared__ float dz[8][kDpChunk];
  const int c0 = blockIdx.x * kDpChunk;
  const int nc = min(kDpChunk, C - c0);
  for (int b0 = 0; b0 < B; b0 += 8) {
    const int nb = min(8, B - b0);
    __syncthreads();
    for (int i = threadIdx.x; i < nb * kDpChunk; i += blockDim.x) {
      const int j = i / kDpChunk, cc = i - j * kDpChunk;
      dz[j][cc] = (cc < nc) ? d_logits[static_cast<long long>(b0 + j) * C + c0 + cc] : 0.f;
    }
    __syncthreads();
    for (int k = threadIdx.x; k < d; k += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      float wv[kDpChunk];
#pragma unroll
      for (int cc = 0; cc < kDpChunk; ++cc)            // all loads first: they are independent
        wv[cc] = cc < nc ? w[static_cast<long long>(c0 + cc) * d + k] : 0.f;
#pragma unroll
      for (int cc = 0; cc < kDpChunk; ++cc) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(dz[j][cc], wv[cc], acc[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nb) partial[(static_cast<long long>(blockIdx.x) * B + b0 + j) * d + k] = acc[j];
    }
  }
}
__global__ void dpooled_finish_kernel(const float* __restrict__ partial, float* __restrict__ d_pooled,
                                      int nchunks, int total) {
  // eight adjacent lanes share one output: each sums every eighth partial, then a fixed-order shuffle reduce
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = t >> 3, sub = t & 7;
  float acc = 0.f;
  if (i < total)
    for (int ch = sub; ch < nchunks; ch += 8) acc += partial[static_cast<long long>(ch) * total + i];
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (i < total && sub == 0) d_pooled[i] = acc;
}
// d_h[b, t, :] (+)= d_pooled[b, :] / L; one thread per 8 consecutive columns of one row (d % 8 == 0),
// falling back to one element per thread otherwise
template <typename T>
__global__ void dh_broadcast_kernel(const float* __restrict__ d_pooled, T* __restrict__ d_h, int L, int d,
                                    long long rows, int accumulate) {
  const float invL = 1.f / static_cast<float>(L);
  if ((d & 7) == 0) {
    const int per_row = d >> 3;
    const long long total = rows * per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long row = i / per_row;
      const int c = static_cast<int>(i - row * per_row) << 3;
      const int b = static_cast<int>(row / L);
      const float4 p0 = *reinterpret_cast<const float4*>(d_pooled + static_cast<long long>(b) * d + c);
      const float4 p1 = *reinterpret_cast<const float4*>(d_pooled + static_cast<long long>(b) * d + c + 4);
      float v[8] = {p0.x * invL, p0.y * invL, p0.z * invL, p0.w * invL, p1.x * invL, p1.y * invL, p1.z * invL, p1.w * invL};
      T* dst = d_h + row * d + c;
      if (accumulate) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] += to_f32(dst[j]);
      }
      if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
      } else {
        uint4 o;
        o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
        o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(dst) = o;
      }
    }
  } else {
    const long long total = rows * d;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long row = i / d;
      const int c = static_cast<int>(i - row * d);
      const int b = static_cast<int>(row / L);
      float v = d_pooled[static_cast<long long>(b) * d + c] * invL;
      if (accumulate) v += to_f32(d_h[i]);
      if constexpr (sizeof(T) == 4) d_h[i] = v; else d_h[i] = __float2bfloat16(v);
    }
  }
}

inline int k_selected(const moc_router_shape* s) {
  int k = s->top_k;
  const int avail = s->num_chapters - s->num_shared;
  if (k > avail) k = avail;
  return k < 0 ? 0 : k;
}
// Scratch layout: [ pooling partials | d_pooled partials ] (they never live at once), then the loss partials.
// A call that neither pools (token rows, or pooled states handed in) nor produces d_pooled needs the loss part only.
inline size_t ws_floats(const moc_router_shape* s, bool pool, bool dpooled) {
  const size_t p = pool ? static_cast<size_t>(s->batch) * kPoolSplits * s->hidden_dim : 0;
  const size_t dp = dpooled ? static_cast<size_t>(ceil_div(s->num_chapters, kDpChunk)) * s->batch * s->hidden_dim : 0;
  return p > dp ? p : dp;
}
// row ranges of the loss statistics: one for the handful of rows of sequence-level routing, ~128 rows each otherwise
inline int loss_row_splits(const moc_router_shape* s) {
  return s->batch <= 256 ? 1 : (ceil_div(s->batch, 128) < 64 ? ceil_div(s->batch, 128) : 64);
}
inline size_t loss_floats(const moc_router_shape* s) {
  const int splits = loss_row_splits(s);
  // (the per-range records are float4: four floats of slack let the block start on a 16-byte boundary)
  const size_t rows_part = splits > 1 ? static_cast<size_t>(splits) * s->num_chapters * 4 + 4 : 0;
  return static_cast<size_t>(ceil_div(s->num_chapters, kLossChunk)) * 3 + rows_part;
}
inline size_t ws_bytes(const moc_router_shape* s) { return (ws_floats(s, true, true) + loss_floats(s)) * sizeof(float); }
inline int check_shape(const moc_router_shape* s) {
  MOC_REQUIRE(s != nullptr, "shape is NULL");
  MOC_REQUIRE(s->batch > 0 && s->seq > 0 && s->hidden_dim > 0, "empty router input");
  MOC_REQUIRE(s->num_chapters > 0, "num_chapters must be > 0");
  MOC_REQUIRE(s->top_k > 0 && s->top_k <= s->num_chapters, "top_k must be in [1, num_chapters]");
  MOC_REQUIRE(s->num_shared >= 0 && s->num_shared <= s->num_chapters, "exclude_prefix_chapters out of range");
  MOC_REQUIRE(s->top_k <= 1024, "top_k above 1024 is not supported");
  MOC_REQUIRE(s->h_dtype == MOC_F32 || s->h_dtype == MOC_BF16, "bad h_dtype");
  MOC_REQUIRE((static_cast<size_t>(s->num_chapters) + 2 * 1024) * 4 <= 200 * 1024, "num_chapters too large");
  return MOC_OK;
}

}  // namespace
}  // namespace moc

using namespace moc;

extern "C" size_t moc_router_workspace_bytes(const moc_router_shape* s) { return s ? ws_bytes(s) : 0; }
extern "C" size_t moc_router_workspace_bytes_parts(const moc_router_shape* s, int32_t fwd_parts, int32_t bwd_parts) {
  if (!s) return 0;
  const bool pool = (fwd_parts & 1) && !(fwd_parts & 8);
  return (ws_floats(s, pool, (bwd_parts & 4) != 0) + loss_floats(s)) * sizeof(float);
}

extern "C" int moc_router_fwd_parts(const moc_router_shape* s, const void* h, const float* w, const float* bias,
                                    float* pooled, float* logits, float* probs, int64_t* idx, float* weights,
                                    int32_t* comb_idx, float* comb_w, float* row_stats, float* chapter_stats,
                                    float* losses, void* workspace, size_t workspace_bytes, int32_t parts,
                                    int32_t* status, void* stream_) {
  int rc = check_shape(s);
  if (rc != MOC_OK) return rc;
  const size_t front = ws_floats(s, (parts & 1) && !(parts & 8), false);
  MOC_REQUIRE(workspace_bytes >= (front + loss_floats(s)) * sizeof(float), "router workspace too small");
  MOC_REQUIRE((h || (parts & 8)) && w && pooled && logits && probs && comb_idx && comb_w && row_stats,
              "NULL router buffer");
  (void)status;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int B = s->batch, L = s->seq, d = s->hidden_dim, C = s->num_chapters, S = s->num_shared;
  const int k_sel = k_selected(s);
  MOC_REQUIRE(k_sel == 0 || (idx && weights), "NULL index / weight buffer");
  float* ws = static_cast<float*>(workspace);
  // the loss partials sit behind the front part of whatever layout the caller sized the workspace for
  float* loss_partial = ws + (workspace_bytes / sizeof(float) - loss_floats(s));

  dim3 pg(B, kPoolSplits);
  if (parts & 1) {
  if (!(parts & 8)) {      // bit 8: `pooled` already holds the pooled states (another pooling rule ran first)
  if (s->h_dtype == MOC_F32)
    pool_partial_kernel<float><<<pg, 256, 0, stream>>>(static_cast<const float*>(h), ws, L, d);
  else
    pool_partial_kernel<__nv_bfloat16><<<pg, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(h), ws, L, d);
  pool_finish_kernel<<<ceil_div(B * d, 256), 256, 0, stream>>>(ws, pooled, L, d, B * d);
  }
  if (parts & 16) {        // bit 16: `logits` already holds pooled x W^T (a projection kernel ran); only the bias is missing
    if (bias != nullptr) {
      const long long total = static_cast<long long>(B) * C;
      long long blocks = (total + 255) / 256;
      if (blocks > 148LL * 16) blocks = 148LL * 16;
      add_bias_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(logits, bias, total, C);
    }
  } else {
    const int warps = 8;
    const size_t sm = static_cast<size_t>(8) * d * sizeof(float);
    MOC_CUDA_OK(cudaFuncSetAttribute(logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm)));
    logits_kernel<<<ceil_div(C, warps * kLogitsPerWarp), warps * 32, sm, stream>>>(pooled, w, bias, logits, B, d, C);
  }
  {
    const size_t sm = (static_cast<size_t>(C) + 2 * static_cast<size_t>(k_sel > 0 ? k_sel : 1)) * 4;
    MOC_CUDA_OK(cudaFuncSetAttribute(select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm)));
    select_kernel<<<B, kSelectThreads, sm, stream>>>(logits, probs, reinterpret_cast<long long*>(idx), weights,
                                                     comb_idx, comb_w, row_stats, C, k_sel, S, s->routed_scale);
  }
  }
  if ((parts & 2) && losses != nullptr) {
    MOC_REQUIRE(chapter_stats != nullptr, "chapter_stats is NULL");
    const int nblk = ceil_div(C, kLossChunk);
    const int splits = loss_row_splits(s);
    if (splits > 1) {
      float* rows_part = reinterpret_cast<float*>(
          (reinterpret_cast<uintptr_t>(loss_partial + static_cast<size_t>(nblk) * 3) + 15) & ~uintptr_t(15));
      const int rows_per_split = ceil_div(B, splits);
      loss_rows_partial_kernel<<<dim3(nblk, splits), kLossChunk, 0, stream>>>(
          probs, reinterpret_cast<const long long*>(idx), rows_part, B, C, k_sel, rows_per_split);
      loss_rows_finish_kernel<<<nblk, kLossChunk, 0, stream>>>(rows_part, chapter_stats, loss_partial, B, C, splits);
    } else {
      loss_partial_kernel<<<nblk, kLossChunk, 0, stream>>>(probs, reinterpret_cast<const long long*>(idx),
                                                           chapter_stats, loss_partial, B, C, k_sel);
    }
    loss_finish_kernel<<<1, 32, 0, stream>>>(loss_partial, row_stats, losses, nblk, B, C);
  }
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_router_fwd(const moc_router_shape* s, const void* h, const float* w, const float* bias,
                              float* pooled, float* logits, float* probs, int64_t* idx, float* weights,
                              int32_t* comb_idx, float* comb_w, float* row_stats, float* chapter_stats,
                              float* losses, void* workspace, size_t workspace_bytes, int32_t* status,
                              void* stream_) {
  return moc_router_fwd_parts(s, h, w, bias, pooled, logits, probs, idx, weights, comb_idx, comb_w, row_stats,
                              chapter_stats, losses, workspace, workspace_bytes, 3, status, stream_);
}

extern "C" int moc_router_bwd_parts(const moc_router_shape* s, const float* w, const float* pooled,
                                    const float* probs, const int64_t* idx, const float* weights,
                                    const float* comb_w, const float* row_stats, const float* chapter_stats,
                                    const float* d_weights, const float* d_comb_w, const float* d_losses,
                                    float* d_logits, float* d_w, float* d_bias, float* d_pooled, void* d_h,
                                    int32_t accumulate_dh, void* workspace, size_t workspace_bytes, int32_t parts,
                                    int32_t* status, void* stream_) {
  int rc = check_shape(s);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(workspace_bytes >= ws_floats(s, false, (parts & 4) != 0) * sizeof(float), "router workspace too small");
  MOC_REQUIRE(w && pooled && probs && comb_w && row_stats && d_logits && d_w && d_pooled, "NULL router buffer");
  MOC_REQUIRE(d_losses == nullptr || chapter_stats != nullptr, "loss gradients need chapter_stats");
  (void)status;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int B = s->batch, L = s->seq, d = s->hidden_dim, C = s->num_chapters, S = s->num_shared;
  const int k_sel = k_selected(s);
  float* ws = static_cast<float*>(workspace);
  if (parts & 1) {
    const size_t sm = static_cast<size_t>(C) * 4;
    MOC_CUDA_OK(cudaFuncSetAttribute(dlogits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm)));
    dlogits_kernel<<<B, kSelectThreads, sm, stream>>>(probs, reinterpret_cast<const long long*>(idx), weights,
                                                      comb_w, row_stats, chapter_stats, d_weights, d_comb_w,
                                                      d_losses, d_logits, B, C, k_sel, S, s->routed_scale);
  }
  if (parts & 2) {
    const size_t sm = static_cast<size_t>(8) * d * sizeof(float);
    MOC_CUDA_OK(cudaFuncSetAttribute(dweight_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm)));
    dweight_kernel<<<ceil_div(C, 8 * kLogitsPerWarp), 256, sm, stream>>>(d_logits, pooled, d_w, d_bias, B, d, C);
  }
  const int nchunks = ceil_div(C, kDpChunk);
  if (parts & 4) {
    dpooled_partial_kernel<<<nchunks, 256, 0, stream>>>(d_logits, w, ws, B, d, C);
    dpooled_finish_kernel<<<ceil_div(B * d * 8, 256), 256, 0, stream>>>(ws, d_pooled, nchunks, B * d);
  }
  if ((parts & 4) && d_h != nullptr) {
    const long long rows = static_cast<long long>(B) * L;
    const long long work = (d & 7) == 0 ? rows * (d >> 3) : rows * d;
    long long blocks = (work + 255) / 256;
    if (blocks > 148LL * 32) blocks = 148LL * 32;
    if (s->h_dtype == MOC_F32)
      dh_broadcast_kernel<float><<<static_cast<int>(blocks), 256, 0, stream>>>(d_pooled, static_cast<float*>(d_h), L, d, rows, accumulate_dh);
    else
      dh_broadcast_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, stream>>>(d_pooled, static_cast<__nv_bfloat16*>(d_h), L, d, rows, accumulate_dh);
  }
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_router_bwd(const moc_router_shape* s, const float* w, const float* pooled,
                              const float* probs, const int64_t* idx, const float* weights,
                              const float* comb_w, const float* row_stats, const float* chapter_stats,
                              const float* d_weights, const float* d_comb_w, const float* d_losses,
                              float* d_logits, float* d_w, float* d_bias, float* d_pooled, void* d_h,
                              int32_t accumulate_dh, void* workspace, size_t workspace_bytes,
                              int32_t* status, void* stream_) {
  return moc_router_bwd_parts(s, w, pooled, probs, idx, weights, comb_w, row_stats, chapter_stats, d_weights,
                              d_comb_w, d_losses, d_logits, d_w, d_bias, d_pooled, d_h, accumulate_dh, workspace,
                              workspace_bytes, 7, status, stream_);
}


extern "C" int moc_pool_weighted_fwd(const void* h, int32_t h_dtype, const float* pos_weight, float* pooled,
                                     int32_t batch, int32_t seq, int32_t dim, void* workspace,
                                     size_t workspace_bytes, void* stream_) {
  MOC_REQUIRE(h && pos_weight && pooled && workspace, "NULL buffer");
  MOC_REQUIRE(batch > 0 && seq > 0 && dim > 0, "empty input");
  MOC_REQUIRE(h_dtype == MOC_F32 || h_dtype == MOC_BF16, "bad h_dtype");
  MOC_REQUIRE(workspace_bytes >= static_cast<size_t>(batch) * kPoolSplits * dim * sizeof(float),
              "pooling workspace too small");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  float* ws = static_cast<float*>(workspace);
  dim3 pg(batch, kPoolSplits);
  if (h_dtype == MOC_F32)
    pool_weighted_partial_kernel<float><<<pg, 256, 0, stream>>>(static_cast<const float*>(h), pos_weight, ws, seq, dim);
  else
    pool_weighted_partial_kernel<__nv_bfloat16><<<pg, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(h),
                                                                        pos_weight, ws, seq, dim);
  pool_weighted_finish_kernel<<<ceil_div(batch * dim, 256), 256, 0, stream>>>(ws, pooled, dim, batch * dim);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_pool_weighted_bwd(const float* d_pooled, const float* pos_weight, void* d_h, int32_t h_dtype,
                                     int32_t batch, int32_t seq, int32_t dim, int32_t accumulate, void* stream_) {
  MOC_REQUIRE(d_pooled && pos_weight && d_h, "NULL buffer");
  MOC_REQUIRE(batch > 0 && seq > 0 && dim > 0, "empty input");
  MOC_REQUIRE(h_dtype == MOC_F32 || h_dtype == MOC_BF16, "bad h_dtype");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long total = static_cast<long long>(batch) * seq * dim;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  if (h_dtype == MOC_F32)
    pool_weighted_bwd_kernel<float><<<static_cast<int>(blocks), 256, 0, stream>>>(
        d_pooled, pos_weight, static_cast<float*>(d_h), seq, dim, total, accumulate);
  else
    pool_weighted_bwd_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, stream>>>(
        d_pooled, pos_weight, static_cast<__nv_bfloat16*>(d_h), seq, dim, total, accumulate);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}


extern "C" int moc_sum_terms(const float* src, const float* bias, float* dst, int64_t rows, int32_t cols, int32_t ld,
                             int32_t terms, void* stream_) {
  MOC_REQUIRE(src && dst && rows >= 0 && cols > 0 && ld >= cols && terms >= 1, "bad sum_terms arguments");
  if (rows == 0) return MOC_OK;
  long long blocks = (rows * cols + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  sum_terms_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream_)>>>(src, bias, dst, rows, cols,
                                                                                             ld, terms);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_col_sum(const float* x, float* out, int64_t rows, int32_t cols, void* stream_) {
  MOC_REQUIRE(x && out && rows > 0 && cols > 0, "bad column-sum arguments");
  col_sum_kernel<<<ceil_div(cols, 32), 256, 0, static_cast<cudaStream_t>(stream_)>>>(x, out, rows, cols);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}
