// Chapter gather (selected chapters -> per-batch memory rows), optional per-row normalisation and
// router-weight scaling, and the backward that writes gradients only for touched chapters.
// All kernels are HBM bound: one warp per 1-D row, vector accesses where alignment allows.
#include <math.h>

#include "moc_common.cuh"

namespace moc {
namespace {

template <typename T> __device__ __forceinline__ float ld(const T* p, long long i);
template <> __device__ __forceinline__ float ld<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <typename T> __device__ __forceinline__ void st(T* p, long long i, float v);
template <> __device__ __forceinline__ void st<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) {
  p[i] = __float2bfloat16(v);
}

// 8 consecutive elements (16-byte aligned for bf16, 32-byte for fp32)
__device__ __forceinline__ void ld8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void st8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// Streaming forms (evict-first in L2) for data that is read or written exactly once -- the exchange's consumer runs
// beside the next step's attention kernels, whose K/V tiles live on L2 hits.
__device__ __forceinline__ void ld8_stream(const float* p, float (&v)[8]) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ld8_stream(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void st8_stream(float* p, const float (&v)[8]) {
  __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
  __stcs(reinterpret_cast<float4*>(p + 4), make_float4(v[4], v[5], v[6], v[7]));
}
__device__ __forceinline__ void st8_stream(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
  __stcs(reinterpret_cast<uint4*>(p), o);
}

// statistics of one bank row as the normalisation needs them: {mean, 1/sqrt(var or meansq + eps)}
template <typename TB>
__device__ __forceinline__ void row_norm_stats(const TB* row, int dim, int norm_type, float eps, int lane,
                                               float& mean, float& rinv) {
  mean = 0.f;
  rinv = 1.f;
  if (norm_type == MOC_NORM_NONE) return;
  if (norm_type == MOC_NORM_LAYERNORM) {
    float s = 0.f;
    for (int c = lane; c < dim; c += 32) s += ld(row, c);
    mean = warp_sum(s) / static_cast<float>(dim);
  }
  float s2 = 0.f;
  for (int c = lane; c < dim; c += 32) {
    const float v = ld(row, c) - mean;
    s2 += v * v;
  }
  s2 = warp_sum(s2) / static_cast<float>(dim);
  rinv = 1.f / sqrtf(s2 + eps);
}

template <typename TB, typename TO>
__global__ void gather_rows_kernel(const TB* __restrict__ bank, long long bank_rows, int dim, int T,
                                   const int* __restrict__ comb_idx, const float* __restrict__ comb_w,
                                   long long n_rows, int norm_type, float eps, TO* __restrict__ out,
                                   float* __restrict__ row_stats, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  if (r >= n_rows) return;
  const long long pair = r / T;
  const int within = static_cast<int>(r - pair * T);
  const long long chapter = comb_idx[pair];
  const long long src = chapter * T + within;
  TO* dst = out + r * dim;
  if (chapter < 0 || src >= bank_rows) {
    if (lane == 0) atomicMax(status, MOC_DEV_BAD_INDEX);
    for (int c = lane; c < dim; c += 32) st(dst, c, 0.f);
    return;
  }
  const TB* row = bank + src * dim;
  float mean, rinv;
  row_norm_stats(row, dim, norm_type, eps, lane, mean, rinv);
  if (norm_type != MOC_NORM_NONE && row_stats != nullptr && lane == 0) {
    row_stats[r * 2] = mean;
    row_stats[r * 2 + 1] = rinv;
  }
  const float w = comb_w ? comb_w[pair] : 1.f;
  if ((dim & 7) == 0) {
    for (int c = lane * 8; c < dim; c += 256) {
      float v[8];
      ld8(row + c, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (v[i] - mean) * rinv * w;
      st8(dst + c, v);
    }
  } else {
    for (int c = lane; c < dim; c += 32) st(dst, c, (ld(row, c) - mean) * rinv * w);
  }
}

// Groups (batch, slot) pairs by chapter id.  Single CTA.
__global__ void __launch_bounds__(1024)
chapter_segments_kernel(const int* __restrict__ comb_idx, int n_pairs, int C, int* __restrict__ uniq,
                        int* __restrict__ seg_offsets, int* __restrict__ seg_pairs,
                        int* __restrict__ pair_to_uniq, int* __restrict__ num_unique, int* __restrict__ status) {
  extern __shared__ int sh[];          // count[C], then start[C], urank[C]
  int* count = sh;
  int* start = sh + C;
  int* urank = sh + 2 * C;
  __shared__ int warp_tot[2][32];
  for (int c = threadIdx.x; c < C; c += blockDim.x) count[c] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int c = comb_idx[i];
    if (c < 0 || c >= C) atomicMax(status, MOC_DEV_BAD_INDEX);
    else atomicAdd(&count[c], 1);
  }
  __syncthreads();
  // exclusive scans of count[] and (count[] > 0), each thread owning a contiguous span
  const int per = (C + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * per, hi = min(C, lo + per);
  int s0 = 0, s1 = 0;
  for (int c = lo; c < hi; ++c) { s0 += count[c]; s1 += (count[c] > 0); }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int i0 = s0, i1 = s1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t0 = __shfl_up_sync(0xffffffffu, i0, o), t1 = __shfl_up_sync(0xffffffffu, i1, o);
    if (lane >= o) { i0 += t0; i1 += t1; }
  }
  if (lane == 31) { warp_tot[0][warp] = i0; warp_tot[1][warp] = i1; }
  __syncthreads();
  if (warp == 0) {
    int w0 = warp_tot[0][lane], w1 = warp_tot[1][lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t0 = __shfl_up_sync(0xffffffffu, w0, o), t1 = __shfl_up_sync(0xffffffffu, w1, o);
      if (lane >= o) { w0 += t0; w1 += t1; }
    }
    warp_tot[0][lane] = w0; warp_tot[1][lane] = w1;   // inclusive
  }
  __syncthreads();
  int e0 = i0 - s0 + (warp > 0 ? warp_tot[0][warp - 1] : 0);
  int e1 = i1 - s1 + (warp > 0 ? warp_tot[1][warp - 1] : 0);
  for (int c = lo; c < hi; ++c) {
    start[c] = e0; urank[c] = e1;
    if (count[c] > 0) { uniq[e1] = c; seg_offsets[e1] = e0; }
    e0 += count[c]; e1 += (count[c] > 0);
  }
  __syncthreads();
  const int U = warp_tot[1][31];
  if (threadIdx.x == 0) { num_unique[0] = U; seg_offsets[U] = warp_tot[0][31]; }
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int c = comb_idx[i];
    if (c < 0 || c >= C) { pair_to_uniq[i] = -1; continue; }
    int pos = 0;
    for (int j = 0; j < i; ++j) pos += (comb_idx[j] == c);
    seg_pairs[start[c] + pos] = i;
    pair_to_uniq[i] = urank[c];
  }
}

// Union of the ranks' chapter lists (rank r holds counts[r] distinct ids in ids_all[r, :]).  One small CTA, linear
// in the number of entries: a bit mask per chapter says which ranks hold it; a chapter's contributions are ordered
// by rank, so an entry's place inside its chapter is the number of lower ranks holding the same chapter.
// Shared memory: mask[C] (which ranks), then packed[C] = (first pair slot << 16) | union rank  (entries <= 65535).
__global__ void __launch_bounds__(256)
union_segments_kernel(const int* __restrict__ ids_all, const int* __restrict__ counts, int world, int per_rank,
                      int C, int* __restrict__ uniq, int* __restrict__ seg_offsets, int* __restrict__ seg_pairs,
                      int* __restrict__ pair_to_uniq, int* __restrict__ num_unique, int* __restrict__ status) {
  extern __shared__ unsigned int ush[];
  unsigned int* mask = ush;
  unsigned int* packed = ush + C;
  __shared__ int warp_tot[2][8];
  const int n_pairs = world * per_rank;
  for (int c = threadIdx.x; c < C; c += blockDim.x) mask[c] = 0u;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int r = i / per_rank;
    if (i - r * per_rank >= counts[r]) continue;
    const int c = ids_all[i];
    if (c < 0 || c >= C) atomicMax(status, MOC_DEV_BAD_INDEX);
    else atomicOr(&mask[c], 1u << r);
  }
  __syncthreads();
  const int per = (C + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * per, hi = min(C, lo + per);
  int s0 = 0, s1 = 0;
  for (int c = lo; c < hi; ++c) { s0 += __popc(mask[c]); s1 += (mask[c] != 0u); }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int i0 = s0, i1 = s1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t0 = __shfl_up_sync(0xffffffffu, i0, o), t1 = __shfl_up_sync(0xffffffffu, i1, o);
    if (lane >= o) { i0 += t0; i1 += t1; }
  }
  if (lane == 31) { warp_tot[0][warp] = i0; warp_tot[1][warp] = i1; }
  __syncthreads();
  int b0 = 0, b1 = 0, tot0 = 0, tot1 = 0;
  for (int w = 0; w < 8; ++w) {
    if (w < warp) { b0 += warp_tot[0][w]; b1 += warp_tot[1][w]; }
    tot0 += warp_tot[0][w]; tot1 += warp_tot[1][w];
  }
  int e0 = i0 - s0 + b0, e1 = i1 - s1 + b1;
  for (int c = lo; c < hi; ++c) {
    packed[c] = (static_cast<unsigned int>(e0) << 16) | static_cast<unsigned int>(e1);
    if (mask[c] != 0u) { uniq[e1] = c; seg_offsets[e1] = e0; }
    e0 += __popc(mask[c]); e1 += (mask[c] != 0u);
  }
  __syncthreads();
  if (threadIdx.x == 0) { num_unique[0] = tot1; seg_offsets[tot1] = tot0; }
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int r = i / per_rank;
    const int c = (i - r * per_rank < counts[r]) ? ids_all[i] : -1;
    if (c < 0 || c >= C) { pair_to_uniq[i] = -1; continue; }
    const unsigned int pk = packed[c];
    seg_pairs[(pk >> 16) + __popc(mask[c] & ((1u << r) - 1u))] = i;
    pair_to_uniq[i] = static_cast<int>(pk & 0xFFFFu);
  }
}

// Sum of the ranks' compact gradient rows over the union of their chapter lists: one warp per output row;
// the contributions of a chapter are added in ascending (rank, slot) order, so every rank computes the same bits.
struct RankRows { const void* p[16]; };
template <typename TR, typename TO>
__global__ void union_sum_kernel(RankRows src, int per_list, int T, int dim, const int* __restrict__ seg_offsets,
                                 const int* __restrict__ seg_pairs, const int* __restrict__ num_unique,
                                 long long max_rows, float scale, TO* __restrict__ out) {
  // grid-stride over the output rows, one warp per row
  const int lane = threadIdx.x & 31;
  const long long n_rows = min(max_rows, static_cast<long long>(num_unique[0]) * T);
  const long long stride = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; r < n_rows; r += stride) {
    const int u = static_cast<int>(r / T);
    const int within = static_cast<int>(r - static_cast<long long>(u) * T);
    const int p0 = seg_offsets[u], p1 = seg_offsets[u + 1];
    TO* dst = out + r * dim;
    if ((dim & 7) == 0) {
      for (int c = lane * 8; c < dim; c += 256) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int q = p0; q < p1; ++q) {
          const int pair = seg_pairs[q];
          const TR* rows = static_cast<const TR*>(src.p[pair / per_list]);
          float g[8];
          ld8_stream(rows + (static_cast<long long>(pair % per_list) * T + within) * dim + c, g);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += g[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= scale;
        st8_stream(dst + c, acc);
      }
      continue;
    }
    for (int c = lane; c < dim; c += 32) {
      float acc = 0.f;
      for (int q = p0; q < p1; ++q) {
        const int pair = seg_pairs[q];
        const TR* rows = static_cast<const TR*>(src.p[pair / per_list]);
        acc += ld(rows + (static_cast<long long>(pair % per_list) * T + within) * dim, c);
      }
      st(dst, c, acc * scale);
    }
  }
}

// d_comb_w[pair] = sum over the pair's rows of <d_mem row, normalised bank row>; one CTA per pair
template <typename TG, typename TB>
__global__ void dcombw_kernel(const TG* __restrict__ d_mem, const TB* __restrict__ bank, long long bank_rows,
                              int dim, int T, const int* __restrict__ comb_idx,
                              const float* __restrict__ row_stats, int norm_type,
                              float* __restrict__ d_comb_w) {
  __shared__ float red[32];
  const long long pair = blockIdx.x;
  const long long chapter = comb_idx[pair];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float acc = 0.f;
  if (chapter >= 0 && (chapter + 1) * T <= bank_rows) {
    if ((dim & 7) == 0) {
      const int per_row = dim >> 3;
      const int total = T * per_row;
      for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int r = i / per_row, c = (i - r * per_row) << 3;
        const long long orow = pair * T + r;
        float g[8], x[8];
        ld8(d_mem + orow * dim + c, g);
        ld8(bank + (chapter * T + r) * dim + c, x);
        float mean = 0.f, rinv = 1.f;
        if (norm_type != MOC_NORM_NONE) { mean = row_stats[orow * 2]; rinv = row_stats[orow * 2 + 1]; }
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) a = fmaf(g[j], x[j] - mean, a);
        acc = fmaf(a, rinv, acc);
      }
    } else {
      for (int r = warp; r < T; r += nw) {
        const long long orow = pair * T + r;
        const TB* row = bank + (chapter * T + r) * dim;
        const TG* g = d_mem + orow * dim;
        float mean = 0.f, rinv = 1.f;
        if (norm_type != MOC_NORM_NONE) { mean = row_stats[orow * 2]; rinv = row_stats[orow * 2 + 1]; }
        for (int c = lane; c < dim; c += 32) acc += ld(g, c) * (ld(row, c) - mean) * rinv;
      }
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) d_comb_w[pair] = t;
  }
}

// compact bank gradient: one warp per (unique chapter, row)
template <typename TG, typename TB>
__global__ void bank_grad_kernel(const TG* __restrict__ d_mem, const TB* __restrict__ bank, int dim, int T,
                                 const float* __restrict__ comb_w, const float* __restrict__ row_stats,
                                 int norm_type, const int* __restrict__ uniq,
                                 const int* __restrict__ seg_offsets, const int* __restrict__ seg_pairs,
                                 const int* __restrict__ num_unique, long long max_rows,
                                 float* __restrict__ bank_grad, __nv_bfloat16* __restrict__ bank_grad_wire) {
  const int lane = threadIdx.x & 31;
  const long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  if (r >= max_rows) return;
  const int u = static_cast<int>(r / T);
  if (u >= num_unique[0]) return;
  const int within = static_cast<int>(r - static_cast<long long>(u) * T);
  const int p0 = seg_offsets[u], p1 = seg_offsets[u + 1];
  float* dst = bank_grad + r * dim;
  // optional second copy in bf16: what travels between ranks when the exchange is asked to halve its volume
  __nv_bfloat16* wire = bank_grad_wire ? bank_grad_wire + r * dim : nullptr;
  if (norm_type == MOC_NORM_NONE && (dim & 7) == 0) {
    for (int c = lane * 8; c < dim; c += 256) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int q = p0; q < p1; ++q) {
        const long long pair = seg_pairs[q];
        const float w = comb_w ? comb_w[pair] : 1.f;
        float g[8];
        ld8(d_mem + (pair * T + within) * dim + c, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, g[j], acc[j]);
      }
      st8(dst + c, acc);
      if (wire) st8(wire + c, acc);
    }
    return;
  }
  if (norm_type == MOC_NORM_NONE) {
    for (int c = lane; c < dim; c += 32) {
      float acc = 0.f;
      for (int q = p0; q < p1; ++q) {
        const long long pair = seg_pairs[q];
        acc = fmaf(comb_w ? comb_w[pair] : 1.f, ld(d_mem + (pair * T + within) * dim, c), acc);
      }
      dst[c] = acc;
      if (wire) wire[c] = __float2bfloat16(acc);
    }
    return;
  }
  // normalised rows: g = sum_p w_p * d_mem_p is the gradient of y; push it through the row norm
  const long long chapter = uniq[u];
  const TB* row = bank + (chapter * T + within) * dim;
  const long long first = static_cast<long long>(seg_pairs[p0]) * T + within;
  const float mean = row_stats[first * 2], rinv = row_stats[first * 2 + 1];
  float sg = 0.f, sgy = 0.f;
  for (int c = lane; c < dim; c += 32) {
    float acc = 0.f;
    for (int q = p0; q < p1; ++q) {
      const long long pair = seg_pairs[q];
      acc = fmaf(comb_w ? comb_w[pair] : 1.f, ld(d_mem + (pair * T + within) * dim, c), acc);
    }
    dst[c] = acc;
    sg += acc;
    sgy += acc * (ld(row, c) - mean) * rinv;
  }
  sg = warp_sum(sg) / static_cast<float>(dim);
  sgy = warp_sum(sgy) / static_cast<float>(dim);
  if (norm_type == MOC_NORM_RMS) sg = 0.f;
  __syncwarp();
  for (int c = lane; c < dim; c += 32) {
    const float y = (ld(row, c) - mean) * rinv;
    const float v = rinv * (dst[c] - sg - y * sgy);
    dst[c] = v;
    if (wire) wire[c] = __float2bfloat16(v);
  }
}

// ---- fused gather-and-project path: no gathered rows are materialised in the forward pass --------------------
// K = s_r * (bank_row W^T) with s_r = u~[pair] (* 1/rms of the bank row): the forward reads the bank through the TMA
// gather list and applies s_r in the projection epilogue.  Its backward works from g'_r = s_r * dM~_r (the dK/dV
// kernel scales its output rows by s_r before the memory-row projection):
//   d u~[pair] = (1 / u~[pair]) * sum_r <g'_r, m_r>            (both without and with the rms norm)
//   d m_r      = G_r - m_r * inv_rms_r^2 * <G_r, m_r> / dim    with G_r = sum over the pairs of the chapter of g'_r
//                (second term only with the rms norm)

// inv_rms[row] = 1 / sqrt(mean(row^2) + eps) for every bank row; one warp per row
template <typename TB>
__global__ void row_inv_rms_kernel(const TB* __restrict__ bank, long long rows, int dim, float eps,
                                   float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  if (r >= rows) return;
  const TB* row = bank + r * dim;
  float acc = 0.f;
  for (int c = lane; c < dim; c += 32) { const float x = ld(row, c); acc = fmaf(x, x, acc); }
  acc = warp_sum(acc);
  if (lane == 0) out[r] = rsqrtf(acc / static_cast<float>(dim) + eps);
}
// scale[pair * T + r] = comb_w[pair] * (inv_rms ? inv_rms[comb_idx[pair] * T + r] : 1)
__global__ void row_scale_kernel(const int* __restrict__ comb_idx, const float* __restrict__ comb_w,
                                 const float* __restrict__ inv_rms, long long bank_rows, int n_pairs, int T,
                                 float* __restrict__ scale, int* __restrict__ status) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= static_cast<long long>(n_pairs) * T) return;
  const int pair = static_cast<int>(i / T), r = static_cast<int>(i - static_cast<long long>(pair) * T);
  const long long c = comb_idx[pair];
  float v = comb_w ? comb_w[pair] : 1.f;
  if (c < 0 || (c + 1) * T > bank_rows) { atomicMax(status, MOC_DEV_BAD_INDEX); v = 0.f; }
  else if (inv_rms) v *= inv_rms[c * T + r];
  scale[i] = v;
}
template <typename TG, typename TB>
__global__ void dcombw_prescaled_kernel(const TG* __restrict__ g, const TB* __restrict__ bank, long long bank_rows,
                                        int dim, int T, const int* __restrict__ comb_idx,
                                        const float* __restrict__ comb_w, float* __restrict__ d_comb_w) {
  __shared__ float red[32];
  const long long pair = blockIdx.x;
  const long long chapter = comb_idx[pair];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float acc = 0.f;
  if (chapter >= 0 && (chapter + 1) * T <= bank_rows) {
    if ((dim & 7) == 0) {
      const int per_row = dim >> 3;
      for (int i = threadIdx.x; i < T * per_row; i += blockDim.x) {
        const int r = i / per_row, c = (i - r * per_row) << 3;
        float gv[8], x[8];
        ld8(g + (pair * T + r) * dim + c, gv);
        ld8(bank + (chapter * T + r) * dim + c, x);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(gv[j], x[j], acc);
      }
    } else {
      for (int r = warp; r < T; r += nw)
        for (int c = lane; c < dim; c += 32)
          acc += ld(g + (pair * T + r) * dim, c) * ld(bank + (chapter * T + r) * dim, c);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) {
      const float u = comb_w ? comb_w[pair] : 1.f;
      d_comb_w[pair] = (fabsf(u) > 1e-30f) ? t / u : 0.f;
    }
  }
}
template <typename TG, typename TB>
__global__ void bank_grad_prescaled_kernel(const TG* __restrict__ g, const TB* __restrict__ bank, int dim, int T,
                                           const float* __restrict__ inv_rms, const int* __restrict__ uniq,
                                           const int* __restrict__ seg_offsets, const int* __restrict__ seg_pairs,
                                           const int* __restrict__ num_unique, long long max_rows,
                                           float* __restrict__ bank_grad, __nv_bfloat16* __restrict__ bank_grad_wire) {
  const int lane = threadIdx.x & 31;
  const long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  if (r >= max_rows) return;
  const int u = static_cast<int>(r / T);
  if (u >= num_unique[0]) return;
  const int within = static_cast<int>(r - static_cast<long long>(u) * T);
  const int p0 = seg_offsets[u], p1 = seg_offsets[u + 1];
  // bank_grad may be NULL when only the bf16 rows are wanted (a data-parallel step whose mean gradient is formed
  // from the ranks' bf16 rows): the vector path below then skips the fp32 store
  float* dst = bank_grad ? bank_grad + r * dim : nullptr;
  __nv_bfloat16* wire = bank_grad_wire ? bank_grad_wire + r * dim : nullptr;
  const long long brow = static_cast<long long>(uniq[u]) * T + within;
  const TB* row = bank + brow * dim;
  if ((dim & 7) == 0 && dim <= 8 * 32 * 4) {
    // 16-byte accesses: lane l owns columns [8 l + 256 n, +8); the sums stay in registers for the norm term
    float acc[4][8];
    float sgm = 0.f;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int c = lane * 8 + n * 256;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[n][j] = 0.f;
      if (c < dim) {
        for (int q = p0; q < p1; ++q) {
          float gv[8];
          ld8(g + (static_cast<long long>(seg_pairs[q]) * T + within) * dim + c, gv);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[n][j] += gv[j];
        }
        if (inv_rms) {
          float x[8];
          ld8(row + c, x);
#pragma unroll
          for (int j = 0; j < 8; ++j) sgm = fmaf(acc[n][j], x[j], sgm);
        }
      }
    }
    float k = 0.f;
    if (inv_rms) {
      const float ir = inv_rms[brow];
      k = warp_sum(sgm) * ir * ir / static_cast<float>(dim);
    }
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int c = lane * 8 + n * 256;
      if (c < dim) {
        if (inv_rms) {
          float x[8];
          ld8(row + c, x);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[n][j] -= x[j] * k;
        }
        if (dst) st8(dst + c, acc[n]);
        if (wire) st8(wire + c, acc[n]);
      }
    }
    return;
  }
  float sgm = 0.f;
  for (int c = lane; c < dim; c += 32) {
    float acc = 0.f;
    for (int q = p0; q < p1; ++q) acc += ld(g + (static_cast<long long>(seg_pairs[q]) * T + within) * dim, c);
    dst[c] = acc;
    if (inv_rms) sgm = fmaf(acc, ld(row, c), sgm);
  }
  if (inv_rms == nullptr) {
    if (wire) { __syncwarp(); for (int c = lane; c < dim; c += 32) wire[c] = __float2bfloat16(dst[c]); }
    return;
  }
  const float ir = inv_rms[brow];
  const float k = warp_sum(sgm) * ir * ir / static_cast<float>(dim);
  __syncwarp();
  for (int c = lane; c < dim; c += 32) {
    const float v = dst[c] - ld(row, c) * k;
    dst[c] = v;
    if (wire) wire[c] = __float2bfloat16(v);
  }
}

__global__ void scatter_bank_grad_kernel(const float* __restrict__ bank_grad, const int* __restrict__ uniq,
                                         const int* __restrict__ num_unique, long long max_rows, int T, int dim,
                                         float* __restrict__ dense, long long bank_rows) {
  const int lane = threadIdx.x & 31;
  const long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  if (r >= max_rows) return;
  const int u = static_cast<int>(r / T);
  if (u >= num_unique[0]) return;
  const long long row = static_cast<long long>(uniq[u]) * T + (r - static_cast<long long>(u) * T);
  if (row < 0 || row >= bank_rows) return;
  for (int c = lane; c < dim; c += 32) dense[row * dim + c] += bank_grad[r * dim + c];
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16(src[i]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __bfloat162float(src[i]);
}

// dst[c, r] = src[r, c] with dtype conversion; 32 x 32 tiles through shared memory
template <typename TS, typename TD>
__global__ void transpose_kernel(const TS* __restrict__ src, TD* __restrict__ dst, int rows, int cols) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (r < rows && c < cols) ? ld(src, static_cast<long long>(r) * cols + c) : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (c < cols && r < rows) st(dst, static_cast<long long>(c) * rows + r, tile[threadIdx.x][i]);
  }
}

// Up to four row-major matrices converted in one launch: dst[i] = src[i] in the output dtype and, when
// dst_t[i] is given, dst_t[i] = src[i]^T.  blockIdx.z selects the matrix.
struct PackJob { const void* src; void* dst; void* dst_t; int rows, cols, ldt; };
struct PackJobs { PackJob j[4]; int n; };
template <typename TS>
__global__ void pack_weights_kernel(PackJobs jobs) {
  const PackJob jb = jobs.j[blockIdx.z];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  if (r0 >= jb.rows || c0 >= jb.cols) return;
  __shared__ float tile[32][33];
  const TS* src = static_cast<const TS*>(jb.src);
  __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(jb.dst);
  __nv_bfloat16* dst_t = static_cast<__nv_bfloat16*>(jb.dst_t);
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    float v = 0.f;
    if (r < jb.rows && c < jb.cols) {
      v = ld(src, static_cast<long long>(r) * jb.cols + c);
      if (dst != nullptr) dst[static_cast<long long>(r) * jb.cols + c] = __float2bfloat16(v);
    }
    tile[i][threadIdx.x] = v;
  }
  if (dst_t == nullptr) return;
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (c < jb.cols && r < jb.rows) dst_t[static_cast<long long>(c) * jb.ldt + r] = __float2bfloat16(tile[threadIdx.x][i]);
  }
}

inline int grid_for(long long n, int per_block) {
  long long g = (n + per_block - 1) / per_block;
  const long long cap = 148LL * 32;
  return static_cast<int>(g < cap ? (g > 0 ? g : 1) : cap);
}

}  // namespace
}  // namespace moc

using namespace moc;

extern "C" int moc_gather_rows_fwd(const void* bank, int32_t bank_dtype, int64_t bank_rows, int32_t dim,
                                   int32_t T, const int32_t* comb_idx, const float* comb_w, int32_t batch,
                                   int32_t k_sel, int32_t norm_type, float eps, void* out, int32_t out_dtype,
                                   float* row_stats, int32_t* status, void* stream_) {
  MOC_REQUIRE(bank && comb_idx && out && status, "NULL gather buffer");
  MOC_REQUIRE(dim > 0 && T > 0 && batch > 0 && k_sel > 0, "empty gather");
  MOC_REQUIRE(norm_type >= 0 && norm_type <= 2, "bad norm_type");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long n_rows = static_cast<long long>(batch) * k_sel * T;
  const int blocks = static_cast<int>((n_rows * 32 + 255) / 256);
#define MOC_GATHER(TB, TO)                                                                                  \
  gather_rows_kernel<TB, TO><<<blocks, 256, 0, stream>>>(static_cast<const TB*>(bank), bank_rows, dim, T,   \
                                                         comb_idx, comb_w, n_rows, norm_type, eps,          \
                                                         static_cast<TO*>(out), row_stats, status)
  if (bank_dtype == MOC_F32 && out_dtype == MOC_F32) MOC_GATHER(float, float);
  else if (bank_dtype == MOC_F32 && out_dtype == MOC_BF16) MOC_GATHER(float, __nv_bfloat16);
  else if (bank_dtype == MOC_BF16 && out_dtype == MOC_BF16) MOC_GATHER(__nv_bfloat16, __nv_bfloat16);
  else if (bank_dtype == MOC_BF16 && out_dtype == MOC_F32) MOC_GATHER(__nv_bfloat16, float);
  else MOC_REQUIRE(false, "bad dtype");
#undef MOC_GATHER
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_chapter_segments(const int32_t* comb_idx, int32_t n_pairs, int32_t num_chapters,
                                    int32_t* uniq, int32_t* seg_offsets, int32_t* seg_pairs,
                                    int32_t* pair_to_uniq, int32_t* num_unique, int32_t* status, void* stream_) {
  MOC_REQUIRE(comb_idx && uniq && seg_offsets && seg_pairs && pair_to_uniq && num_unique && status, "NULL buffer");
  MOC_REQUIRE(n_pairs > 0 && n_pairs <= 65536, "n_pairs out of range");
  MOC_REQUIRE(num_chapters > 0 && static_cast<size_t>(num_chapters) * 12 <= 200 * 1024, "num_chapters too large");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const size_t sm = static_cast<size_t>(num_chapters) * 12;
  MOC_CUDA_OK(cudaFuncSetAttribute(chapter_segments_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm)));
  chapter_segments_kernel<<<1, 1024, sm, stream>>>(comb_idx, n_pairs, num_chapters, uniq, seg_offsets, seg_pairs,
                                                   pair_to_uniq, num_unique, status);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_bank_grad_merge_to(const void* const* rank_rows, int32_t rows_dtype, int32_t world,
                                      const int32_t* ids_all, const int32_t* counts, int32_t per_rank, int32_t T,
                                      int32_t dim, int32_t num_chapters, float scale, int32_t* uniq,
                                      int32_t* seg_offsets, int32_t* seg_pairs, int32_t* pair_to_uniq,
                                      int32_t* num_unique, void* rows_out, int32_t rows_out_dtype,
                                      int64_t rows_out_capacity, int32_t* status, void* stream_) {
  MOC_REQUIRE(rows_out_dtype == MOC_F32 || rows_out_dtype == MOC_BF16, "bad rows_out_dtype");
  MOC_REQUIRE(rank_rows && ids_all && counts && uniq && seg_offsets && seg_pairs && pair_to_uniq && num_unique &&
              rows_out && status, "NULL buffer");
  MOC_REQUIRE(world >= 1 && world <= 16, "world size must be in [1, 16]");
  MOC_REQUIRE(per_rank > 0 && T > 0 && dim > 0, "empty lists");
  MOC_REQUIRE(rows_dtype == MOC_F32 || rows_dtype == MOC_BF16, "bad rows_dtype");
  const int n_pairs = world * per_rank;
  MOC_REQUIRE(n_pairs <= 65535, "too many list entries");
  MOC_REQUIRE(num_chapters > 0 && num_chapters <= 65535 && static_cast<size_t>(num_chapters) * 8 <= 200 * 1024,
              "num_chapters too large");
  const long long cap = n_pairs < num_chapters ? n_pairs : num_chapters;     // the union cannot be larger
  MOC_REQUIRE(rows_out_capacity >= cap * T, "rows_out too small for the largest possible union");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const size_t sm = static_cast<size_t>(num_chapters) * 8;
  MOC_CUDA_OK(cudaFuncSetAttribute(union_segments_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm)));
  union_segments_kernel<<<1, 256, sm, stream>>>(ids_all, counts, world, per_rank, num_chapters, uniq, seg_offsets,
                                                seg_pairs, pair_to_uniq, num_unique, status);
  RankRows src;
  for (int r = 0; r < 16; ++r) src.p[r] = r < world ? rank_rows[r] : nullptr;
  for (int r = 0; r < world; ++r) MOC_REQUIRE(src.p[r] != nullptr, "NULL rank rows");
  const long long max_rows = cap * T;
  // one warp per output row over the whole grid: capping the grid at 1-4 CTAs per SM (a smaller footprint beside
  // the next step's compute) measured no better at two GPUs (1.246 ms per step uncapped, 1.259-1.267 capped)
  const long long blocks = (max_rows * 32 + 255) / 256;
#define MOC_USUM(TR, TO)                                                                                     \
  union_sum_kernel<TR, TO><<<static_cast<int>(blocks), 256, 0, stream>>>(src, per_rank, T, dim, seg_offsets,   \
                                                                         seg_pairs, num_unique, max_rows, scale, \
                                                                         static_cast<TO*>(rows_out))
  if (rows_dtype == MOC_F32 && rows_out_dtype == MOC_F32) MOC_USUM(float, float);
  else if (rows_dtype == MOC_F32) MOC_USUM(float, __nv_bfloat16);
  else if (rows_out_dtype == MOC_F32) MOC_USUM(__nv_bfloat16, float);
  else MOC_USUM(__nv_bfloat16, __nv_bfloat16);
#undef MOC_USUM
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_bank_grad_merge(const void* const* rank_rows, int32_t rows_dtype, int32_t world,
                                   const int32_t* ids_all, const int32_t* counts, int32_t per_rank, int32_t T,
                                   int32_t dim, int32_t num_chapters, float scale, int32_t* uniq,
                                   int32_t* seg_offsets, int32_t* seg_pairs, int32_t* pair_to_uniq,
                                   int32_t* num_unique, float* rows_out, int64_t rows_out_capacity,
                                   int32_t* status, void* stream_) {
  return moc_bank_grad_merge_to(rank_rows, rows_dtype, world, ids_all, counts, per_rank, T, dim, num_chapters, scale,
                                uniq, seg_offsets, seg_pairs, pair_to_uniq, num_unique, rows_out, MOC_F32,
                                rows_out_capacity, status, stream_);
}

extern "C" int moc_gather_rows_bwd(const void* d_mem, int32_t d_mem_dtype, const void* bank, int32_t bank_dtype,
                                   int64_t bank_rows, int32_t dim, int32_t T, const int32_t* comb_idx,
                                   const float* comb_w, int32_t batch, int32_t k_sel, int32_t norm_type,
                                   float eps, const float* row_stats, const int32_t* uniq,
                                   const int32_t* seg_offsets, const int32_t* seg_pairs,
                                   const int32_t* num_unique, float* d_comb_w, float* bank_grad,
                                   void* bank_grad_bf16, int32_t* status, void* stream_) {
  (void)eps; (void)status;
  MOC_REQUIRE(d_mem && bank && comb_idx && uniq && seg_offsets && seg_pairs && num_unique, "NULL buffer");
  MOC_REQUIRE(norm_type == MOC_NORM_NONE || row_stats != nullptr, "row_stats needed for normalised rows");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int n_pairs = batch * k_sel;
  const long long max_rows = static_cast<long long>(n_pairs) * T;
  const int blocks = static_cast<int>((max_rows * 32 + 255) / 256);
#define MOC_GBWD(TG, TB)                                                                                      \
  do {                                                                                                        \
    if (d_comb_w != nullptr)                                                                                  \
      dcombw_kernel<TG, TB><<<n_pairs, 256, 0, stream>>>(static_cast<const TG*>(d_mem),                       \
                                                         static_cast<const TB*>(bank), bank_rows, dim, T,     \
                                                         comb_idx, row_stats, norm_type, d_comb_w);           \
    if (bank_grad != nullptr)                                                                                 \
      bank_grad_kernel<TG, TB><<<blocks, 256, 0, stream>>>(static_cast<const TG*>(d_mem),                     \
                                                           static_cast<const TB*>(bank), dim, T, comb_w,      \
                                                           row_stats, norm_type, uniq, seg_offsets,           \
                                                           seg_pairs, num_unique, max_rows, bank_grad,        \
                                                           static_cast<__nv_bfloat16*>(bank_grad_bf16));      \
  } while (0)
  if (d_mem_dtype == MOC_F32 && bank_dtype == MOC_F32) MOC_GBWD(float, float);
  else if (d_mem_dtype == MOC_F32 && bank_dtype == MOC_BF16) MOC_GBWD(float, __nv_bfloat16);
  else if (d_mem_dtype == MOC_BF16 && bank_dtype == MOC_F32) MOC_GBWD(__nv_bfloat16, float);
  else if (d_mem_dtype == MOC_BF16 && bank_dtype == MOC_BF16) MOC_GBWD(__nv_bfloat16, __nv_bfloat16);
  else MOC_REQUIRE(false, "bad dtype");
#undef MOC_GBWD
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_scatter_bank_grad(const float* bank_grad, const int32_t* uniq, const int32_t* num_unique,
                                     int32_t max_unique, int32_t T, int32_t dim, float* bank_dense,
                                     int64_t bank_rows, int32_t* status, void* stream_) {
  (void)status;
  MOC_REQUIRE(bank_grad && uniq && num_unique && bank_dense, "NULL buffer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long max_rows = static_cast<long long>(max_unique) * T;
  const int blocks = static_cast<int>((max_rows * 32 + 255) / 256);
  scatter_bank_grad_kernel<<<blocks, 256, 0, stream>>>(bank_grad, uniq, num_unique, max_rows, T, dim, bank_dense,
                                                       bank_rows);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_cast_f32_to_bf16(const float* src, void* dst, int64_t n, void* stream_) {
  MOC_REQUIRE(src && dst && n >= 0, "bad cast arguments");
  if (n == 0) return MOC_OK;
  cast_f32_bf16_kernel<<<grid_for(n, 256 * 8), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      src, static_cast<__nv_bfloat16*>(dst), n);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}
extern "C" int moc_cast_bf16_to_f32(const void* src, float* dst, int64_t n, void* stream_) {
  MOC_REQUIRE(src && dst && n >= 0, "bad cast arguments");
  if (n == 0) return MOC_OK;
  cast_bf16_f32_kernel<<<grid_for(n, 256 * 8), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const __nv_bfloat16*>(src), dst, n);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

// x = t0 + t1 + t2 (+ rounding below 2^-24 |x|): successive bf16 roundings of the residual.  Products of the terms
// with bf16 operands are exact in fp32, so sums of tensor-core products over the terms reach fp32-grade accuracy.
__global__ void split_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n,
                                  int terms) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  float r = src[i];
  for (int t = 0; t < terms; ++t) {
    const __nv_bfloat16 b = __float2bfloat16_rn(r);
    dst[t * n + i] = b;
    r -= __bfloat162float(b);
  }
}
extern "C" int moc_split_bf16(const float* src, void* dst, int64_t n, int32_t terms, void* stream_) {
  MOC_REQUIRE(src && dst && n >= 0 && terms >= 1 && terms <= 3, "bad split arguments");
  if (n == 0) return MOC_OK;
  split_bf16_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      src, static_cast<__nv_bfloat16*>(dst), n, terms);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_transpose(const void* src, int32_t src_dtype, void* dst, int32_t dst_dtype, int32_t rows,
                             int32_t cols, void* stream_) {
  MOC_REQUIRE(src && dst && rows > 0 && cols > 0, "bad transpose arguments");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  dim3 grid(ceil_div(cols, 32), ceil_div(rows, 32)), block(32, 8);
  if (src_dtype == MOC_F32 && dst_dtype == MOC_BF16)
    transpose_kernel<float, __nv_bfloat16><<<grid, block, 0, stream>>>(static_cast<const float*>(src), static_cast<__nv_bfloat16*>(dst), rows, cols);
  else if (src_dtype == MOC_BF16 && dst_dtype == MOC_BF16)
    transpose_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), rows, cols);
  else if (src_dtype == MOC_F32 && dst_dtype == MOC_F32)
    transpose_kernel<float, float><<<grid, block, 0, stream>>>(static_cast<const float*>(src), static_cast<float*>(dst), rows, cols);
  else if (src_dtype == MOC_BF16 && dst_dtype == MOC_F32)
    transpose_kernel<__nv_bfloat16, float><<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), static_cast<float*>(dst), rows, cols);
  else MOC_REQUIRE(false, "bad dtype");
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_pack_weights(int32_t n, const void* const* src, int32_t src_dtype, void* const* dst,
                                void* const* dst_t, const int32_t* rows, const int32_t* cols,
                                const int32_t* ldt, void* stream_) {
  MOC_REQUIRE(n >= 1 && n <= 4 && src && dst && dst_t && rows && cols && ldt, "bad pack arguments");
  PackJobs jobs;
  jobs.n = n;
  int max_r = 0, max_c = 0;
  for (int i = 0; i < n; ++i) {
    MOC_REQUIRE(src[i] != nullptr && rows[i] > 0 && cols[i] > 0, "bad pack job");
    jobs.j[i] = PackJob{src[i], dst[i], dst_t[i], rows[i], cols[i], ldt[i] > 0 ? ldt[i] : rows[i]};
    if (rows[i] > max_r) max_r = rows[i];
    if (cols[i] > max_c) max_c = cols[i];
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  dim3 grid(ceil_div(max_c, 32), ceil_div(max_r, 32), n), block(32, 8);
  if (src_dtype == MOC_F32) pack_weights_kernel<float><<<grid, block, 0, stream>>>(jobs);
  else if (src_dtype == MOC_BF16) pack_weights_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(jobs);
  else MOC_REQUIRE(false, "bad dtype");
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}


extern "C" int moc_row_inv_rms(const void* bank, int32_t bank_dtype, int64_t rows, int32_t dim, float eps,
                               float* out, void* stream_) {
  MOC_REQUIRE(bank && out && rows > 0 && dim > 0, "bad arguments");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int blocks = static_cast<int>((rows * 32 + 255) / 256);
  if (bank_dtype == MOC_F32)
    row_inv_rms_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(bank), rows, dim, eps, out);
  else if (bank_dtype == MOC_BF16)
    row_inv_rms_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(bank), rows, dim,
                                                                  eps, out);
  else MOC_REQUIRE(false, "bad dtype");
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_chapter_row_scale(const int32_t* comb_idx, const float* comb_w, const float* inv_rms,
                                     int64_t bank_rows, int32_t n_pairs, int32_t T, float* scale, int32_t* status,
                                     void* stream_) {
  MOC_REQUIRE(comb_idx && scale && status && n_pairs > 0 && T > 0, "bad arguments");
  const long long total = static_cast<long long>(n_pairs) * T;
  row_scale_kernel<<<static_cast<int>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      comb_idx, comb_w, inv_rms, bank_rows, n_pairs, T, scale, status);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_gather_rows_bwd_prescaled(const void* g, int32_t g_dtype, const void* bank, int32_t bank_dtype,
                                             int64_t bank_rows, int32_t dim, int32_t T, const int32_t* comb_idx,
                                             const float* comb_w, int32_t n_pairs, const float* inv_rms,
                                             const int32_t* uniq, const int32_t* seg_offsets,
                                             const int32_t* seg_pairs, const int32_t* num_unique, float* d_comb_w,
                                             float* bank_grad, void* bank_grad_bf16, int32_t* status, void* stream_) {
  (void)status;
  MOC_REQUIRE(g && bank && comb_idx && uniq && seg_offsets && seg_pairs && num_unique, "NULL buffer");
  MOC_REQUIRE(bank_grad != nullptr || bank_grad_bf16 == nullptr || ((dim & 7) == 0 && dim <= 1024),
              "bf16 rows without the fp32 rows need dim % 8 == 0 and dim <= 1024");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long max_rows = static_cast<long long>(n_pairs) * T;
  const int blocks = static_cast<int>((max_rows * 32 + 255) / 256);
#define MOC_GPRE(TG, TB)                                                                                          \
  do {                                                                                                            \
    if (d_comb_w != nullptr)                                                                                      \
      dcombw_prescaled_kernel<TG, TB><<<n_pairs, 256, 0, stream>>>(static_cast<const TG*>(g),                     \
                                                                   static_cast<const TB*>(bank), bank_rows, dim,  \
                                                                   T, comb_idx, comb_w, d_comb_w);                \
    if (bank_grad != nullptr || bank_grad_bf16 != nullptr)                                                        \
      bank_grad_prescaled_kernel<TG, TB><<<blocks, 256, 0, stream>>>(                                             \
          static_cast<const TG*>(g), static_cast<const TB*>(bank), dim, T, inv_rms, uniq, seg_offsets, seg_pairs, \
          num_unique, max_rows, bank_grad, static_cast<__nv_bfloat16*>(bank_grad_bf16));                          \
  } while (0)
  if (g_dtype == MOC_F32 && bank_dtype == MOC_F32) MOC_GPRE(float, float);
  else if (g_dtype == MOC_F32 && bank_dtype == MOC_BF16) MOC_GPRE(float, __nv_bfloat16);
  else if (g_dtype == MOC_BF16 && bank_dtype == MOC_F32) MOC_GPRE(__nv_bfloat16, float);
  else if (g_dtype == MOC_BF16 && bank_dtype == MOC_BF16) MOC_GPRE(__nv_bfloat16, __nv_bfloat16);
  else MOC_REQUIRE(false, "bad dtype");
#undef MOC_GPRE
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}
