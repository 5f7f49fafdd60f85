// Per-token chapter mixture on the tensor cores (bf16, head_dim 64, 64-row chapters), for sm_100a.
//
//   out[t] = base[t] + rho * sum_s w[t, s] * softmax(q_t K_{c(t,s)}^T * scale) V_{c(t,s)}      (one softmax per chapter)
//
// Every token picks its own chapters, so a token-stationary kernel would have to fetch a different K/V tile for every
// row.  The work is therefore turned round: an inverted index (chapter -> the (token, slot) pairs that selected it) is
// built on the device, and a CTA takes up to 128 such pairs of one chapter, gathers their query rows into a
// 128-byte-swizzled shared-memory tile and runs S = Q K_c^T and O = P V_c as tcgen05 products with the chapter's K / V
// tile (one TMA box each) stationary.  A chapter's softmax is complete inside one 64-key tile, so there is no
// running maximum; the weighted per-(pair, head) outputs go to a partial buffer that a second kernel sums over a
// token's slots in slot order (no atomics: results do not depend on scheduling).
//
// The backward pass keeps the same organisation with one CTA per chapter: S and dP = dO V_c^T are recomputed, dQ
// leaves as per-pair partials, and dK_c / dV_c accumulate in tensor memory over all pairs (and query heads) of the
// chapter through one 128 x 128 product  [Pw | dS]^T [dO | Q]  whose diagonal blocks are dV_c and dK_c (the
// off-diagonal blocks are not used: 64-row chapters would otherwise need 64-row MMA tiles).
#define MOC_KERNEL_TAG 5
#include <algorithm>

#include "moc_common.cuh"

namespace moc {
namespace {

constexpr int kTok = 128;        // (token, slot) pairs per tile
constexpr int kKeys = 64;        // rows of a chapter
constexpr int kD = 64;           // head dim
constexpr int kTileQ = kTok * kD * 2;     // 16 KiB
constexpr int kTileKV = kKeys * kD * 2;   // 8 KiB
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- inverted index ----------------------------------------------------------------------------------------
// pairs are numbered p = ((b * TQ + t) * HI + hi) * S + s (HI = 1: one chapter list per token for all heads;
// HI = HK: a list per KV head); buckets are numbered (b * HI + hi) * M + chapter.
struct IndexShape { int B, TQ, HI, S, M; };

__device__ __forceinline__ int bucket_of(const IndexShape& x, long long p, int chapter) {
  const long long bh = p / x.S;                       // (b * TQ + t) * HI + hi
  const int hi = static_cast<int>(bh % x.HI);
  const int b = static_cast<int>((bh / x.HI) / x.TQ);
  return (b * x.HI + hi) * x.M + chapter;
}

__global__ void mix_count_kernel(const int* __restrict__ idx, IndexShape x, long long n_pairs, int* __restrict__ cnt,
                                 int* __restrict__ status) {
  const long long p = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (p >= n_pairs) return;
  const int c = idx[p];
  if (c < 0 || c >= x.M) { atomicMax(status, MOC_DEV_BAD_INDEX); return; }
  atomicAdd(&cnt[bucket_of(x, p, c)], 1);
}

// exclusive scans of the bucket sizes and of the tiles per bucket; one CTA of 1024 threads
__global__ void mix_scan_kernel(const int* __restrict__ cnt, int n_buckets, int* __restrict__ bucket_off,
                                int* __restrict__ tile_off, int* __restrict__ totals) {
  __shared__ int warp_tot[2][32];
  const int per = (n_buckets + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * per, hi = min(n_buckets, lo + per);
  int s0 = 0, s1 = 0;
  for (int i = lo; i < hi; ++i) { s0 += cnt[i]; s1 += (cnt[i] + kTok - 1) / kTok; }
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
    warp_tot[0][lane] = w0; warp_tot[1][lane] = w1;
  }
  __syncthreads();
  int e0 = i0 - s0 + (warp > 0 ? warp_tot[0][warp - 1] : 0);
  int e1 = i1 - s1 + (warp > 0 ? warp_tot[1][warp - 1] : 0);
  for (int i = lo; i < hi; ++i) {
    bucket_off[i] = e0; tile_off[i] = e1;
    e0 += cnt[i]; e1 += (cnt[i] + kTok - 1) / kTok;
  }
  if (threadIdx.x == 0) {
    bucket_off[n_buckets] = warp_tot[0][31]; tile_off[n_buckets] = warp_tot[1][31];
    totals[0] = warp_tot[1][31];       // number of tiles
  }
}

__global__ void mix_fill_kernel(const int* __restrict__ idx, IndexShape x, long long n_pairs,
                                const int* __restrict__ bucket_off, int* __restrict__ cursor,
                                int* __restrict__ entries) {
  const long long p = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (p >= n_pairs) return;
  const int c = idx[p];
  if (c < 0 || c >= x.M) return;
  const int bkt = bucket_of(x, p, c);
  entries[bucket_off[bkt] + atomicAdd(&cursor[bkt], 1)] = static_cast<int>(p);
}

// Pairs of a bucket in ascending order (the fill above places them in arrival order): with it the sums the backward
// forms over a chapter's pairs do not depend on scheduling.  One CTA per bucket, rank sort in shared memory; buckets
// above 2,048 pairs are left in arrival order.
constexpr int kSortMax = 2048;
__global__ void mix_sort_kernel(const int* __restrict__ bucket_off, int* __restrict__ entries) {
  __shared__ int buf[kSortMax];
  const int first = bucket_off[blockIdx.x], n = bucket_off[blockIdx.x + 1] - first;
  if (n <= 1 || n > kSortMax) return;
  for (int i = threadIdx.x; i < n; i += blockDim.x) buf[i] = entries[first + i];
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int v = buf[i];
    int rank = 0;
    for (int j = 0; j < n; ++j) rank += (buf[j] < v);
    entries[first + rank] = v;           // pair ids are distinct
  }
}

__global__ void mix_tiles_kernel(const int* __restrict__ bucket_off, const int* __restrict__ tile_off, int n_buckets,
                                 int* __restrict__ tile_bucket, int* __restrict__ tile_first,
                                 int* __restrict__ tile_cnt) {
  const int bkt = blockIdx.x * blockDim.x + threadIdx.x;
  if (bkt >= n_buckets) return;
  const int first = bucket_off[bkt], n = bucket_off[bkt + 1] - first;
  int t = tile_off[bkt];
  for (int o = 0; o < n; o += kTok, ++t) {
    tile_bucket[t] = bkt;
    tile_first[t] = first + o;
    tile_cnt[t] = min(kTok, n - o);
  }
}

struct IndexBuffers {
  int *cnt, *cursor, *bucket_off, *tile_off, *entries, *tile_bucket, *tile_first, *tile_cnt, *totals;
};
inline long long max_tiles(long long n_pairs, long long n_buckets) { return n_pairs / kTok + n_buckets; }
inline size_t index_ints(long long n_pairs, long long n_buckets) {
  return static_cast<size_t>(4 * n_buckets + 2 + n_pairs + 3 * max_tiles(n_pairs, n_buckets) + 4);
}
inline IndexBuffers carve(int* ws, long long n_pairs, long long n_buckets) {
  IndexBuffers b;
  b.cnt = ws; ws += n_buckets;
  b.cursor = ws; ws += n_buckets;
  b.bucket_off = ws; ws += n_buckets + 1;
  b.tile_off = ws; ws += n_buckets + 1;
  b.entries = ws; ws += n_pairs;
  const long long mt = max_tiles(n_pairs, n_buckets);
  b.tile_bucket = ws; ws += mt;
  b.tile_first = ws; ws += mt;
  b.tile_cnt = ws; ws += mt;
  b.totals = ws;
  return b;
}

int build_index(const int* idx, const IndexShape& x, int* ws, int* status, cudaStream_t stream) {
  const long long n_pairs = static_cast<long long>(x.B) * x.TQ * x.HI * x.S;
  const long long n_buckets = static_cast<long long>(x.B) * x.HI * x.M;
  IndexBuffers ib = carve(ws, n_pairs, n_buckets);
  MOC_CUDA_OK(cudaMemsetAsync(ib.cnt, 0, static_cast<size_t>(2 * n_buckets) * sizeof(int), stream));   // cnt + cursor
  const int pb = static_cast<int>((n_pairs + 255) / 256);
  mix_count_kernel<<<pb, 256, 0, stream>>>(idx, x, n_pairs, ib.cnt, status);
  mix_scan_kernel<<<1, 1024, 0, stream>>>(ib.cnt, static_cast<int>(n_buckets), ib.bucket_off, ib.tile_off, ib.totals);
  mix_fill_kernel<<<pb, 256, 0, stream>>>(idx, x, n_pairs, ib.bucket_off, ib.cursor, ib.entries);
  mix_sort_kernel<<<static_cast<int>(n_buckets), 128, 0, stream>>>(ib.bucket_off, ib.entries);
  mix_tiles_kernel<<<static_cast<int>((n_buckets + 255) / 256), 256, 0, stream>>>(
      ib.bucket_off, ib.tile_off, static_cast<int>(n_buckets), ib.tile_bucket, ib.tile_first, ib.tile_cnt);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

// ---- MMA groups issued by one elected lane of a converged warp ------------------------------------------------
// One SS product over 4 K steps, A K-major, B K-major (BSTEP 2) or MN-major (BSTEP 128): [d] (+)= A * B.
template <int BSTEP>
__device__ __forceinline__ void issue_ss_one(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) umma_ss_w(d, a + kk * 2, b + kk * BSTEP, idesc, kk > 0 ? 1u : acc);
}
// One TS product over 4 K steps with MN-major B: [d] (+)= A * B, A K step kk at column a + 8 kk.
__device__ __forceinline__ void issue_ts_one(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) umma_ts_w(d, a + kk * 8, b + kk * 128, idesc, kk > 0 ? 1u : acc);
}
// One SS product over 8 K steps (128 rows), both operands MN-major.
__device__ __forceinline__ void issue_ss_mn128(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) umma_ss_w(d, a + kk * 128, b + kk * 128, idesc, kk > 0 ? 1u : acc);
}

// a 128-byte row (64 bf16) from global memory into row `r` of a 128-byte-swizzled tile
__device__ __forceinline__ void gather_row(uint8_t* tile, int r, const __nv_bfloat16* src, bool valid) {
  const uint4* g = reinterpret_cast<const uint4*>(src);
  uint4 v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = valid ? g[j] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(tile + r * 128 + ((j ^ (r & 7)) << 4)) = v[j];
}

struct MixShape {
  int B, TQ, TK, HQ, HK, HI, S, M;
  float scale, scale_log2, out_scale;
};

// ---- forward -------------------------------------------------------------------------------------------------
struct MixFwdParams {
  const __nv_bfloat16* q;        // [B*TQ, HQ*64]
  const float* w;                // [B*TQ, S]
  __nv_bfloat16* partial;        // [B*TQ, S, HQ, 64]
  float* lse_slots;              // [B*TQ, HQ, S]
  const int *entries, *tile_bucket, *tile_first, *tile_cnt, *totals;
  MixShape x;
  int* status;
};
constexpr int kMixThreads = 160;                       // 4 row-owning warps + 1 control warp (TMA, MMA issue)
constexpr int kFwdSmem = kTileQ + 2 * kTileKV + 1024;

__global__ void __launch_bounds__(kMixThreads, 4)
token_mix_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                        MixFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t kv_bar, q_ready, s_bar, p_bar, o_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = base;
  uint8_t* k_s = base + kTileQ;
  uint8_t* v_s = k_s + kTileKV;
  const MixShape& x = p.x;
  const int G = x.HQ / x.HK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&kv_bar, 1); mbar_init(&q_ready, kTok); mbar_init(&s_bar, 1); mbar_init(&p_bar, kTok);
    mbar_init(&o_bar, 1);
    fence_mbar_init();
    prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
  }
  if (warp == 4) { tmem_alloc(&tmem_slot, 128); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const int n_tiles = p.totals[0];
  uint32_t it = 0, kvn = 0;
  bool ok = true;

  for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
    const int bkt = p.tile_bucket[tile], first = p.tile_first[tile], cnt = p.tile_cnt[tile];
    const int c = bkt % x.M, bh = bkt / x.M, hi = bh % x.HI, b = bh / x.HI;
    const int hq_lo = x.HI == 1 ? 0 : hi * G, hq_hi = x.HI == 1 ? x.HQ : hq_lo + G;
    const int kv_row = b * x.TK + c * kKeys;
    if (warp == 4) {
      const uint32_t idesc_s = umma_idesc_bf16(kTok, kKeys, 0, 0);
      const uint32_t idesc_o = umma_idesc_bf16(kTok, kD, 0, 1);
      const uint64_t q_desc = umma_desc_sw128(smem_u32(q_s), 16, 1024);
      const uint64_t k_desc = umma_desc_sw128(smem_u32(k_s), 16, 1024);
      const uint64_t v_desc = umma_desc_sw128(smem_u32(v_s), 8192, 1024);     // V tile as MN-major B
      for (int hq = hq_lo; hq < hq_hi && ok; ++hq, ++it) {
        const bool reload = hq == hq_lo || hq % G == 0;
        if (it > 0) ok = mbar_wait_w(&o_bar, (it - 1) & 1, &abort_flag, p.status);   // K/V tiles and TMEM free
        if (!ok) break;
        if (reload && lane == 0) {
          mbar_arrive_expect_tx(&kv_bar, 2 * kTileKV);
          tma_load_2d(k_s, &tmap_k, &kv_bar, (hq / G) * kD, kv_row);
          tma_load_2d(v_s, &tmap_v, &kv_bar, (hq / G) * kD, kv_row);
        }
        __syncwarp();
        ok = mbar_wait_w(&q_ready, it & 1, &abort_flag, p.status);
        if (ok && reload) { ok = mbar_wait_w(&kv_bar, kvn & 1, &abort_flag, p.status); ++kvn; }
        if (!ok) break;
        tc_fence_after();
        issue_ss_one<2>(tmem, q_desc, k_desc, idesc_s, 0u);
        tc_commit_w(&s_bar);
        ok = mbar_wait_w(&p_bar, it & 1, &abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        issue_ts_one(tmem + 64, tmem, v_desc, idesc_o, 0u);
        tc_commit_w(&o_bar);
      }
    } else {
      const int r = threadIdx.x;
      const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;
      const bool valid = r < cnt;
      const int pair = valid ? p.entries[first + r] : 0;
      const int s = pair % x.S;
      const long long tokrow = (pair / x.S) / x.HI;
      const float wv = valid ? p.w[tokrow * x.S + s] : 0.f;
      for (int hq = hq_lo; hq < hq_hi && ok; ++hq, ++it) {
        gather_row(q_s, r, p.q + tokrow * (x.HQ * kD) + hq * kD, valid);
        fence_proxy_async();
        mbar_arrive(&q_ready);
        ok = mbar_wait(&s_bar, it & 1, &abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float m, l = 0.f;
        {
          uint32_t s0[32], s1[32], pk[32];
          tmem_ld32(tmem + lane_sel, s0);
          tmem_ld32(tmem + lane_sel + 32, s1);
          tmem_wait_ld();
          m = __uint_as_float(s0[0]);
#pragma unroll
          for (int i = 0; i < 32; ++i) m = fmaxf(m, fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])));
          const float mm = m * x.scale_log2;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float a0 = ex2(fmaf(__uint_as_float(s0[i]), x.scale_log2, -mm));
            const float a1 = ex2(fmaf(__uint_as_float(s0[i + 1]), x.scale_log2, -mm));
            const float b0 = ex2(fmaf(__uint_as_float(s1[i]), x.scale_log2, -mm));
            const float b1 = ex2(fmaf(__uint_as_float(s1[i + 1]), x.scale_log2, -mm));
            l += (a0 + a1) + (b0 + b1);
            pk[i / 2] = pack_bf16x2(a0, a1);
            pk[16 + i / 2] = pack_bf16x2(b0, b1);
          }
          tmem_st32(tmem + lane_sel, pk);          // P over the first half of S's columns (own lanes only)
          tmem_wait_st();
        }
        tc_fence_before();
        mbar_arrive(&p_bar);
        ok = mbar_wait(&o_bar, it & 1, &abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const float f = x.out_scale * wv / l;
        __nv_bfloat16* dst = p.partial + ((tokrow * x.S + s) * x.HQ + hq) * kD;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t o[32];
          tmem_ld32(tmem + lane_sel + 64 + half * 32, o);
          tmem_wait_ld();
          if (valid) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[8 * j + 0]) * f, __uint_as_float(o[8 * j + 1]) * f);
              v.y = pack_bf16x2(__uint_as_float(o[8 * j + 2]) * f, __uint_as_float(o[8 * j + 3]) * f);
              v.z = pack_bf16x2(__uint_as_float(o[8 * j + 4]) * f, __uint_as_float(o[8 * j + 5]) * f);
              v.w = pack_bf16x2(__uint_as_float(o[8 * j + 6]) * f, __uint_as_float(o[8 * j + 7]) * f);
              *reinterpret_cast<uint4*>(dst + half * 32 + j * 8) = v;
            }
          }
        }
        if (valid) p.lse_slots[(tokrow * x.HQ + hq) * x.S + s] = fmaf(m, x.scale, __logf(l));
        tc_fence_before();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag) { for (int i = 0; i < 200; ++i) __nanosleep(1000); }
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem, 128); }
}

// out[t] = base[t] + sum_s partial[t, s] in slot order, fp32 sums; one thread per 8 elements.  Slots whose chapter
// id is out of range were never written and are skipped.
__global__ void slot_reduce_kernel(const __nv_bfloat16* __restrict__ partial, const __nv_bfloat16* __restrict__ base,
                                   const int* __restrict__ idx, __nv_bfloat16* __restrict__ out, long long rows,
                                   int S, int HQ, int HK, int HI, int M) {
  const int chunks = HQ * (kD / 8);
  const long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (t >= rows * chunks) return;
  const long long row = t / chunks;
  const int ch = static_cast<int>(t % chunks);
  const int hi = HI == 1 ? 0 : (ch >> 3) / (HQ / HK);
  float acc[8];
  if (base != nullptr) {
    const uint4 v = reinterpret_cast<const uint4*>(base)[t];
    const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] = __uint_as_float(wd[i] << 16);
      acc[2 * i + 1] = __uint_as_float(wd[i] & 0xFFFF0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  }
  for (int s = 0; s < S; ++s) {
    const int c = idx[(row * HI + hi) * S + s];
    if (c < 0 || c >= M) continue;
    const uint4 v = reinterpret_cast<const uint4*>(partial)[(row * S + s) * chunks + ch];
    const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += __uint_as_float(wd[i] << 16);
      acc[2 * i + 1] += __uint_as_float(wd[i] & 0xFFFF0000u);
    }
  }
  uint4 o;
  o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
  o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
  reinterpret_cast<uint4*>(out)[t] = o;
}

// ---- backward ------------------------------------------------------------------------------------------------
struct MixBwdParams {
  const __nv_bfloat16* q;        // [B*TQ, HQ*64]
  const __nv_bfloat16* d_o;      // [B*TQ, HQ*64]
  const float* w;                // [B*TQ, S]
  const float* lse_slots;        // [B*TQ, HQ, S]
  __nv_bfloat16* dq_partial;     // [B*TQ, S, HQ, 64]
  float* d_w_heads;              // [B*TQ, HQ, S]
  __nv_bfloat16 *d_k, *d_v;      // rows b*TK + key, row stride dkv_ld elements; head kh at column kh*64
  long long dkv_ld;
  const int *entries, *bucket_off;
  int n_buckets;
  MixShape x;
  int* status;
};
constexpr int kBwdSmem = 4 * kTileQ + 4 * kTileKV + 1024;
constexpr uint32_t kColS = 0, kColDP = 64, kColD = 128;      // dQ reuses S's columns

// The (chapter bucket, KV head) groups a CTA works through: buckets blockIdx.x, + gridDim.x, ... that hold pairs,
// and for each the KV heads that read its index list.  The control warp and the row warps walk the same sequence.
struct GroupIter {
  int bkt, kh, kh_hi, first, n, kv_row;
  // first non-empty bucket at or after bkt; with zero_row >= 0 (thread index of a row-owning thread) the dK / dV rows
  // of the empty buckets passed on the way are zero-filled, so the caller need not clear the buffers
  __device__ __forceinline__ void seek(const MixBwdParams& p, int zero_row = -1) {
    for (; bkt < p.n_buckets; bkt += gridDim.x) {
      first = p.bucket_off[bkt];
      n = p.bucket_off[bkt + 1] - first;
      if (n > 0) break;
      if (zero_row >= 0) {
        const MixShape& x = p.x;
        const int c = bkt % x.M, bh = bkt / x.M, hi = bh % x.HI, b = bh / x.HI;
        const int h0 = x.HI == 1 ? 0 : hi, h1 = x.HI == 1 ? x.HK : hi + 1;
        __nv_bfloat16* dst = (zero_row >= 64 ? p.d_k : p.d_v) +
                             (static_cast<long long>(b) * x.TK + c * kKeys + (zero_row & 63)) * p.dkv_ld;
        for (int e = h0 * (kD / 8); e < h1 * (kD / 8); ++e) reinterpret_cast<uint4*>(dst)[e] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (bkt >= p.n_buckets) return;
    const MixShape& x = p.x;
    const int c = bkt % x.M, bh = bkt / x.M, hi = bh % x.HI, b = bh / x.HI;
    kh = x.HI == 1 ? 0 : hi;
    kh_hi = x.HI == 1 ? x.HK : hi + 1;
    kv_row = b * x.TK + c * kKeys;
  }
  __device__ __forceinline__ void start(const MixBwdParams& p, int zero_row = -1) { bkt = blockIdx.x; seek(p, zero_row); }
  __device__ __forceinline__ bool done(const MixBwdParams& p) const { return bkt >= p.n_buckets; }
  __device__ __forceinline__ void next(const MixBwdParams& p, int zero_row = -1) {
    if (++kh < kh_hi) return;
    bkt += gridDim.x;
    seek(p, zero_row);
  }
};

__global__ void __launch_bounds__(kMixThreads, 2)
token_mix_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                        MixBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t kv_bar[2], in_ready, sdp_bar, ds_ready, done_bar, d_read;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* do_s = base;                  // [dO | Q]: the two 64-column blocks of the MN-major B operand of D
  uint8_t* q_s = base + kTileQ;
  uint8_t* pw_s = base + 2 * kTileQ;     // [Pw | dS]: the two 64-row blocks of the MN-major A operand of D
  uint8_t* ds_s = base + 3 * kTileQ;
  uint8_t* kv_s = base + 4 * kTileQ;     // two (K, V) tile pairs: the next group's pair arrives under this group's work
  const MixShape& x = p.x;
  const int G = x.HQ / x.HK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&kv_bar[0], 1); mbar_init(&kv_bar[1], 1);
    mbar_init(&in_ready, kTok); mbar_init(&sdp_bar, 1); mbar_init(&ds_ready, kTok);
    mbar_init(&done_bar, 1); mbar_init(&d_read, kTok);
    fence_mbar_init();
    prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
  }
  if (warp == 4) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  uint32_t it = 0, kvn = 0;      // tile iterations and (bucket, KV head) groups this CTA has run
  bool ok = true;
  GroupIter gi;
  gi.start(p, warp < 4 ? static_cast<int>(threadIdx.x) : -1);

  if (warp == 4) {
    const uint32_t idesc_kk = umma_idesc_bf16(kTok, kKeys, 0, 0);     // S, dP: both operands K-major
    const uint32_t idesc_dq = umma_idesc_bf16(kTok, kD, 0, 1);        // dQ = dS K: B = K tile, MN-major
    const uint32_t idesc_d = umma_idesc_bf16(128, 128, 1, 1);         // D = [Pw|dS]^T [dO|Q]
    const uint64_t q_desc = umma_desc_sw128(smem_u32(q_s), 16, 1024);
    const uint64_t do_desc = umma_desc_sw128(smem_u32(do_s), 16, 1024);
    const uint64_t ds_desc = umma_desc_sw128(smem_u32(ds_s), 16, 1024);
    const uint64_t k_desc0 = umma_desc_sw128(smem_u32(kv_s), 16, 1024);
    const uint64_t v_desc0 = umma_desc_sw128(smem_u32(kv_s) + kTileKV, 16, 1024);
    const uint64_t kmn_desc0 = umma_desc_sw128(smem_u32(kv_s), 8192, 1024);
    const uint64_t a_d = umma_desc_sw128(smem_u32(pw_s), kTileQ, 1024);
    const uint64_t b_d = umma_desc_sw128(smem_u32(do_s), kTileQ, 1024);
    constexpr uint64_t kBufOff = (2 * kTileKV) >> 4;
    auto load_kv = [&](const GroupIter& g, uint32_t n) {
      if (lane == 0) {
        uint8_t* dst = kv_s + (n & 1) * 2 * kTileKV;
        mbar_arrive_expect_tx(&kv_bar[n & 1], 2 * kTileKV);
        tma_load_2d(dst, &tmap_k, &kv_bar[n & 1], g.kh * kD, g.kv_row);
        tma_load_2d(dst + kTileKV, &tmap_v, &kv_bar[n & 1], g.kh * kD, g.kv_row);
      }
      __syncwarp();
    };
    if (!gi.done(p)) load_kv(gi, 0);
    for (; !gi.done(p) && ok; ++kvn) {
      const int iters = G * ((gi.n + kTok - 1) / kTok);
      GroupIter nxt = gi;
      nxt.next(p);
      // the other K/V buffer is free once every product of the previous group has completed
      if (it > 0) ok = mbar_wait_w(&done_bar, (it - 1) & 1, &abort_flag, p.status);
      if (!ok) break;
      if (!nxt.done(p)) load_kv(nxt, kvn + 1);
      ok = mbar_wait_w(&kv_bar[kvn & 1], (kvn >> 1) & 1, &abort_flag, p.status);
      const uint64_t boff = (kvn & 1) * kBufOff;
      for (int u = 0; u < iters && ok; ++u, ++it) {
        ok = mbar_wait_w(&in_ready, it & 1, &abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        issue_ss_one<2>(tmem + kColS, q_desc, k_desc0 + boff, idesc_kk, 0u);
        issue_ss_one<2>(tmem + kColDP, do_desc, v_desc0 + boff, idesc_kk, 0u);
        tc_commit_w(&sdp_bar);
        ok = mbar_wait_w(&ds_ready, it & 1, &abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        issue_ss_one<128>(tmem + kColS, ds_desc, kmn_desc0 + boff, idesc_dq, 0u);
        if (u == 0 && kvn > 0) {        // D of the previous group has been read out
          ok = mbar_wait_w(&d_read, (kvn - 1) & 1, &abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
        }
        issue_ss_mn128(tmem + kColD, a_d, b_d, idesc_d, u > 0 ? 1u : 0u);
        tc_commit_w(&done_bar);
      }
      gi = nxt;
    }
  } else {
    const int r = threadIdx.x;
    const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;
    // D of a finished group is read out after this thread has handed over the inputs of the next iteration, so
    // that the read runs beside that iteration's S / dP products: rows 0..63 x columns 0..63 = dV_c, rows
    // 64..127 x columns 64..127 = dK_c (before the softmax scale)
    bool pending = false;
    long long pend_row = 0;
    int pend_kh = 0;
    auto flush_d = [&]() {
      const int key = r & 63;
      const bool is_k = r >= 64;
      const float f = is_k ? x.scale : 1.f;
      __nv_bfloat16* dst = (is_k ? p.d_k : p.d_v) + (pend_row + key) * p.dkv_ld + pend_kh * kD;
      tc_fence_after();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t o[32];
        tmem_ld32(tmem + lane_sel + kColD + (is_k ? 64 : 0) + half * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(o[8 * j + 0]) * f, __uint_as_float(o[8 * j + 1]) * f);
          v.y = pack_bf16x2(__uint_as_float(o[8 * j + 2]) * f, __uint_as_float(o[8 * j + 3]) * f);
          v.z = pack_bf16x2(__uint_as_float(o[8 * j + 4]) * f, __uint_as_float(o[8 * j + 5]) * f);
          v.w = pack_bf16x2(__uint_as_float(o[8 * j + 6]) * f, __uint_as_float(o[8 * j + 7]) * f);
          *reinterpret_cast<uint4*>(dst + half * 32 + j * 8) = v;
        }
      }
      tc_fence_before();
      mbar_arrive(&d_read);
      pending = false;
    };
    // pair ids and per-pair constants of an iteration; fetched one iteration ahead, so that the two dependent global
    // loads (bucket offsets -> pair id -> weight / log-sum-exp) run under the previous iteration's products
    struct Meta { long long tokrow; int s, hq; float wv, nl2; bool valid; };
    auto fetch_meta = [&](const GroupIter& g, int u) {
      Meta m;
      const int tiles = (g.n + kTok - 1) / kTok;
      const int tl = u % tiles;
      m.hq = g.kh * G + u / tiles;
      m.valid = tl * kTok + r < g.n;
      const int pair = m.valid ? p.entries[g.first + tl * kTok + r] : 0;
      m.s = pair % x.S;
      m.tokrow = (pair / x.S) / x.HI;
      m.wv = m.valid ? p.w[m.tokrow * x.S + m.s] * x.out_scale : 0.f;
      m.nl2 = m.valid ? -p.lse_slots[(m.tokrow * x.HQ + m.hq) * x.S + m.s] * kLog2e : 0.f;
      return m;
    };
    int u = 0;
    Meta next_m = {0, 0, 0, 0.f, 0.f, false};
    if (!gi.done(p)) next_m = fetch_meta(gi, 0);
    while (!gi.done(p) && ok) {
      {
        const int iters = G * ((gi.n + kTok - 1) / kTok);
        const Meta m = next_m;
        const int hq = m.hq, s = m.s;
        const bool valid = m.valid;
        const long long tokrow = m.tokrow;
        const float wv = m.wv, nl2 = m.nl2;
        // the tiles are free: this thread has seen done_bar of the previous iteration
        gather_row(do_s, r, p.d_o + tokrow * (x.HQ * kD) + hq * kD, valid);
        gather_row(q_s, r, p.q + tokrow * (x.HQ * kD) + hq * kD, valid);
        fence_proxy_async();
        mbar_arrive(&in_ready);
        GroupIter ngi = gi;
        int nu = u + 1;
        const bool last = nu == iters;
        if (last) { ngi.next(p, r); nu = 0; }
        if (!ngi.done(p)) next_m = fetch_meta(ngi, nu);
        if (pending) flush_d();
        ok = mbar_wait(&sdp_bar, it & 1, &abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float pr[64];
        float delta = 0.f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t rs[32], rd[32];
          tmem_ld32(tmem + lane_sel + kColS + half * 32, rs);
          tmem_ld32(tmem + lane_sel + kColDP + half * 32, rd);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float pj = ex2(fmaf(__uint_as_float(rs[i]), x.scale_log2, nl2));
            delta = fmaf(pj, __uint_as_float(rd[i]), delta);
            pr[half * 32 + i] = pj;
          }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t rd[32];
          tmem_ld32(tmem + lane_sel + kColDP + half * 32, rd);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t a[4], d[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int e = j * 8 + 2 * i;
              const float p0 = wv * pr[half * 32 + e], p1 = wv * pr[half * 32 + e + 1];
              a[i] = pack_bf16x2(p0, p1);
              d[i] = pack_bf16x2(p0 * (__uint_as_float(rd[e]) - delta), p1 * (__uint_as_float(rd[e + 1]) - delta));
            }
            const int chunk = ((half * 4 + j) ^ (r & 7)) << 4;
            *reinterpret_cast<uint4*>(pw_s + r * 128 + chunk) = valid ? make_uint4(a[0], a[1], a[2], a[3])
                                                                      : make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(ds_s + r * 128 + chunk) = valid ? make_uint4(d[0], d[1], d[2], d[3])
                                                                      : make_uint4(0u, 0u, 0u, 0u);
          }
        }
        if (valid) p.d_w_heads[(tokrow * x.HQ + hq) * x.S + s] = x.out_scale * delta;
        tc_fence_before();
        fence_proxy_async();
        mbar_arrive(&ds_ready);
        ok = mbar_wait(&done_bar, it & 1, &abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        __nv_bfloat16* dst = p.dq_partial + ((tokrow * x.S + s) * x.HQ + hq) * kD;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t o[32];
          tmem_ld32(tmem + lane_sel + kColS + half * 32, o);
          tmem_wait_ld();
          if (valid) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[8 * j + 0]) * x.scale, __uint_as_float(o[8 * j + 1]) * x.scale);
              v.y = pack_bf16x2(__uint_as_float(o[8 * j + 2]) * x.scale, __uint_as_float(o[8 * j + 3]) * x.scale);
              v.z = pack_bf16x2(__uint_as_float(o[8 * j + 4]) * x.scale, __uint_as_float(o[8 * j + 5]) * x.scale);
              v.w = pack_bf16x2(__uint_as_float(o[8 * j + 6]) * x.scale, __uint_as_float(o[8 * j + 7]) * x.scale);
              *reinterpret_cast<uint4*>(dst + half * 32 + j * 8) = v;
            }
          }
        }
        tc_fence_before();
        ++it;
        if (last) {            // D of this group is complete: done_bar of its last iteration has been seen
          pending = true;
          pend_row = gi.kv_row;
          pend_kh = gi.kh;
        }
        gi = ngi;
        u = nu;
      }
    }
    if (ok && pending) flush_d();
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag) { for (int i = 0; i < 200; ++i) __nanosleep(1000); }
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      n = 148;
  }
  return n;
}

int check_shape(const moc_sparse_attn_shape* s, int index_heads, MixShape* x) {
  MOC_REQUIRE(s != nullptr, "shape is NULL");
  MOC_REQUIRE(s->dtype == MOC_BF16 && s->head_dim == kD && s->block_size == kKeys,
              "the tensor-core token mixture takes bf16, head_dim 64 and 64-row chapters");
  MOC_REQUIRE(s->hq % s->h == 0 && (index_heads == 1 || index_heads == s->h), "index_heads must be 1 or the KV head count");
  MOC_REQUIRE(s->tk % kKeys == 0 && s->n_select > 0, "whole chapters only");
  const long long n_pairs = static_cast<long long>(s->batch) * s->tq * index_heads * s->n_select;
  const long long n_buckets = static_cast<long long>(s->batch) * index_heads * (s->tk / kKeys);
  MOC_REQUIRE(n_pairs < (1ll << 31) && n_buckets < (1ll << 30), "too many (token, slot) pairs for 32-bit pair ids");
  x->B = s->batch; x->TQ = s->tq; x->TK = s->tk; x->HQ = s->hq; x->HK = s->h; x->HI = index_heads;
  x->S = s->n_select; x->M = s->tk / kKeys;
  x->scale = s->scale; x->scale_log2 = s->scale * kLog2e; x->out_scale = 1.f;
  return MOC_OK;
}

int kv_maps(const MixShape& x, const void* k, const void* v, long long ld, CUtensorMap* mk, CUtensorMap* mv) {
  const uint64_t rows = static_cast<uint64_t>(x.B) * x.TK, cols = static_cast<uint64_t>(x.HK) * kD;
  int rc = make_tmap_bf16_2d(mk, k, rows, cols, static_cast<uint64_t>(ld), kKeys, kD);
  if (rc != MOC_OK) return rc;
  return make_tmap_bf16_2d(mv, v, rows, cols, static_cast<uint64_t>(ld), kKeys, kD);
}

}  // namespace
}  // namespace moc

using namespace moc;

extern "C" size_t moc_token_mix_workspace_bytes(const moc_sparse_attn_shape* s, int32_t index_heads) {
  if (s == nullptr || index_heads <= 0 || s->block_size <= 0) return 0;
  const long long n_pairs = static_cast<long long>(s->batch) * s->tq * index_heads * s->n_select;
  const long long n_buckets = static_cast<long long>(s->batch) * index_heads * (s->tk / s->block_size);
  return index_ints(n_pairs, n_buckets) * sizeof(int);
}

extern "C" int moc_token_mix_index(const moc_sparse_attn_shape* s, int32_t index_heads, const int32_t* block_indices,
                                   void* workspace, int32_t* status, void* stream) {
  MixShape x;
  int rc = check_shape(s, index_heads, &x);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(block_indices && workspace && status, "NULL argument");
  const IndexShape ix{x.B, x.TQ, x.HI, x.S, x.M};
  return build_index(block_indices, ix, static_cast<int*>(workspace), status, static_cast<cudaStream_t>(stream));
}

extern "C" int moc_token_mix_fwd(const moc_sparse_attn_shape* s, int32_t index_heads, const void* q, const void* k,
                                 const void* v, int64_t kv_row_stride, const int32_t* block_indices,
                                 const float* weights, const void* base, float out_scale, const void* workspace,
                                 void* partial, void* o, float* lse_slots, int32_t* status, void* stream) {
  MixShape x;
  int rc = check_shape(s, index_heads, &x);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(q && k && v && block_indices && weights && workspace && partial && o && lse_slots && status,
              "NULL argument");
  MOC_REQUIRE(kv_row_stride >= static_cast<int64_t>(x.HK) * kD && kv_row_stride % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(k) % 16 == 0 && reinterpret_cast<uintptr_t>(v) % 16 == 0,
              "K / V rows must be 16-byte aligned");
  x.out_scale = out_scale;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap mk, mv;
  rc = kv_maps(x, k, v, kv_row_stride, &mk, &mv);
  if (rc != MOC_OK) return rc;
  const long long n_pairs = static_cast<long long>(x.B) * x.TQ * x.HI * x.S;
  const long long n_buckets = static_cast<long long>(x.B) * x.HI * x.M;
  IndexBuffers ib = carve(static_cast<int*>(const_cast<void*>(workspace)), n_pairs, n_buckets);
  MixFwdParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.w = weights;
  p.partial = static_cast<__nv_bfloat16*>(partial); p.lse_slots = lse_slots;
  p.entries = ib.entries; p.tile_bucket = ib.tile_bucket; p.tile_first = ib.tile_first; p.tile_cnt = ib.tile_cnt;
  p.totals = ib.totals; p.x = x; p.status = status;
  static bool attr_set = false;
  if (!attr_set) {
    MOC_CUDA_OK(cudaFuncSetAttribute(token_mix_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem));
    attr_set = true;
  }
  const long long grid = std::min<long long>(max_tiles(n_pairs, n_buckets), static_cast<long long>(sm_count()) * 4);
  token_mix_fwd_tc_kernel<<<static_cast<int>(grid), kMixThreads, kFwdSmem, st>>>(mk, mv, p);
  const long long rows = static_cast<long long>(x.B) * x.TQ;
  const long long threads = rows * x.HQ * (kD / 8);
  slot_reduce_kernel<<<static_cast<int>((threads + 255) / 256), 256, 0, st>>>(
      p.partial, static_cast<const __nv_bfloat16*>(base), block_indices, static_cast<__nv_bfloat16*>(o), rows, x.S, x.HQ,
      x.HK, x.HI, x.M);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_token_mix_bwd(const moc_sparse_attn_shape* s, int32_t index_heads, const void* q, const void* k,
                                 const void* v, int64_t kv_row_stride, const int32_t* block_indices,
                                 const float* weights, float out_scale, const float* lse_slots, const void* d_o,
                                 const void* workspace, void* dq_partial, const void* d_q_base, void* d_q, void* d_k,
                                 void* d_v, int64_t dkv_row_stride, float* d_w_heads, int32_t* status, void* stream) {
  MixShape x;
  int rc = check_shape(s, index_heads, &x);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(q && k && v && block_indices && weights && lse_slots && d_o && workspace && dq_partial && d_q && d_k &&
                  d_v && d_w_heads && status, "NULL argument");
  MOC_REQUIRE(kv_row_stride >= static_cast<int64_t>(x.HK) * kD && kv_row_stride % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(k) % 16 == 0 && reinterpret_cast<uintptr_t>(v) % 16 == 0,
              "K / V rows must be 16-byte aligned");
  MOC_REQUIRE(dkv_row_stride >= static_cast<int64_t>(x.HK) * kD && dkv_row_stride % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(d_k) % 16 == 0 && reinterpret_cast<uintptr_t>(d_v) % 16 == 0,
              "dK / dV rows must be 16-byte aligned");
  x.out_scale = out_scale;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap mk, mv;
  rc = kv_maps(x, k, v, kv_row_stride, &mk, &mv);
  if (rc != MOC_OK) return rc;
  const long long n_pairs = static_cast<long long>(x.B) * x.TQ * x.HI * x.S;
  const long long n_buckets = static_cast<long long>(x.B) * x.HI * x.M;
  IndexBuffers ib = carve(static_cast<int*>(const_cast<void*>(workspace)), n_pairs, n_buckets);
  MixBwdParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.d_o = static_cast<const __nv_bfloat16*>(d_o);
  p.w = weights; p.lse_slots = lse_slots;
  p.dq_partial = static_cast<__nv_bfloat16*>(dq_partial); p.d_w_heads = d_w_heads;
  p.d_k = static_cast<__nv_bfloat16*>(d_k); p.d_v = static_cast<__nv_bfloat16*>(d_v); p.dkv_ld = dkv_row_stride;
  p.entries = ib.entries; p.bucket_off = ib.bucket_off; p.n_buckets = static_cast<int>(n_buckets);
  p.x = x; p.status = status;
  static bool attr_set = false;
  if (!attr_set) {
    MOC_CUDA_OK(cudaFuncSetAttribute(token_mix_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem));
    attr_set = true;
  }
  const long long grid = std::min<long long>(n_buckets, static_cast<long long>(sm_count()) * 2);
  token_mix_bwd_tc_kernel<<<static_cast<int>(grid), kMixThreads, kBwdSmem, st>>>(mk, mv, p);
  const long long rows = static_cast<long long>(x.B) * x.TQ;
  const long long threads = rows * x.HQ * (kD / 8);
  slot_reduce_kernel<<<static_cast<int>((threads + 255) / 256), 256, 0, st>>>(
      p.dq_partial, static_cast<const __nv_bfloat16*>(d_q_base), block_indices, static_cast<__nv_bfloat16*>(d_q), rows,
      x.S, x.HQ, x.HK, x.HI, x.M);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}
