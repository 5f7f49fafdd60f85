// Per-token chapter-sparse attention.  Two mixing rules:
//   joint     each query token attends to its own list of selected chapters with one joint softmax
//             (the contract of memory_cross_attn and FSA_topk_sparse_attention_bthd);
//   weighted  every selected chapter has its own softmax and the per-chapter outputs are mixed by the router
//             weights, out = base + rho * sum_s w_s softmax(q K_s^T) V_s (the exact mixture rule of
//             FSA_topk_sparse_attention_weighted_bthd and of the token-routed module path).  One warp per (batch, token, query head); lane j walks keys
// j, j+32, ... of the selected chapters with a private online softmax that is merged across the
// warp at the end.  Backward recomputes the probabilities and adds dK / dV with fp32 atomics, the
// same accumulation scheme as the reference's "strategy b".
#include <math.h>

#include "moc_common.cuh"

namespace moc {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) {
  p[i] = __float2bfloat16(v);
}

struct SpShape { int B, TQ, TK, HQ, H, S, BS; float scale; };

template <typename T, int D>
__global__ void __launch_bounds__(128)
sparse_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                  const int* __restrict__ bidx, T* __restrict__ o, float* __restrict__ lse, SpShape s,
                  int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long total = static_cast<long long>(s.B) * s.TQ * s.HQ;
  if (w >= total) return;
  const int hq = static_cast<int>(w % s.HQ);
  const long long bt = w / s.HQ;
  const int b = static_cast<int>(bt / s.TQ);
  const int h = hq / (s.HQ / s.H);
  const T* qp = q + (bt * s.HQ + hq) * D;
  float qr[D];
#pragma unroll
  for (int i = 0; i < D; ++i) qr[i] = ldf(qp, i) * s.scale;
  float acc[D];
#pragma unroll
  for (int i = 0; i < D; ++i) acc[i] = 0.f;
  float m = -INFINITY, den = 0.f;
  const int* bi = bidx + (bt * s.H + h) * s.S;
  const int n_blocks = s.TK / s.BS;
  for (int sl = 0; sl < s.S; ++sl) {
    const int blk = bi[sl];
    if (blk < 0 || blk >= n_blocks) {
      if (lane == 0) atomicMax(status, MOC_DEV_BAD_INDEX);
      continue;
    }
    for (int j = lane; j < s.BS; j += 32) {
      const long long row = ((static_cast<long long>(b) * s.TK + static_cast<long long>(blk) * s.BS + j) * s.H + h) * D;
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) sc = fmaf(qr[i], ldf(k, row + i), sc);
      const float mn = fmaxf(m, sc);
      const float alpha = expf(m - mn), pv = expf(sc - mn);
      den = den * alpha + pv;
#pragma unroll
      for (int i = 0; i < D; ++i) acc[i] = fmaf(pv, ldf(v, row + i), acc[i] * alpha);
      m = mn;
    }
  }
  // merge the 32 private softmax states
  const float mw = warp_max(m);
  const float f = (m == -INFINITY) ? 0.f : expf(m - mw);
  den = warp_sum(den * f);
  const float inv = den > 0.f ? 1.f / den : 0.f;
  T* op = o + (bt * s.HQ + hq) * D;
#pragma unroll
  for (int i = 0; i < D; ++i) {
    const float t = warp_sum(acc[i] * f);
    if (lane == (i & 31)) stf(op, i, t * inv);
  }
  if (lane == 0) lse[bt * s.HQ + hq] = mw + logf(den);
}

template <typename T, int D>
__global__ void __launch_bounds__(128)
sparse_bwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                  const int* __restrict__ bidx, const T* __restrict__ o, const float* __restrict__ lse,
                  const T* __restrict__ d_o, T* __restrict__ d_q, float* __restrict__ d_k,
                  float* __restrict__ d_v, SpShape s) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long total = static_cast<long long>(s.B) * s.TQ * s.HQ;
  if (w >= total) return;
  const int hq = static_cast<int>(w % s.HQ);
  const long long bt = w / s.HQ;
  const int b = static_cast<int>(bt / s.TQ);
  const int h = hq / (s.HQ / s.H);
  const long long qoff = (bt * s.HQ + hq) * D;
  float qr[D], gr[D], dq[D];
  float delta = 0.f;
#pragma unroll
  for (int i = 0; i < D; ++i) {
    qr[i] = ldf(q, qoff + i);
    gr[i] = ldf(d_o, qoff + i);
    delta = fmaf(ldf(o, qoff + i), gr[i], delta);
    dq[i] = 0.f;
  }
  const float ls = lse[bt * s.HQ + hq];
  const int* bi = bidx + (bt * s.H + h) * s.S;
  const int n_blocks = s.TK / s.BS;
  for (int sl = 0; sl < s.S; ++sl) {
    const int blk = bi[sl];
    if (blk < 0 || blk >= n_blocks) continue;
    for (int j = lane; j < s.BS; j += 32) {
      const long long row = ((static_cast<long long>(b) * s.TK + static_cast<long long>(blk) * s.BS + j) * s.H + h) * D;
      float sc = 0.f, dp = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) {
        sc = fmaf(qr[i], ldf(k, row + i), sc);
        dp = fmaf(gr[i], ldf(v, row + i), dp);
      }
      const float p = expf(sc * s.scale - ls);
      const float ds = p * (dp - delta) * s.scale;
#pragma unroll
      for (int i = 0; i < D; ++i) {
        dq[i] = fmaf(ds, ldf(k, row + i), dq[i]);
        atomicAdd(d_k + row + i, ds * qr[i]);
        atomicAdd(d_v + row + i, p * gr[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < D; ++i) {
    const float t = warp_sum(dq[i]);
    if (lane == (i & 31)) stf(d_q, qoff + i, t);
  }
}

// ---- weighted (per-chapter softmax) -------------------------------------------------------------------------
struct SpWeighted {
  long long ldk;        // elements between consecutive key rows of k and of v (H * D when contiguous)
  long long ldg;        // same for the fp32 d_k / d_v accumulators
  float out_scale;      // rho
  int accumulate_dq;
};

// One warp per (batch, token, query head).  Per slot: scores of the chapter's keys (lane j owns keys j, j+32, ...),
// warp max and sum -> that chapter's own softmax; lanes accumulate (rho w_s / den_s) p v privately over all slots
// and one warp reduction per output element finishes the row.  lse_slots[b, t, hq, s] keeps every chapter's
// log-sum-exp for the backward pass.
template <typename T, int D>
__global__ void __launch_bounds__(128)
sparse_weighted_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                           const int* __restrict__ bidx, const float* __restrict__ wts, const T* __restrict__ base,
                           T* __restrict__ o, float* __restrict__ lse_slots, SpShape s, SpWeighted x,
                           int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long total = static_cast<long long>(s.B) * s.TQ * s.HQ;
  if (w >= total) return;
  const int hq = static_cast<int>(w % s.HQ);
  const long long bt = w / s.HQ;
  const int b = static_cast<int>(bt / s.TQ);
  const int h = hq / (s.HQ / s.H);
  const T* qp = q + (bt * s.HQ + hq) * D;
  float qr[D];
#pragma unroll
  for (int i = 0; i < D; ++i) qr[i] = ldf(qp, i) * s.scale;
  float acc[D];
#pragma unroll
  for (int i = 0; i < D; ++i) acc[i] = 0.f;
  const int* bi = bidx + (bt * s.H + h) * s.S;
  const float* wp = wts + bt * s.S;
  const int n_blocks = s.TK / s.BS;
  for (int sl = 0; sl < s.S; ++sl) {
    const int blk = bi[sl];
    float* lp = lse_slots + (bt * s.HQ + hq) * s.S + sl;
    if (blk < 0 || blk >= n_blocks) {
      if (lane == 0) { atomicMax(status, MOC_DEV_BAD_INDEX); *lp = 0.f; }
      continue;
    }
    const long long row0 = (static_cast<long long>(b) * s.TK + static_cast<long long>(blk) * s.BS) * x.ldk + h * D;
    float m = -INFINITY;
    for (int j = lane; j < s.BS; j += 32) {
      const long long row = row0 + j * x.ldk;
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) sc = fmaf(qr[i], ldf(k, row + i), sc);
      m = fmaxf(m, sc);
    }
    m = warp_max(m);
    float den = 0.f;
    for (int j = lane; j < s.BS; j += 32) {
      const long long row = row0 + j * x.ldk;
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) sc = fmaf(qr[i], ldf(k, row + i), sc);
      den += expf(sc - m);
    }
    den = warp_sum(den);
    const float coef = x.out_scale * wp[sl] / den;
    for (int j = lane; j < s.BS; j += 32) {
      const long long row = row0 + j * x.ldk;
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) sc = fmaf(qr[i], ldf(k, row + i), sc);
      const float pv = expf(sc - m) * coef;
#pragma unroll
      for (int i = 0; i < D; ++i) acc[i] = fmaf(pv, ldf(v, row + i), acc[i]);
    }
    if (lane == 0) *lp = m + logf(den);
  }
  T* op = o + (bt * s.HQ + hq) * D;
  const T* bp = base ? base + (bt * s.HQ + hq) * D : nullptr;
#pragma unroll
  for (int i = 0; i < D; ++i) {
    const float t = warp_sum(acc[i]);
    if (lane == (i & 31)) stf(op, i, t + (bp ? ldf(bp, i) : 0.f));
  }
}

// Backward of the weighted rule.  Per slot s:  p = exp(score - lse_s),  dp = <dO, v>,  delta_s = sum_j p dp
// (that chapter's own softmax), d w_s = rho * delta_s (summed over heads by the caller: written per head),
// d score = rho w_s p (dp - delta_s).  d_k / d_v receive fp32 atomic adds (rows shared by many tokens).
template <typename T, int D>
__global__ void __launch_bounds__(128)
sparse_weighted_bwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                           const int* __restrict__ bidx, const float* __restrict__ wts,
                           const float* __restrict__ lse_slots, const T* __restrict__ d_o, T* __restrict__ d_q,
                           float* __restrict__ d_k, float* __restrict__ d_v, float* __restrict__ d_w_heads,
                           SpShape s, SpWeighted x) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long total = static_cast<long long>(s.B) * s.TQ * s.HQ;
  if (w >= total) return;
  const int hq = static_cast<int>(w % s.HQ);
  const long long bt = w / s.HQ;
  const int b = static_cast<int>(bt / s.TQ);
  const int h = hq / (s.HQ / s.H);
  const long long qoff = (bt * s.HQ + hq) * D;
  float qr[D], gr[D], dq[D];
#pragma unroll
  for (int i = 0; i < D; ++i) {
    qr[i] = ldf(q, qoff + i);
    gr[i] = ldf(d_o, qoff + i);
    dq[i] = 0.f;
  }
  const int* bi = bidx + (bt * s.H + h) * s.S;
  const float* wp = wts + bt * s.S;
  const int n_blocks = s.TK / s.BS;
  for (int sl = 0; sl < s.S; ++sl) {
    const int blk = bi[sl];
    float* dwp = d_w_heads + (bt * s.HQ + hq) * s.S + sl;
    if (blk < 0 || blk >= n_blocks) {
      if (lane == 0) *dwp = 0.f;
      continue;
    }
    const float ls = lse_slots[(bt * s.HQ + hq) * s.S + sl];
    const long long row0 = (static_cast<long long>(b) * s.TK + static_cast<long long>(blk) * s.BS) * x.ldk + h * D;
    const long long grow0 = (static_cast<long long>(b) * s.TK + static_cast<long long>(blk) * s.BS) * x.ldg + h * D;
    float delta = 0.f;
    for (int j = lane; j < s.BS; j += 32) {
      const long long row = row0 + j * x.ldk;
      float sc = 0.f, dp = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) {
        sc = fmaf(qr[i], ldf(k, row + i), sc);
        dp = fmaf(gr[i], ldf(v, row + i), dp);
      }
      delta = fmaf(expf(sc * s.scale - ls), dp, delta);
    }
    delta = warp_sum(delta);
    if (lane == 0) *dwp = x.out_scale * delta;
    const float rw = x.out_scale * wp[sl];
    for (int j = lane; j < s.BS; j += 32) {
      const long long row = row0 + j * x.ldk, grow = grow0 + j * x.ldg;
      float sc = 0.f, dp = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) {
        sc = fmaf(qr[i], ldf(k, row + i), sc);
        dp = fmaf(gr[i], ldf(v, row + i), dp);
      }
      const float p = expf(sc * s.scale - ls) * rw;
      const float ds = p * (dp - delta) * s.scale;
#pragma unroll
      for (int i = 0; i < D; ++i) {
        dq[i] = fmaf(ds, ldf(k, row + i), dq[i]);
        atomicAdd(d_k + grow + i, ds * qr[i]);
        atomicAdd(d_v + grow + i, p * gr[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < D; ++i) {
    const float t = warp_sum(dq[i]);
    if (lane == (i & 31)) stf(d_q, qoff + i, t + (x.accumulate_dq ? ldf(d_q, qoff + i) : 0.f));
  }
}

template <typename T>
int weighted_dispatch(bool backward, const moc_sparse_attn_shape* s, const void* q, const void* k, const void* v,
                      const int* bidx, const float* wts, const void* base, void* o, float* lse_slots,
                      const void* d_o, void* d_q, float* d_k, float* d_v, float* d_w_heads, SpWeighted x,
                      int* status, cudaStream_t stream) {
  SpShape sp{s->batch, s->tq, s->tk, s->hq, s->h, s->n_select, s->block_size, s->scale};
  const long long total = static_cast<long long>(s->batch) * s->tq * s->hq;
  const int blocks = static_cast<int>((total * 32 + 127) / 128);
#define MOC_SPW(DD)                                                                                               \
  do {                                                                                                            \
    if (!backward)                                                                                                \
      sparse_weighted_fwd_kernel<T, DD><<<blocks, 128, 0, stream>>>(                                              \
          static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), bidx, wts,                \
          static_cast<const T*>(base), static_cast<T*>(o), lse_slots, sp, x, status);                             \
    else                                                                                                          \
      sparse_weighted_bwd_kernel<T, DD><<<blocks, 128, 0, stream>>>(                                              \
          static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), bidx, wts, lse_slots,     \
          static_cast<const T*>(d_o), static_cast<T*>(d_q), d_k, d_v, d_w_heads, sp, x);                          \
  } while (0)
  switch (s->head_dim) {
    case 16: MOC_SPW(16); break;
    case 32: MOC_SPW(32); break;
    case 64: MOC_SPW(64); break;
    case 128: MOC_SPW(128); break;
    default: set_last_error("head_dim", "sparse attention supports head_dim 16, 32, 64, 128"); return MOC_ERR_UNSUPPORTED;
  }
#undef MOC_SPW
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

template <typename T>
int fwd_dispatch(const moc_sparse_attn_shape* s, const void* q, const void* k, const void* v, const int* bidx,
                 void* o, float* lse, int* status, cudaStream_t stream) {
  SpShape sp{s->batch, s->tq, s->tk, s->hq, s->h, s->n_select, s->block_size, s->scale};
  const long long total = static_cast<long long>(s->batch) * s->tq * s->hq;
  const int blocks = static_cast<int>((total * 32 + 127) / 128);
#define MOC_SP_FWD(DD)                                                                                       \
  sparse_fwd_kernel<T, DD><<<blocks, 128, 0, stream>>>(static_cast<const T*>(q), static_cast<const T*>(k),   \
                                                       static_cast<const T*>(v), bidx, static_cast<T*>(o),   \
                                                       lse, sp, status)
  switch (s->head_dim) {
    case 16: MOC_SP_FWD(16); break;
    case 32: MOC_SP_FWD(32); break;
    case 64: MOC_SP_FWD(64); break;
    case 128: MOC_SP_FWD(128); break;
    default: set_last_error("head_dim", "sparse attention supports head_dim 16, 32, 64, 128"); return MOC_ERR_UNSUPPORTED;
  }
#undef MOC_SP_FWD
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

template <typename T>
int bwd_dispatch(const moc_sparse_attn_shape* s, const void* q, const void* k, const void* v, const int* bidx,
                 const void* o, const float* lse, const void* d_o, void* d_q, float* d_k, float* d_v,
                 cudaStream_t stream) {
  SpShape sp{s->batch, s->tq, s->tk, s->hq, s->h, s->n_select, s->block_size, s->scale};
  const long long total = static_cast<long long>(s->batch) * s->tq * s->hq;
  const int blocks = static_cast<int>((total * 32 + 127) / 128);
#define MOC_SP_BWD(DD)                                                                                       \
  sparse_bwd_kernel<T, DD><<<blocks, 128, 0, stream>>>(static_cast<const T*>(q), static_cast<const T*>(k),   \
                                                       static_cast<const T*>(v), bidx, static_cast<const T*>(o), \
                                                       lse, static_cast<const T*>(d_o), static_cast<T*>(d_q), \
                                                       d_k, d_v, sp)
  switch (s->head_dim) {
    case 16: MOC_SP_BWD(16); break;
    case 32: MOC_SP_BWD(32); break;
    case 64: MOC_SP_BWD(64); break;
    case 128: MOC_SP_BWD(128); break;
    default: set_last_error("head_dim", "sparse attention supports head_dim 16, 32, 64, 128"); return MOC_ERR_UNSUPPORTED;
  }
#undef MOC_SP_BWD
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

int check(const moc_sparse_attn_shape* s) {
  MOC_REQUIRE(s != nullptr, "shape is NULL");
  MOC_REQUIRE(s->batch > 0 && s->tq > 0 && s->tk > 0 && s->n_select > 0 && s->block_size > 0, "empty problem");
  MOC_REQUIRE(s->h > 0 && s->hq % s->h == 0, "HQ must be multiple of H (GQA grouping).");
  MOC_REQUIRE(s->tk % s->block_size == 0, "TK must be divisible by block_size (chapter size) for clean chapter blocks.");
  return MOC_OK;
}

}  // namespace
}  // namespace moc

using namespace moc;

extern "C" int moc_sparse_attn_fwd(const moc_sparse_attn_shape* s, const void* q, const void* k, const void* v,
                                   const int32_t* block_indices, void* o, float* lse, int32_t* status,
                                   void* stream_) {
  int rc = check(s);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(q && k && v && block_indices && o && lse && status, "NULL buffer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (s->dtype == MOC_F32) return fwd_dispatch<float>(s, q, k, v, block_indices, o, lse, status, stream);
  if (s->dtype == MOC_BF16) return fwd_dispatch<__nv_bfloat16>(s, q, k, v, block_indices, o, lse, status, stream);
  set_last_error("dtype", "unknown dtype");
  return MOC_ERR_INVALID;
}

extern "C" int moc_sparse_attn_bwd(const moc_sparse_attn_shape* s, const void* q, const void* k, const void* v,
                                   const int32_t* block_indices, const void* o, const float* lse,
                                   const void* d_o, void* d_q, float* d_k, float* d_v, int32_t* status,
                                   void* stream_) {
  int rc = check(s);
  if (rc != MOC_OK) return rc;
  (void)status;
  MOC_REQUIRE(q && k && v && block_indices && o && lse && d_o && d_q && d_k && d_v, "NULL buffer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const size_t kv_elems = static_cast<size_t>(s->batch) * s->tk * s->h * s->head_dim;
  MOC_CUDA_OK(cudaMemsetAsync(d_k, 0, kv_elems * sizeof(float), stream));
  MOC_CUDA_OK(cudaMemsetAsync(d_v, 0, kv_elems * sizeof(float), stream));
  if (s->dtype == MOC_F32) return bwd_dispatch<float>(s, q, k, v, block_indices, o, lse, d_o, d_q, d_k, d_v, stream);
  if (s->dtype == MOC_BF16)
    return bwd_dispatch<__nv_bfloat16>(s, q, k, v, block_indices, o, lse, d_o, d_q, d_k, d_v, stream);
  set_last_error("dtype", "unknown dtype");
  return MOC_ERR_INVALID;
}


extern "C" int moc_sparse_attn_weighted_fwd(const moc_sparse_attn_shape* s, const void* q, const void* k,
                                            const void* v, int64_t kv_row_stride, const int32_t* block_indices,
                                            const float* weights, const void* base, float out_scale, void* o,
                                            float* lse_slots, int32_t* status, void* stream_) {
  int rc = check(s);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(q && k && v && block_indices && weights && o && lse_slots && status, "NULL buffer");
  MOC_REQUIRE(kv_row_stride >= static_cast<int64_t>(s->h) * s->head_dim, "kv_row_stride below one row of heads");
  SpWeighted x{kv_row_stride, 0, out_scale, 0};
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (s->dtype == MOC_F32)
    return weighted_dispatch<float>(false, s, q, k, v, block_indices, weights, base, o, lse_slots, nullptr, nullptr,
                                    nullptr, nullptr, nullptr, x, status, stream);
  if (s->dtype == MOC_BF16)
    return weighted_dispatch<__nv_bfloat16>(false, s, q, k, v, block_indices, weights, base, o, lse_slots, nullptr,
                                            nullptr, nullptr, nullptr, nullptr, x, status, stream);
  set_last_error("dtype", "unknown dtype");
  return MOC_ERR_INVALID;
}

extern "C" int moc_sparse_attn_weighted_bwd(const moc_sparse_attn_shape* s, const void* q, const void* k,
                                            const void* v, int64_t kv_row_stride, const int32_t* block_indices,
                                            const float* weights, float out_scale, const float* lse_slots,
                                            const void* d_o, void* d_q, int32_t accumulate_dq, float* d_k,
                                            float* d_v, int64_t dkv_row_stride, float* d_w_heads, int32_t* status,
                                            void* stream_) {
  int rc = check(s);
  if (rc != MOC_OK) return rc;
  (void)status;
  MOC_REQUIRE(q && k && v && block_indices && weights && lse_slots && d_o && d_q && d_k && d_v && d_w_heads,
              "NULL buffer");
  MOC_REQUIRE(kv_row_stride >= static_cast<int64_t>(s->h) * s->head_dim &&
              dkv_row_stride >= static_cast<int64_t>(s->h) * s->head_dim, "row stride below one row of heads");
  SpWeighted x{kv_row_stride, dkv_row_stride, out_scale, accumulate_dq};
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (s->dtype == MOC_F32)
    return weighted_dispatch<float>(true, s, q, k, v, block_indices, weights, nullptr, nullptr,
                                    const_cast<float*>(lse_slots), d_o, d_q, d_k, d_v, d_w_heads, x, status, stream);
  if (s->dtype == MOC_BF16)
    return weighted_dispatch<__nv_bfloat16>(true, s, q, k, v, block_indices, weights, nullptr, nullptr,
                                            const_cast<float*>(lse_slots), d_o, d_q, d_k, d_v, d_w_heads, x, status,
                                            stream);
  set_last_error("dtype", "unknown dtype");
  return MOC_ERR_INVALID;
}
