// Per-token chapter-sparse attention (each query token attends to its own list of selected
// chapters with one joint softmax).  One warp per (batch, token, query head); lane j walks keys
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
