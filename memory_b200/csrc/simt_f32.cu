// fp32 kernels of the memory layer: strided SGEMM and joint-softmax attention forward / backward on
// the FMA pipes.  This is the fp32 arithmetic mode of the operators (tensor cores cannot deliver
// 1e-4 agreement with an fp32 reference); shapes are unrestricted apart from head_dim.
#include <math.h>

#include "moc_common.cuh"

namespace moc {
namespace {

// ---------------------------------------------------------------------------------------------
// SGEMM: C[m,n] (+)= sum_k A(m,k) * B(k,n), arbitrary element strides, 64x64x16 tiles
// ---------------------------------------------------------------------------------------------
constexpr int GT = 64, GK = 16;

__global__ void __launch_bounds__(256)
sgemm_kernel(const float* __restrict__ a, long long sa_m, long long sa_k, const float* __restrict__ b,
             long long sb_k, long long sb_n, float* __restrict__ c, long long ldc, int M, int N, int K,
             const float* __restrict__ row_scale, int scale_block, int accumulate,
             const float* __restrict__ residual, long long ldr) {
  __shared__ float As[GK][GT + 4];
  __shared__ float Bs[GK][GT + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += GK) {
    for (int i = threadIdx.x; i < GT * GK; i += 256) {
      int mm, kk;
      if (sa_k == 1) { kk = i % GK; mm = i / GK; } else { mm = i % GT; kk = i / GT; }
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? a[gm * sa_m + gk * sa_k] : 0.f;
      int nn, kb;
      if (sb_k == 1) { kb = i % GK; nn = i / GK; } else { nn = i % GT; kb = i / GT; }
      const int gn = n0 + nn, gkb = k0 + kb;
      Bs[kb][nn] = (gn < N && gkb < K) ? b[gkb * sb_k + gn * sb_n] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
    const float rs = row_scale ? row_scale[gm / scale_block] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float* dst = c + gm * ldc + gn;
      float v = acc[i][j] * rs;
      if (residual != nullptr) v += residual[gm * ldr + gn];
      *dst = accumulate ? *dst + v : v;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// attention, one thread per query (forward, dQ) or per key (dK, dV); tiles of the other side in
// shared memory.  q [B,L,H*D], kv [B,n_sel,2*HK*D], lse/delta [B,H,L].
// ---------------------------------------------------------------------------------------------
constexpr int kTile = 32;

template <int D>
__global__ void __launch_bounds__(128)
attn_fwd_kernel(const float* __restrict__ q, const float* __restrict__ kv, float* __restrict__ o,
                float* __restrict__ lse, int L, int n_sel, int H, int HK, float scale) {
  __shared__ float Ks[kTile][D];
  __shared__ float Vs[kTile][D];
  const int b = blockIdx.z, h = blockIdx.y;
  const int kh = h / (H / HK);
  const int l = blockIdx.x * 128 + threadIdx.x;
  const bool live = l < L;
  const int ldq = H * D, ldkv = 2 * HK * D;
  float qr[D], acc[D];
#pragma unroll
  for (int i = 0; i < D; ++i) {
    qr[i] = live ? q[(static_cast<long long>(b) * L + l) * ldq + h * D + i] * scale : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, den = 0.f;
  for (int j0 = 0; j0 < n_sel; j0 += kTile) {
    const int nt = min(kTile, n_sel - j0);
    __syncthreads();
    for (int i = threadIdx.x; i < kTile * D; i += 128) {
      const int jj = i / D, dd = i - jj * D;
      const long long row = (static_cast<long long>(b) * n_sel + j0 + jj) * ldkv;
      Ks[jj][dd] = jj < nt ? kv[row + kh * D + dd] : 0.f;
      Vs[jj][dd] = jj < nt ? kv[row + HK * D + kh * D + dd] : 0.f;
    }
    __syncthreads();
    float s[kTile];
    float tm = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < kTile; ++jj) {
      float d0 = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) d0 = fmaf(qr[i], Ks[jj][i], d0);
      s[jj] = jj < nt ? d0 : -INFINITY;
      tm = fmaxf(tm, s[jj]);
    }
    const float mn = fmaxf(m, tm);
    const float alpha = expf(m - mn);
    den *= alpha;
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] *= alpha;
#pragma unroll
    for (int jj = 0; jj < kTile; ++jj) {
      const float pv = expf(s[jj] - mn);
      den += pv;
#pragma unroll
      for (int i = 0; i < D; ++i) acc[i] = fmaf(pv, Vs[jj][i], acc[i]);
    }
    m = mn;
  }
  if (live) {
    const float inv = 1.f / den;
#pragma unroll
    for (int i = 0; i < D; ++i) o[(static_cast<long long>(b) * L + l) * ldq + h * D + i] = acc[i] * inv;
    lse[(static_cast<long long>(b) * H + h) * L + l] = m + logf(den);
  }
}

template <typename T>
__global__ void delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta,
                             int B, int L, int H, int D) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long total = static_cast<long long>(B) * L * H;
  if (w >= total) return;
  const int h = static_cast<int>(w % H);
  const long long bl = w / H;
  const int l = static_cast<int>(bl % L);
  const int b = static_cast<int>(bl / L);
  const T* po = o + bl * H * D + h * D;
  const T* pd = d_o + bl * H * D + h * D;
  float acc = 0.f;
  for (int i = lane; i < D; i += 32) acc += static_cast<float>(po[i]) * static_cast<float>(pd[i]);
  acc = warp_sum(acc);
  if (lane == 0) delta[(static_cast<long long>(b) * H + h) * L + l] = acc;
}

template <int D>
__global__ void __launch_bounds__(128)
attn_bwd_dq_kernel(const float* __restrict__ q, const float* __restrict__ kv, const float* __restrict__ d_o,
                   const float* __restrict__ lse, const float* __restrict__ delta, float* __restrict__ d_q,
                   int L, int n_sel, int H, int HK, float scale) {
  __shared__ float Ks[kTile][D];
  __shared__ float Vs[kTile][D];
  const int b = blockIdx.z, h = blockIdx.y;
  const int kh = h / (H / HK);
  const int l = blockIdx.x * 128 + threadIdx.x;
  const bool live = l < L;
  const int ldq = H * D, ldkv = 2 * HK * D;
  float qr[D], dor[D], dq[D];
  const long long qoff = (static_cast<long long>(b) * L + (live ? l : 0)) * ldq + h * D;
#pragma unroll
  for (int i = 0; i < D; ++i) {
    qr[i] = live ? q[qoff + i] * scale : 0.f;
    dor[i] = live ? d_o[qoff + i] : 0.f;
    dq[i] = 0.f;
  }
  const float ls = live ? lse[(static_cast<long long>(b) * H + h) * L + l] : 0.f;
  const float dl = live ? delta[(static_cast<long long>(b) * H + h) * L + l] : 0.f;
  for (int j0 = 0; j0 < n_sel; j0 += kTile) {
    const int nt = min(kTile, n_sel - j0);
    __syncthreads();
    for (int i = threadIdx.x; i < kTile * D; i += 128) {
      const int jj = i / D, dd = i - jj * D;
      const long long row = (static_cast<long long>(b) * n_sel + j0 + jj) * ldkv;
      Ks[jj][dd] = jj < nt ? kv[row + kh * D + dd] : 0.f;
      Vs[jj][dd] = jj < nt ? kv[row + HK * D + kh * D + dd] : 0.f;
    }
    __syncthreads();
    for (int jj = 0; jj < nt; ++jj) {
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int i = 0; i < D; ++i) { s = fmaf(qr[i], Ks[jj][i], s); dp = fmaf(dor[i], Vs[jj][i], dp); }
      const float ds = expf(s - ls) * (dp - dl) * scale;
#pragma unroll
      for (int i = 0; i < D; ++i) dq[i] = fmaf(ds, Ks[jj][i], dq[i]);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < D; ++i) d_q[qoff + i] = dq[i];
  }
}

// MODE 0: dV, MODE 1: dK.  One thread per key; query tiles (all heads of the KV group) in shared memory.
template <int D, int MODE>
__global__ void __launch_bounds__(128)
attn_bwd_dkv_kernel(const float* __restrict__ q, const float* __restrict__ kv, const float* __restrict__ d_o,
                    const float* __restrict__ lse, const float* __restrict__ delta, float* __restrict__ d_kv,
                    int L, int n_sel, int H, int HK, float scale) {
  __shared__ float Qs[kTile][D];
  __shared__ float Os[kTile][D];
  __shared__ float Ls[kTile], Ds[kTile];
  const int b = blockIdx.z, kh = blockIdx.y;
  const int G = H / HK;
  const int j = blockIdx.x * 128 + threadIdx.x;
  const bool live = j < n_sel;
  const int ldq = H * D, ldkv = 2 * HK * D;
  const long long krow = (static_cast<long long>(b) * n_sel + (live ? j : 0)) * ldkv;
  float kr[D], vr[MODE == 1 ? D : 1], acc[D];
#pragma unroll
  for (int i = 0; i < D; ++i) {
    kr[i] = live ? kv[krow + kh * D + i] : 0.f;
    if (MODE == 1) vr[i] = live ? kv[krow + HK * D + kh * D + i] : 0.f;
    acc[i] = 0.f;
  }
  for (int g = 0; g < G; ++g) {
    const int h = kh * G + g;
    for (int l0 = 0; l0 < L; l0 += kTile) {
      const int nt = min(kTile, L - l0);
      __syncthreads();
      for (int i = threadIdx.x; i < kTile * D; i += 128) {
        const int ll = i / D, dd = i - ll * D;
        const long long off = (static_cast<long long>(b) * L + l0 + ll) * ldq + h * D + dd;
        Qs[ll][dd] = ll < nt ? q[off] * scale : 0.f;
        Os[ll][dd] = ll < nt ? d_o[off] : 0.f;
      }
      if (threadIdx.x < kTile) {
        const long long off = (static_cast<long long>(b) * H + h) * L + l0 + threadIdx.x;
        Ls[threadIdx.x] = threadIdx.x < nt ? lse[off] : 0.f;
        Ds[threadIdx.x] = threadIdx.x < nt ? delta[off] : 0.f;
      }
      __syncthreads();
      for (int ll = 0; ll < nt; ++ll) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < D; ++i) s = fmaf(kr[i], Qs[ll][i], s);
        const float p = expf(s - Ls[ll]);
        if (MODE == 0) {
#pragma unroll
          for (int i = 0; i < D; ++i) acc[i] = fmaf(p, Os[ll][i], acc[i]);
        } else {
          float dp = 0.f;
#pragma unroll
          for (int i = 0; i < D; ++i) dp = fmaf(vr[i], Os[ll][i], dp);
          const float ds = p * (dp - Ds[ll]);    // Qs already carries the softmax scale
#pragma unroll
          for (int i = 0; i < D; ++i) acc[i] = fmaf(ds, Qs[ll][i], acc[i]);
        }
      }
    }
  }
  if (live) {
    const int col = (MODE == 0 ? HK * D : 0) + kh * D;
#pragma unroll
    for (int i = 0; i < D; ++i) d_kv[krow + col + i] = acc[i];
  }
}

}  // namespace

int launch_sgemm(const moc_gemm_desc* g, const float* a, const float* b, float* c, const float* row_scale,
                 cudaStream_t stream) {
  MOC_REQUIRE(g->c_dtype == MOC_F32, "fp32 projection writes fp32");
  const long long sa_m = g->a_kmajor ? g->lda : 1, sa_k = g->a_kmajor ? 1 : g->lda;
  const long long sb_k = g->b_kmajor ? 1 : g->ldb, sb_n = g->b_kmajor ? g->ldb : 1;
  dim3 grid(ceil_div(g->n, GT), ceil_div(g->m, GT));
  sgemm_kernel<<<grid, 256, 0, stream>>>(a, sa_m, sa_k, b, sb_k, sb_n, c, g->ldc, g->m, g->n, g->k, row_scale,
                                         g->scale_block_rows > 0 ? g->scale_block_rows : 1, g->accumulate,
                                         g->residual, g->ldr);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

int launch_delta(int dtype, const void* o, const void* d_o, float* delta, int B, int L, int H, int D,
                 cudaStream_t stream) {
  const long long total = static_cast<long long>(B) * L * H;
  const int blocks = static_cast<int>((total * 32 + 255) / 256);
  if (dtype == MOC_F32)
    delta_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(o), static_cast<const float*>(d_o),
                                                    delta, B, L, H, D);
  else
    delta_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(o),
                                                            static_cast<const __nv_bfloat16*>(d_o), delta, B, L, H, D);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

template <int D>
static int attn_f32_fwd_d(const moc_attn_shape* s, const float* q, const float* kv, float* o, float* lse,
                          cudaStream_t stream) {
  dim3 grid(ceil_div(s->seq, 128), s->num_heads, s->batch);
  attn_fwd_kernel<D><<<grid, 128, 0, stream>>>(q, kv, o, lse, s->seq, s->n_sel, s->num_heads, s->num_kv_heads, s->scale);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}
template <int D>
static int attn_f32_bwd_d(const moc_attn_shape* s, const float* q, const float* kv, const float* d_o,
                          const float* lse, const float* delta, float* d_q, float* d_kv, cudaStream_t stream) {
  dim3 gq(ceil_div(s->seq, 128), s->num_heads, s->batch);
  attn_bwd_dq_kernel<D><<<gq, 128, 0, stream>>>(q, kv, d_o, lse, delta, d_q, s->seq, s->n_sel, s->num_heads,
                                                s->num_kv_heads, s->scale);
  dim3 gk(ceil_div(s->n_sel, 128), s->num_kv_heads, s->batch);
  attn_bwd_dkv_kernel<D, 0><<<gk, 128, 0, stream>>>(q, kv, d_o, lse, delta, d_kv, s->seq, s->n_sel, s->num_heads,
                                                    s->num_kv_heads, s->scale);
  attn_bwd_dkv_kernel<D, 1><<<gk, 128, 0, stream>>>(q, kv, d_o, lse, delta, d_kv, s->seq, s->n_sel, s->num_heads,
                                                    s->num_kv_heads, s->scale);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

int launch_attn_f32_fwd(const moc_attn_shape* s, const float* q, const float* kv, float* o, float* lse,
                        cudaStream_t stream) {
  switch (s->head_dim) {
    case 16: return attn_f32_fwd_d<16>(s, q, kv, o, lse, stream);
    case 32: return attn_f32_fwd_d<32>(s, q, kv, o, lse, stream);
    case 64: return attn_f32_fwd_d<64>(s, q, kv, o, lse, stream);
    case 128: return attn_f32_fwd_d<128>(s, q, kv, o, lse, stream);
  }
  set_last_error("head_dim", "fp32 attention supports head_dim 16, 32, 64, 128");
  return MOC_ERR_UNSUPPORTED;
}
int launch_attn_f32_bwd(const moc_attn_shape* s, const float* q, const float* kv, const float* d_o,
                        const float* lse, const float* delta, float* d_q, float* d_kv, cudaStream_t stream) {
  switch (s->head_dim) {
    case 16: return attn_f32_bwd_d<16>(s, q, kv, d_o, lse, delta, d_q, d_kv, stream);
    case 32: return attn_f32_bwd_d<32>(s, q, kv, d_o, lse, delta, d_q, d_kv, stream);
    case 64: return attn_f32_bwd_d<64>(s, q, kv, d_o, lse, delta, d_q, d_kv, stream);
    case 128: return attn_f32_bwd_d<128>(s, q, kv, d_o, lse, delta, d_q, d_kv, stream);
  }
  set_last_error("head_dim", "fp32 attention supports head_dim 16, 32, 64, 128");
  return MOC_ERR_UNSUPPORTED;
}

}  // namespace moc
