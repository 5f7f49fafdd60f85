// Pre-attention normalisation of the memory sub-block: y = norm(x) feeding the memory cross-attention
// whose output is added back to x (memory_block.py:549-558 of the reference: residual, memory_layernorm,
// memory_attn, residual add).  RMSNorm follows memory_block.py:26-28 (x / sqrt(mean(x^2) + eps) * w),
// LayerNorm follows torch.nn.LayerNorm.  Both kernels are bound by HBM: one warp per row, float4 accesses.
#include "moc_common.cuh"

namespace moc {
namespace {

constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;
constexpr int kBwdRowsPerBlock = 32;       // rows of one backward block, 4 per warp
constexpr int kBwdChunk = 1024;            // columns whose weight-gradient sums a warp keeps in registers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// stats[row] = (mean, 1/sqrt(var + eps)); mean is 0 for RMSNorm.
template <bool LN>
__global__ void __launch_bounds__(kNormThreads)
norm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                float eps, long long rows, int d, float* __restrict__ y32, __nv_bfloat16* __restrict__ y16,
                float* __restrict__ stats) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kNormWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float4* xr = reinterpret_cast<const float4*>(x + row * d);
  const int nv = d >> 2;
  float mean = 0.f;
  if (LN) {
    float s = 0.f;
    for (int i = lane; i < nv; i += 32) {
      const float4 v = xr[i];
      s += (v.x + v.y) + (v.z + v.w);
    }
    mean = warp_sum(s) / static_cast<float>(d);
  }
  float ss = 0.f;
  for (int i = lane; i < nv; i += 32) {
    const float4 v = xr[i];
    const float a = v.x - mean, b = v.y - mean, c = v.z - mean, e = v.w - mean;
    ss += (a * a + b * b) + (c * c + e * e);
  }
  const float inv = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(d) + eps);
  if (lane == 0) {
    stats[2 * row] = mean;
    stats[2 * row + 1] = inv;
  }
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const float4* b4 = reinterpret_cast<const float4*>(bias);
  for (int i = lane; i < nv; i += 32) {
    const float4 v = xr[i];
    const float4 g = w4[i];
    float4 o;
    o.x = (v.x - mean) * inv * g.x; o.y = (v.y - mean) * inv * g.y;
    o.z = (v.z - mean) * inv * g.z; o.w = (v.w - mean) * inv * g.w;
    if (LN && bias != nullptr) {
      const float4 bb = b4[i];
      o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
    }
    if (y32 != nullptr) reinterpret_cast<float4*>(y32 + row * d)[i] = o;
    if (y16 != nullptr) {
      uint2 pk;
      pk.x = pack_bf16x2(o.x, o.y);
      pk.y = pack_bf16x2(o.z, o.w);
      reinterpret_cast<uint2*>(y16 + row * d)[i] = pk;
    }
  }
}

// dx = inv * (g*w - mean_d(g*w) [LayerNorm only] - xhat * mean_d(g*w*xhat)) + residual_grad,
// partial[block][0][c] = sum over the block's rows of g*xhat, partial[block][1][c] = sum of g.
template <bool LN>
__global__ void __launch_bounds__(kNormThreads)
norm_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ w,
                const float* __restrict__ stats, const float* __restrict__ residual_grad, long long rows, int d,
                float* __restrict__ dx, float* __restrict__ partial) {
  __shared__ float red[kNormWarps][kBwdChunk];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const long long row0 = static_cast<long long>(blockIdx.x) * kBwdRowsPerBlock;
  constexpr int kRowsPerWarp = kBwdRowsPerBlock / kNormWarps;
  const int nv = d >> 2;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const float inv_d = 1.0f / static_cast<float>(d);

  // per-row sums over the whole row
  float c1[kRowsPerWarp], c2[kRowsPerWarp], mu[kRowsPerWarp], iv[kRowsPerWarp];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const long long row = row0 + warp + r * kNormWarps;
    c1[r] = c2[r] = mu[r] = iv[r] = 0.f;
    if (row >= rows) continue;
    mu[r] = stats[2 * row];
    iv[r] = stats[2 * row + 1];
    const float4* xr = reinterpret_cast<const float4*>(x + row * d);
    const float4* gr = reinterpret_cast<const float4*>(dy + row * d);
    float s1 = 0.f, s2 = 0.f;
    for (int i = lane; i < nv; i += 32) {
      const float4 xv = xr[i], gv = gr[i], wv = w4[i];
      const float g0 = gv.x * wv.x, g1 = gv.y * wv.y, g2 = gv.z * wv.z, g3 = gv.w * wv.w;
      s1 += g0 * ((xv.x - mu[r]) * iv[r]) + g1 * ((xv.y - mu[r]) * iv[r]) + g2 * ((xv.z - mu[r]) * iv[r]) +
            g3 * ((xv.w - mu[r]) * iv[r]);
      s2 += (g0 + g1) + (g2 + g3);
    }
    c1[r] = warp_sum(s1) * inv_d;
    c2[r] = LN ? warp_sum(s2) * inv_d : 0.f;
  }

  float* part_w = partial + static_cast<long long>(blockIdx.x) * 2 * d;
  float* part_b = part_w + d;
  for (int col0 = 0; col0 < d; col0 += kBwdChunk) {
    float4 aw[kBwdChunk / 128], ab[kBwdChunk / 128];
#pragma unroll
    for (int i = 0; i < kBwdChunk / 128; ++i) aw[i] = ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const long long row = row0 + warp + r * kNormWarps;
      if (row >= rows) continue;
      const float4* xr = reinterpret_cast<const float4*>(x + row * d);
      const float4* gr = reinterpret_cast<const float4*>(dy + row * d);
      const float4* rr = reinterpret_cast<const float4*>(residual_grad ? residual_grad + row * d : nullptr);
      float4* dr = reinterpret_cast<float4*>(dx + row * d);
#pragma unroll
      for (int i = 0; i < kBwdChunk / 128; ++i) {
        const int v = (col0 >> 2) + i * 32 + lane;
        if (v >= nv) continue;
        const float4 xv = xr[v], gv = gr[v], wv = w4[v];
        float4 xh;
        xh.x = (xv.x - mu[r]) * iv[r]; xh.y = (xv.y - mu[r]) * iv[r];
        xh.z = (xv.z - mu[r]) * iv[r]; xh.w = (xv.w - mu[r]) * iv[r];
        float4 o;
        o.x = iv[r] * (gv.x * wv.x - c2[r] - xh.x * c1[r]);
        o.y = iv[r] * (gv.y * wv.y - c2[r] - xh.y * c1[r]);
        o.z = iv[r] * (gv.z * wv.z - c2[r] - xh.z * c1[r]);
        o.w = iv[r] * (gv.w * wv.w - c2[r] - xh.w * c1[r]);
        if (residual_grad != nullptr) {
          const float4 rv = rr[v];
          o.x += rv.x; o.y += rv.y; o.z += rv.z; o.w += rv.w;
        }
        dr[v] = o;
        aw[i].x += gv.x * xh.x; aw[i].y += gv.y * xh.y; aw[i].z += gv.z * xh.z; aw[i].w += gv.w * xh.w;
        ab[i].x += gv.x; ab[i].y += gv.y; ab[i].z += gv.z; ab[i].w += gv.w;
      }
    }
    // sum the eight warps' column sums, weight gradient first and bias gradient second
#pragma unroll 1
    for (int which = 0; which < (LN ? 2 : 1); ++which) {
      __syncthreads();
#pragma unroll
      for (int i = 0; i < kBwdChunk / 128; ++i)
        reinterpret_cast<float4*>(red[warp])[i * 32 + lane] = which == 0 ? aw[i] : ab[i];
      __syncthreads();
      for (int c = threadIdx.x; c < kBwdChunk; c += kNormThreads) {
        if (col0 + c >= d) break;
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < kNormWarps; ++k) s += red[k][c];
        (which == 0 ? part_w : part_b)[col0 + c] = s;
      }
    }
  }
}

// 32 columns per block; warp k sums the partial rows k, k + 8, ... and shared memory adds the eight.
__global__ void __launch_bounds__(kNormThreads)
norm_bwd_finish_kernel(const float* __restrict__ partial, int blocks, int d, int with_bias,
                       float* __restrict__ dweight, float* __restrict__ dbias) {
  __shared__ float red[2][kNormWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float sw = 0.f, sb = 0.f;
  if (c < d) {
    for (int b = warp; b < blocks; b += kNormWarps) {
      sw += partial[static_cast<long long>(b) * 2 * d + c];
      if (with_bias) sb += partial[static_cast<long long>(b) * 2 * d + d + c];
    }
  }
  red[0][warp][lane] = sw;
  red[1][warp][lane] = sb;
  __syncthreads();
  if (warp == 0 && c < d) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int k = 0; k < kNormWarps; ++k) {
      tw += red[0][k][lane];
      tb += red[1][k][lane];
    }
    if (dweight != nullptr) dweight[c] = tw;
    if (with_bias && dbias != nullptr) dbias[c] = tb;
  }
}

inline long long bwd_blocks(long long rows) { return (rows + kBwdRowsPerBlock - 1) / kBwdRowsPerBlock; }

}  // namespace
}  // namespace moc

using namespace moc;

extern "C" size_t moc_norm_bwd_workspace_bytes(int64_t rows, int32_t dim) {
  if (rows <= 0 || dim <= 0) return 0;
  return static_cast<size_t>(bwd_blocks(rows)) * 2 * static_cast<size_t>(dim) * sizeof(float);
}

extern "C" int moc_norm_fwd(const float* x, const float* weight, const float* bias, int32_t kind, float eps,
                            int64_t rows, int32_t dim, float* y_f32, void* y_bf16, float* stats,
                            void* stream_) {
  MOC_REQUIRE(x && weight && stats && (y_f32 || y_bf16), "NULL normalisation argument");
  MOC_REQUIRE(kind == MOC_NORM_RMS || kind == MOC_NORM_LAYERNORM, "normalisation kind must be RMS or LayerNorm");
  MOC_REQUIRE(rows > 0 && dim > 0 && dim % 4 == 0, "rows must be positive and dim a positive multiple of 4");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const unsigned grid = static_cast<unsigned>((rows + kNormWarps - 1) / kNormWarps);
  __nv_bfloat16* y16 = static_cast<__nv_bfloat16*>(y_bf16);
  if (kind == MOC_NORM_LAYERNORM)
    norm_fwd_kernel<true><<<grid, kNormThreads, 0, stream>>>(x, weight, bias, eps, rows, dim, y_f32, y16, stats);
  else
    norm_fwd_kernel<false><<<grid, kNormThreads, 0, stream>>>(x, weight, nullptr, eps, rows, dim, y_f32, y16, stats);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_norm_bwd(const float* dy, const float* x, const float* weight, const float* stats,
                            const float* residual_grad, int32_t kind, int64_t rows, int32_t dim, float* dx,
                            float* dweight, float* dbias, void* workspace, void* stream_) {
  MOC_REQUIRE(dy && x && weight && stats && dx && workspace, "NULL normalisation-gradient argument");
  MOC_REQUIRE(kind == MOC_NORM_RMS || kind == MOC_NORM_LAYERNORM, "normalisation kind must be RMS or LayerNorm");
  MOC_REQUIRE(rows > 0 && dim > 0 && dim % 4 == 0, "rows must be positive and dim a positive multiple of 4");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long blocks = bwd_blocks(rows);
  float* partial = static_cast<float*>(workspace);
  const bool ln = kind == MOC_NORM_LAYERNORM;
  if (ln)
    norm_bwd_kernel<true><<<static_cast<unsigned>(blocks), kNormThreads, 0, stream>>>(
        dy, x, weight, stats, residual_grad, rows, dim, dx, partial);
  else
    norm_bwd_kernel<false><<<static_cast<unsigned>(blocks), kNormThreads, 0, stream>>>(
        dy, x, weight, stats, residual_grad, rows, dim, dx, partial);
  MOC_CUDA_OK(cudaGetLastError());
  if (dweight != nullptr || (ln && dbias != nullptr)) {
    norm_bwd_finish_kernel<<<(dim + 31) / 32, kNormThreads, 0, stream>>>(partial, static_cast<int>(blocks), dim,
                                                                   ln ? 1 : 0, dweight, dbias);
    MOC_CUDA_OK(cudaGetLastError());
  }
  return MOC_OK;
}
