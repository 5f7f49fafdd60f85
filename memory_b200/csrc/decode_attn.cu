// Decode-time memory attention over a cache of projected bank rows.
//
// The reference re-gathers (S+k)*T bank rows per sequence at every generated token and re-projects them with Wk / Wv
// (inference/generate.py:194-210 -> model.py:624-692 -> memory_attention.py:241-243).  The bank and the projections
// are constant while decoding, and the chapter weight multiplies a gathered row before the (linear) projection, so
//   K = (u_c * norm(m)) Wk^T = u_c * (norm(m) Wk^T)
// and a per-layer cache  KV_bank = norm(M) [Wk; Wv]^T  (bf16, [C*T, 2*HK*64]) turns the step into a gather of
// cached rows scaled by the chapter weight, followed by one joint softmax over all selected keys:
//   s_r = scale * u_c * <q, K_bank[r]>,   out = sum_r softmax(s)_r * u_c * V_bank[r].
// The kernel is bound by HBM: one CTA per (sequence, query token, head) streams 128-byte K and V rows; every lane
// keeps its own running (max, sum, 64 accumulators) over the rows it owns, so nothing is exchanged between lanes
// until the end.
#include "moc_common.cuh"

namespace moc {
namespace {

constexpr int kDD = 64;
constexpr int kDecThreads = 256;
constexpr int kDecWarps = kDecThreads / 32;
constexpr float kDecLog2e = 1.4426950408889634f;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

__global__ void __launch_bounds__(kDecThreads, 1)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kv_bank,
                   long long bank_rows, const int* __restrict__ comb_idx, const float* __restrict__ comb_w,
                   __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int n_q, int H, int HK, int n_ch, int T,
                   float scale, int* __restrict__ status) {
  __shared__ float red[kDecWarps][kDD + 2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = blockIdx.x, iq = blockIdx.y, b = blockIdx.z;
  const int kh = h / (H / HK);
  const long long row_elems = 2ll * HK * kDD;

  // the query lives in shared memory (broadcast reads): registers go to rows in flight instead
  __shared__ __align__(16) float q_s[kDD];
  if (threadIdx.x < kDD)
    q_s[threadIdx.x] = __bfloat162float(q[(static_cast<long long>(b) * n_q + iq) * H * kDD + h * kDD + threadIdx.x]);
  __syncthreads();
  const float4* q4 = reinterpret_cast<const float4*>(q_s);
  const float c2 = scale * kDecLog2e;
  float m = -INFINITY, l = 0.f;          // running maximum (log2 domain) and sum of this lane's rows
  float acc[kDD];
#pragma unroll
  for (int i = 0; i < kDD; ++i) acc[i] = 0.f;

  // one row: score against the query, then fold it into this lane's running softmax state
  auto fold = [&](const uint4 (&kr)[kDD / 8], const uint4 (&vr)[kDD / 8], float u) {
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kDD / 8; ++i) {
      float f[8];
      unpack8(kr[i], f);
      const float4 qa = q4[2 * i], qb = q4[2 * i + 1];
      dot = fmaf(qa.x, f[0], dot); dot = fmaf(qa.y, f[1], dot); dot = fmaf(qa.z, f[2], dot); dot = fmaf(qa.w, f[3], dot);
      dot = fmaf(qb.x, f[4], dot); dot = fmaf(qb.y, f[5], dot); dot = fmaf(qb.z, f[6], dot); dot = fmaf(qb.w, f[7], dot);
    }
    const float s = dot * u * c2;
    const float m_new = fmaxf(m, s);
    const float corr = exp2f(m - m_new);      // 0 on the first row (m = -inf)
    const float pr = exp2f(s - m_new);
    l = l * corr + pr;
    const float pu = pr * u;
#pragma unroll
    for (int i = 0; i < kDD / 8; ++i) {
      float f[8];
      unpack8(vr[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[8 * i + j] = fmaf(acc[8 * i + j], corr, pu * f[j]);
    }
    m = m_new;
  };

  for (int c = warp; c < n_ch; c += kDecWarps) {
    const int ch = comb_idx[b * n_ch + c];
    if (ch < 0 || (static_cast<long long>(ch) + 1) * T > bank_rows) {
      if (lane == 0) atomicMax(status, MOC_DEV_BAD_INDEX);
      continue;
    }
    const float u = comb_w[b * n_ch + c];
    const __nv_bfloat16* base = kv_bank + static_cast<long long>(ch) * T * row_elems + kh * kDD;
    for (int r = lane; r < T; r += 64) {
      // two rows per pass: 4 KB per lane pair of rows requested before any arithmetic
      const bool two = r + 32 < T;
      const uint4* kp0 = reinterpret_cast<const uint4*>(base + r * row_elems);
      const uint4* vp0 = reinterpret_cast<const uint4*>(base + r * row_elems + HK * kDD);
      const uint4* kp1 = reinterpret_cast<const uint4*>(base + (two ? r + 32 : r) * row_elems);
      const uint4* vp1 = reinterpret_cast<const uint4*>(base + (two ? r + 32 : r) * row_elems + HK * kDD);
      uint4 k0[kDD / 8], v0[kDD / 8], k1[kDD / 8], v1[kDD / 8];
#pragma unroll
      for (int i = 0; i < kDD / 8; ++i) k0[i] = kp0[i];
#pragma unroll
      for (int i = 0; i < kDD / 8; ++i) k1[i] = kp1[i];
#pragma unroll
      for (int i = 0; i < kDD / 8; ++i) v0[i] = vp0[i];
#pragma unroll
      for (int i = 0; i < kDD / 8; ++i) v1[i] = vp1[i];
      fold(k0, v0, u);
      if (two) fold(k1, v1, u);
    }
  }

  // lanes -> warp
  float mw = m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, o));
  const float f_lane = (m == -INFINITY) ? 0.f : exp2f(m - mw);
  l *= f_lane;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
#pragma unroll
  for (int i = 0; i < kDD; ++i) {
    float a = acc[i] * f_lane;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (lane == 0) red[warp][i] = a;
  }
  if (lane == 0) {
    red[warp][kDD] = mw;
    red[warp][kDD + 1] = l;
  }
  __syncthreads();
  // warps -> CTA: thread i < 64 finishes output element i
  if (threadIdx.x < kDD) {
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mt = fmaxf(mt, red[w][kDD]);
    float lt = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float f = (red[w][kDD] == -INFINITY) ? 0.f : exp2f(red[w][kDD] - mt);
      lt += red[w][kDD + 1] * f;
      a += red[w][threadIdx.x] * f;
    }
    const long long o = (static_cast<long long>(b) * n_q + iq) * H * kDD + h * kDD + threadIdx.x;
    out[o] = __float2bfloat16(lt > 0.f ? a / lt : 0.f);
    if (threadIdx.x == 0 && lse != nullptr)
      lse[(static_cast<long long>(b) * n_q + iq) * H + h] = lt > 0.f ? (mt + log2f(lt)) / kDecLog2e : -INFINITY;
  }
}

}  // namespace
}  // namespace moc

using namespace moc;

extern "C" int moc_decode_attn(const moc_decode_shape* s, const void* q, const void* kv_bank, int64_t bank_rows,
                               const int32_t* comb_idx, const float* comb_w, void* out, float* lse,
                               int32_t* status, void* stream_) {
  MOC_REQUIRE(s && q && kv_bank && comb_idx && comb_w && out && status, "NULL decode-attention argument");
  MOC_REQUIRE(s->head_dim == kDD, "decode attention needs head_dim 64");
  MOC_REQUIRE(s->batch > 0 && s->n_q > 0 && s->n_chapters > 0 && s->tokens_per_chapter > 0 && bank_rows > 0,
              "empty decode-attention problem");
  MOC_REQUIRE(s->num_heads > 0 && s->num_kv_heads > 0 && s->num_heads % s->num_kv_heads == 0,
              "num_heads must be a positive multiple of num_kv_heads");
  MOC_REQUIRE(s->n_q <= 65535 && s->batch <= 65535, "too many query tokens or sequences for one launch");
  MOC_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(kv_bank) & 15) == 0,
              "q and the K/V cache must be 16-byte aligned");
  dim3 grid(s->num_heads, s->n_q, s->batch);
  decode_attn_kernel<<<grid, kDecThreads, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(kv_bank), bank_rows, comb_idx, comb_w,
      static_cast<__nv_bfloat16*>(out), lse, s->n_q, s->num_heads, s->num_kv_heads, s->n_chapters,
      s->tokens_per_chapter, s->scale, status);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}
