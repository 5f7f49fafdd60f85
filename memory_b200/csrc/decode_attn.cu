// Decode-time memory attention over a cache of projected bank rows.
//
// The reference re-gathers (S+k)*T bank rows per sequence at every generated token and re-projects them with Wk / Wv
// (inference/generate.py:194-210 -> model.py:624-692 -> memory_attention.py:241-243).  The bank and the projections
// are constant while decoding, and the chapter weight multiplies a gathered row before the (linear) projection, so
//   K = (u_c * norm(m)) Wk^T = u_c * (norm(m) Wk^T)
// and a per-layer cache  KV_bank = norm(M) [Wk; Wv]^T  (bf16, [C*T, 2*HK*64]) turns the step into a gather of
// cached rows scaled by the chapter weight, followed by one joint softmax over all selected keys:
//   s_r = scale * u_c * <q, K_bank[r]>,   out = sum_r softmax(s)_r * u_c * V_bank[r].
// The kernel is bound by HBM: one CTA per (sequence, query token, head) streams the 128-byte K and V slices of the
// selected rows with coalesced requests and keeps the running softmax state in registers.
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

// Lane layout: eight lanes share a row (16 bytes of its 128-byte K slice and of its V slice each), so one warp load
// instruction touches four whole 128-byte lines instead of 32 scattered 16-byte pieces; a warp walks four rows per
// step.  Every 8-lane group keeps a running (max, sum) and each lane 8 of the 64 accumulators.
constexpr int kDecUnroll = 8;        // steps (of four rows) whose loads are issued before any arithmetic

__global__ void __launch_bounds__(kDecThreads, 2)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kv_bank,
                   long long bank_rows, const int* __restrict__ comb_idx, const float* __restrict__ comb_w,
                   __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int n_q, int H, int HK, int n_ch, int T,
                   float scale, int* __restrict__ status) {
  __shared__ float red[kDecWarps][kDD + 2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rg = lane >> 3, part = lane & 7;          // row group 0..3, 8-element slice of the head dimension
  const int h = blockIdx.x, iq = blockIdx.y, b = blockIdx.z;
  const int kh = h / (H / HK);
  const long long row_elems = 2ll * HK * kDD;

  float qf[8];
  unpack8(*reinterpret_cast<const uint4*>(q + (static_cast<long long>(b) * n_q + iq) * H * kDD + h * kDD + part * 8), qf);
  const float c2 = scale * kDecLog2e;
  float m = -INFINITY, l = 0.f;          // running maximum (log2 domain) and sum of this lane group's rows
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  for (int c = warp; c < n_ch; c += kDecWarps) {
    const int ch = comb_idx[b * n_ch + c];
    if (ch < 0 || (static_cast<long long>(ch) + 1) * T > bank_rows) {
      if (lane == 0) atomicMax(status, MOC_DEV_BAD_INDEX);
      continue;
    }
    const float u = comb_w[b * n_ch + c];
    const __nv_bfloat16* base = kv_bank + static_cast<long long>(ch) * T * row_elems + kh * kDD + part * 8;
    for (int r0 = 0; r0 < T; r0 += 4 * kDecUnroll) {
      uint4 kr[kDecUnroll], vr[kDecUnroll];
#pragma unroll
      for (int sidx = 0; sidx < kDecUnroll; ++sidx) {
        const int r = r0 + sidx * 4 + rg;
        const __nv_bfloat16* rp = base + static_cast<long long>(r < T ? r : 0) * row_elems;
        kr[sidx] = *reinterpret_cast<const uint4*>(rp);
        vr[sidx] = *reinterpret_cast<const uint4*>(rp + HK * kDD);
      }
#pragma unroll
      for (int sidx = 0; sidx < kDecUnroll; ++sidx) {
        const int r = r0 + sidx * 4 + rg;
        float f[8];
        unpack8(kr[sidx], f);
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) dot = fmaf(qf[j], f[j], dot);
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        if (r < T) {                                    // uniform within the 8-lane group
          const float sc = dot * u * c2;
          const float m_new = fmaxf(m, sc);
          const float corr = exp2f(m - m_new);          // 0 on the first row (m = -inf)
          const float pr = exp2f(sc - m_new);
          l = l * corr + pr;
          const float pu = pr * u;
          unpack8(vr[sidx], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = fmaf(acc[j], corr, pu * f[j]);
          m = m_new;
        }
      }
    }
  }

  // row groups -> warp (lanes with the same `part` hold the same 8 output elements)
  float mw = m;
  mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, 8));
  mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, 16));
  const float f_lane = (m == -INFINITY) ? 0.f : exp2f(m - mw);
  l *= f_lane;
  l += __shfl_xor_sync(0xffffffffu, l, 8);
  l += __shfl_xor_sync(0xffffffffu, l, 16);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float a = acc[j] * f_lane;
    a += __shfl_xor_sync(0xffffffffu, a, 8);
    a += __shfl_xor_sync(0xffffffffu, a, 16);
    if (rg == 0) red[warp][part * 8 + j] = a;
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
