// bf16 joint-softmax cross attention, backward, for sm_100a: two tcgen05 kernels, no atomics.
//
//  In both kernels two groups of four warps own the 128 rows of a tile: group g works on columns
//  [32g, 32g+32) of the score tile, which puts four row-owning warps on every scheduler partition.
//
//  dQ kernel  (query stationary, CTA = 128 queries of one head): per 64-key tile
//        S = Q K^T, dP = dO V^T            (SS MMAs into tensor memory)
//        dS = exp2(S*c - lse*log2e) * (dP - delta) * scale   (one query row per thread)
//        dQ += dS K                        (A = dS from tensor memory, B = K tile as MN-major operand)
//  dKV kernel (key stationary, CTA = 128 keys of one KV head): per 64-query tile of every head of
//  the KV group
//        S^T = K Q^T, dP^T = V dO^T        (SS MMAs; one key row per thread afterwards)
//        dV += P^T dO, dK += dS^T Q        (A = P^T / dS^T from tensor memory, written over the
//                                           columns S^T / dP^T occupied; B = dO / Q tiles MN-major)
// Recomputing S in both kernels costs 2 extra MMAs per tile pair against a fused 5-MMA backward
// but keeps every accumulator private to one CTA: results are deterministic.
#define MOC_KERNEL_TAG 3
#include "moc_common.cuh"

namespace moc {
namespace {

constexpr int kD = 64;
constexpr int kThreads = 320;      // two groups of 4 row-owning warps + TMA warp + MMA warp
constexpr int kStages = 3;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Three bf16 terms whose sum is x to ~24 bits, so that a tensor-core product with ones reproduces x.
__device__ __forceinline__ void split3_bf16(float x, uint32_t* t) {
  const __nv_bfloat16 hi = __float2bfloat16(x);
  const float r1 = x - __bfloat162float(hi);
  const __nv_bfloat16 mid = __float2bfloat16(r1);
  const __nv_bfloat16 lo = __float2bfloat16(r1 - __bfloat162float(mid));
  t[0] = __bfloat16_as_ushort(hi); t[1] = __bfloat16_as_ushort(mid); t[2] = __bfloat16_as_ushort(lo);
}

// delta[b,h,l] = <O, dO>; nlse2[b,h,l] = -lse * log2(e).  One warp per (b, l) row: lanes read 16-byte
// chunks of the H*64-wide row; a head is 8 chunks, reduced across 8 adjacent lanes.
// statb[b,h,l] = eight bf16: three terms of -lse / scale, three terms of -delta, two zeros -- the per-query
// operand row of the rank-16 products that add these per-column constants to S^T and dP^T in the dK/dV kernel.
__global__ void bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                const float* __restrict__ lse, float* __restrict__ delta,
                                float* __restrict__ nlse2, uint4* __restrict__ statb, float inv_scale, int B, int L,
                                int H) {
  const int lane = threadIdx.x & 31;
  const long long bl = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  if (bl >= static_cast<long long>(B) * L) return;
  const int l = static_cast<int>(bl % L);
  const int b = static_cast<int>(bl / L);
  const int chunks = H * (kD / 8);
  const uint4* po = reinterpret_cast<const uint4*>(o + bl * H * kD);
  const uint4* pd = reinterpret_cast<const uint4*>(d_o + bl * H * kD);
  for (int c0 = 0; c0 < chunks; c0 += 32) {
    const int c = c0 + lane;
    float acc = 0.f;
    if (c < chunks) {
      const uint4 a = po[c], g = pd[c];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(gw[i] << 16), acc);
        acc = fmaf(__uint_as_float(aw[i] & 0xFFFF0000u), __uint_as_float(gw[i] & 0xFFFF0000u), acc);
      }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (c < chunks && (lane & 7) == 0) {
      const int h = c >> 3;
      const long long idx = (static_cast<long long>(b) * H + h) * L + l;
      delta[idx] = acc;
      const float ls = lse[idx];
      nlse2[idx] = -ls * kLog2e;
      uint32_t a[3], d[3];
      split3_bf16(-ls * inv_scale, a);
      split3_bf16(-acc, d);
      statb[idx] = make_uint4(a[0] | (a[1] << 16), a[2] | (d[0] << 16), d[1] | (d[2] << 16), 0u);
    }
  }
}


// ---- MMA groups issued as one instruction block by one elected lane --------------------------------------
// The MMA warp shares its scheduler partition with busy row-owning warps, so the number of instructions per
// MMA, not the tensor pipe, sets the issue rate.  These blocks spend ~3 instructions per MMA (two address adds
// and the MMA) and interleave two independent accumulators: back-to-back MMAs into the same columns cannot
// start closer than ~94 cycles apart.
// Two K-major SS products over 4 K steps:  [d0] = A0 * B0^T,  [d1] = A1 * B1^T  (accumulators overwritten).
__device__ __forceinline__ void issue_ss_pair(uint32_t d0, uint32_t d1, uint64_t a0, uint64_t b0, uint64_t a1,
                                              uint64_t b1, uint32_t idesc) {
#define MOC_SS_STEP(KK, PACC)                                                                  \
  "add.s64 ta, %2, " #KK "*2;\n\t add.s64 tb, %3, " #KK "*2;\n\t"                               \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %6, " PACC ";\n\t"                      \
  "add.s64 ta, %4, " #KK "*2;\n\t add.s64 tb, %5, " #KK "*2;\n\t"                               \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%1], ta, tb, %6, " PACC ";\n\t"
  asm volatile(
      "{\n\t.reg .pred q, pt, pf;\n\t.reg .b64 ta, tb;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      MOC_SS_STEP(0, "pf") MOC_SS_STEP(1, "pt") MOC_SS_STEP(2, "pt") MOC_SS_STEP(3, "pt")
      "}"
      ::"r"(d0), "r"(d1), "l"(a0), "l"(b0), "l"(a1), "l"(b1), "r"(idesc)
      : "memory");
#undef MOC_SS_STEP
}
// One TS product over 4 K steps with MN-major B: [d] += A * B, A K step kk at column a + 8 kk.
__device__ __forceinline__ void issue_ts_single(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
#define MOC_TS1_STEP(KK, PACC)                                                                 \
  "add.u32 ca, %1, " #KK "*8;\n\t add.s64 tb, %2, " #KK "*128;\n\t"                              \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [ca], tb, %3, " PACC ";\n\t"
  asm volatile(
      "{\n\t.reg .pred q, pa, pt;\n\t.reg .b64 tb;\n\t.reg .b32 ca;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.ne.b32 pa, %4, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      MOC_TS1_STEP(0, "pa") MOC_TS1_STEP(1, "pt") MOC_TS1_STEP(2, "pt") MOC_TS1_STEP(3, "pt")
      "}"
      ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
#undef MOC_TS1_STEP
}

// One SS product over 4 K steps, A K-major, B K-major (BSTEP 2) or MN-major (BSTEP 128): [d] (+)= A * B.
template <int BSTEP>
__device__ __forceinline__ void issue_ss_one(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
#define MOC_SS1_STEP(KK, PACC)                                                                 \
  "add.s64 ta, %1, " #KK "*2;\n\t add.s64 tb, %2, " #KK "*%5;\n\t"                              \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, " PACC ";\n\t"
  asm volatile(
      "{\n\t.reg .pred q, pa, pt;\n\t.reg .b64 ta, tb;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.ne.b32 pa, %4, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      MOC_SS1_STEP(0, "pa") MOC_SS1_STEP(1, "pt") MOC_SS1_STEP(2, "pt") MOC_SS1_STEP(3, "pt")
      "}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "n"(BSTEP)
      : "memory");
#undef MOC_SS1_STEP
}
// One accumulating SS MMA (a single K step of 16).
__device__ __forceinline__ void issue_ss_k16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred q, pt;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pt;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc)
      : "memory");
}
// Shared-memory descriptor of a K-major operand without swizzle: 8-row x 16-byte core matrices, `lbo` bytes
// between the two core matrices of a K step, `sbo` bytes between 8-row groups.
__device__ __forceinline__ uint64_t umma_desc_plain(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  return d;
}
// One TS product with MN-major B, A K step kk at column a + (kk >> 1) * a_hi + (kk & 1) * 8: [d] += A * B.
__device__ __forceinline__ void issue_ts_one_hi(uint32_t d, uint32_t a, uint32_t a_hi, uint64_t b, uint32_t idesc,
                                                uint32_t acc) {
#define MOC_TSH_STEP(KK, HI, LO, PACC)                                                         \
  "mad.lo.u32 ca, %2, " #HI ", %1;\n\t add.u32 ca, ca, " #LO ";\n\t add.s64 tb, %3, " #KK "*128;\n\t" \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [ca], tb, %4, " PACC ";\n\t"
  asm volatile(
      "{\n\t.reg .pred q, pa, pt;\n\t.reg .b64 tb;\n\t.reg .b32 ca;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.ne.b32 pa, %5, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      MOC_TSH_STEP(0, 0, 0, "pa") MOC_TSH_STEP(1, 0, 8, "pt") MOC_TSH_STEP(2, 1, 0, "pt") MOC_TSH_STEP(3, 1, 8, "pt")
      "}"
      ::"r"(d), "r"(a), "r"(a_hi), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
#undef MOC_TSH_STEP
}
// ------------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------------
constexpr int kQ = 128, kKeys = 64;
constexpr int kQBytes = kQ * kD * 2;        // 16 KiB (Q and dO tiles)
constexpr int kKvBytes = kKeys * kD * 2;    // 8 KiB
constexpr int kDqSmem = 2 * kQBytes + kStages * 2 * kKvBytes + 1024;
constexpr uint32_t kDqColS = 0, kDqColDP = 64, kDqColDQ = 128, kDqColDS = 192;   // 224 columns used

struct DqParams {
  __nv_bfloat16* d_q;
  const float* delta;
  const float* nlse2;
  int L, n_sel, H, HK;
  float scale, scale_log2;
  int* status;
};

__global__ void __launch_bounds__(kThreads, 2)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                      const __grid_constant__ CUtensorMap tmap_kv, DqParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_bar, kv_full[kStages], kv_empty[kStages], sdp_full, sdp_free, ds_full, dq_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = base;
  uint8_t* do_s = base + kQBytes;
  uint8_t* kv_s = base + 2 * kQBytes;
  const int q0 = blockIdx.x * kQ, h = blockIdx.y, b = blockIdx.z;
  const int kh = h / (p.H / p.HK);
  const int n_tiles = (p.n_sel + kKeys - 1) / kKeys;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&q_bar, 1);
    for (int s = 0; s < kStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(&sdp_full, 1);
    mbar_init(&sdp_free, 256);
    mbar_init(&ds_full, 256);
    mbar_init(&dq_bar, 1);
    fence_mbar_init();
    prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do); prefetch_tmap(&tmap_kv);
  }
  if (warp == 9) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 8) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&q_bar, 2 * kQBytes);
      tma_load_2d(q_s, &tmap_q, &q_bar, h * kD, b * p.L + q0);
      tma_load_2d(do_s, &tmap_do, &q_bar, h * kD, b * p.L + q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kStages;
        if (!mbar_wait(&kv_empty[s], ((j / kStages) & 1) ^ 1, &abort_flag, p.status)) break;
        mbar_arrive_expect_tx(&kv_full[s], 2 * kKvBytes);
        uint8_t* k_s = kv_s + s * 2 * kKvBytes;
        const int row = b * p.n_sel + j * kKeys;
        tma_load_2d(k_s, &tmap_kv, &kv_full[s], kh * kD, row);
        tma_load_2d(k_s + kKvBytes, &tmap_kv, &kv_full[s], p.HK * kD + kh * kD, row);
      }
    }
  } else if (warp == 9) {
    {   // warp-uniform: every lane runs the loop, one elected lane issues
      const uint32_t idesc_kk = umma_idesc_bf16(kQ, kKeys, 0, 0);   // S and dP: both operands K-major
      const uint32_t idesc_dq = umma_idesc_bf16(kQ, kD, 0, 1);      // dQ: B = K tile, MN-major
      // descriptors are built once; a stage or K step only adds a constant to the address field
      const uint64_t q_desc = umma_desc_sw128(smem_u32(q_s), 16, 1024);
      const uint64_t do_desc = umma_desc_sw128(smem_u32(do_s), 16, 1024);
      const uint64_t k_desc0 = umma_desc_sw128(smem_u32(kv_s), 16, 1024);                  // K tile, K-major
      const uint64_t v_desc0 = umma_desc_sw128(smem_u32(kv_s) + kKvBytes, 16, 1024);       // V tile, K-major
      const uint64_t kmn_desc0 = umma_desc_sw128(smem_u32(kv_s), 8192, 1024);              // K tile, MN-major
      constexpr uint64_t kStageOff = (2 * kKvBytes) >> 4;
      bool ok = mbar_wait_w(&q_bar, 0, &abort_flag, p.status);
      for (int j = 0; j <= n_tiles && ok; ++j) {
        if (j < n_tiles) {
          const int s = j % kStages;
          ok = mbar_wait_w(&kv_full[s], (j / kStages) & 1, &abort_flag, p.status);
          if (ok && j > 0) ok = mbar_wait_w(&sdp_free, (j - 1) & 1, &abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint64_t kd = k_desc0 + s * kStageOff, vd = v_desc0 + s * kStageOff;
          issue_ss_pair(tmem + kDqColS, tmem + kDqColDP, q_desc, kd, do_desc, vd, idesc_kk);
          tc_commit_w(&sdp_full);
        }
        if (j > 0) {
          const int jp = j - 1, s = jp % kStages;
          ok = mbar_wait_w(&ds_full, jp & 1, &abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint64_t kd = kmn_desc0 + s * kStageOff;
          issue_ts_single(tmem + kDqColDQ, tmem + kDqColDS, kd, idesc_dq, jp > 0 ? 1u : 0u);
          tc_commit_w(&kv_empty[s]);
          tc_commit_w(&dq_bar);
        }
      }
    }
  } else {
    // row-owning warps: warp & 3 selects the 32 TMEM lanes, warp >> 2 the column half
    const int half = warp >> 2;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int row = (warp & 3) * 32 + lane;
    const int l = q0 + row;
    const long long sidx = (static_cast<long long>(b) * p.H + h) * p.L + (l < p.L ? l : 0);
    const float nl = p.nlse2[sidx], dl = p.delta[sidx];
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = mbar_wait(&sdp_full, j & 1, &abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int valid = p.n_sel - j * kKeys - half * 32;   // columns of this half that are real keys
      uint32_t pk[16];
      {
        uint32_t rs[32], rd[32];
        tmem_ld32(tmem + lane_sel + kDqColS + half * 32, rs);
        tmem_ld32(tmem + lane_sel + kDqColDP + half * 32, rd);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&sdp_free);          // S / dP may be overwritten by the next tile's MMAs
        // dS without the softmax scale: it is applied once when dQ is written
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float d0 = ex2(fmaf(__uint_as_float(rs[c]), p.scale_log2, nl)) * (__uint_as_float(rd[c]) - dl);
          const float d1 = ex2(fmaf(__uint_as_float(rs[c + 1]), p.scale_log2, nl)) * (__uint_as_float(rd[c + 1]) - dl);
          pk[c / 2] = pack_bf16x2(d0, d1);
        }
        if (valid < 32) {
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            if (c >= valid) pk[c / 2] = 0u;
            else if (c + 1 >= valid) pk[c / 2] &= 0x0000FFFFu;
          }
        }
      }
      if (j > 0) {
        ok = mbar_wait(&dq_bar, (j - 1) & 1, &abort_flag, p.status);   // previous dS consumed
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
      }
      tmem_st16(tmem + lane_sel + kDqColDS + half * 16, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&ds_full);
    }
    if (ok) {
      ok = mbar_wait(&dq_bar, (n_tiles - 1) & 1, &abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dst = p.d_q + (static_cast<long long>(b) * p.L + l) * (p.H * kD) + h * kD + half * 32;
      uint32_t r[32];
      tmem_ld32(tmem + lane_sel + kDqColDQ + half * 32, r);
      tmem_wait_ld();
      if (l < p.L) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[8 * c + 0]) * p.scale, __uint_as_float(r[8 * c + 1]) * p.scale);
          v.y = pack_bf16x2(__uint_as_float(r[8 * c + 2]) * p.scale, __uint_as_float(r[8 * c + 3]) * p.scale);
          v.z = pack_bf16x2(__uint_as_float(r[8 * c + 4]) * p.scale, __uint_as_float(r[8 * c + 5]) * p.scale);
          v.w = pack_bf16x2(__uint_as_float(r[8 * c + 6]) * p.scale, __uint_as_float(r[8 * c + 7]) * p.scale);
          *reinterpret_cast<uint4*>(dst + c * 8) = v;
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (abort_flag) { for (int i = 0; i < 200; ++i) __nanosleep(1000); }
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

// ------------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------------
constexpr int kKeysB = 128, kQB = 64;
constexpr int kKBytes = kKeysB * kD * 2;     // 16 KiB (K and V tiles, stationary)
constexpr int kQTileBytes = kQB * kD * 2;    // 8 KiB (Q and dO tiles, streamed)
constexpr int kStatBytes = kQB * 16;         // 1 KiB: the 16-byte constant row of each query, streamed
constexpr int kStageB = 2 * kQTileBytes;      // tile ring stride (keeps every tile 1024-byte aligned)
constexpr int kStageTx = kStageB + kStatBytes;
constexpr int kPtBytes = kKeysB * kQB * 2;   // 16 KiB: P^T tile, the A operand of the dV product
constexpr int kOnesBytes = kKeysB * 16;      // 2 KiB: a 128 x 8 selector operand / its zero second half
constexpr int kDkvSmem = 2 * kKBytes + kStages * kStageB + kPtBytes + kStages * kStatBytes + 3 * kOnesBytes + 1024;
constexpr uint32_t kColST = 0, kColDPT = 64, kColDV = 128, kColDK = 192;   // dS^T aliases dP^T

struct DkvParams {
  const float* row_scale;  // optional per-key-row factor applied to dK and dV when they are written, or nullptr
  float* kv_dot;           // optional [B, n_sel / 64, HK]: per 64-key block and KV head, sum over its rows of
                           // <dK, K> + <dV, V> (the chapter-weight gradient up to 1 / weight), or nullptr
  __nv_bfloat16* d_kv;
  int dkv_tma;             // d_kv written through staging blocks and TMA stores (n_sel % 32 == 0)
  const uint4* statb;
  int L, n_sel, H, HK;
  float scale, scale_log2;
  int* status;
};

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Software pipeline over the query tiles j of one CTA (tensor memory: S^T, dP^T, dV, dK, 64 columns each):
//   MMA warp :  S^T_{j+1} = K Q_{j+1}^T   as soon as the row owners hold S^T_j in registers
//               dV += P^T_j dO_j          A = P^T_j from shared memory (written by the row owners)
//               dK += dS^T_j Q_j          A = dS^T_j from tensor memory, over dP^T_j's columns
//               dP^T_{j+1} = V dO_{j+1}^T after dK_j in issue order, because it overwrites dS^T_j
//   row owners: P^T_j = exp2(S^T_j c - lse c) -> shared memory;  dS^T_j = P^T_j (dP^T_j - delta) -> tensor memory
// so the exponentials of tile j run while the tensor pipe computes S^T_{j+1}, dV_{j-1}... and neither side
// waits for the other in steady state.  P^T lives in shared memory so that S^T's columns are free early.
__global__ void __launch_bounds__(kThreads, 2)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                       const __grid_constant__ CUtensorMap tmap_kv, const __grid_constant__ CUtensorMap tmap_dkv,
                       DkvParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t k_bar, q_full[kStages], q_empty[kStages], s_full, s_free, dp_full, p_full, p_free,
      ds_full, acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = base;
  uint8_t* v_s = base + kKBytes;
  uint8_t* ring = base + 2 * kKBytes;
  uint8_t* pt_s = ring + kStages * kStageB;
  uint8_t* stats = pt_s + kPtBytes;                  // kStages x 64 rows of 16 bytes
  uint8_t* sel_s = stats + kStages * kStatBytes;     // 128 rows (1,1,1,0,0,0,0,0): picks the -lse terms
  uint8_t* sel_d = sel_s + kOnesBytes;               // 128 rows (0,0,0,1,1,1,0,0): picks the -delta terms
  uint8_t* zeros = sel_d + kOnesBytes;               // second half of every rank-16 operand
  const int key0 = blockIdx.x * kKeysB, kh = blockIdx.y, b = blockIdx.z;
  const int G = p.H / p.HK;
  const int q_tiles = p.L / kQB;
  const int n_iter = G * q_tiles;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&k_bar, 1);
    for (int s = 0; s < kStages; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    mbar_init(&s_full, 1);
    mbar_init(&s_free, 256);
    mbar_init(&dp_full, 1);
    mbar_init(&p_full, 256);
    mbar_init(&p_free, 1);
    mbar_init(&ds_full, 256);
    mbar_init(&acc_bar, 1);
    fence_mbar_init();
    prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do); prefetch_tmap(&tmap_kv);
  }
  if (threadIdx.x < kKeysB) {
    reinterpret_cast<uint4*>(sel_s)[threadIdx.x] = make_uint4(0x3F803F80u, 0x00003F80u, 0u, 0u);
    reinterpret_cast<uint4*>(sel_d)[threadIdx.x] = make_uint4(0u, 0x3F800000u, 0x3F803F80u, 0u);
    reinterpret_cast<uint4*>(zeros)[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
  }
  fence_proxy_async();
  if (warp == 9) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 8) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&k_bar, 2 * kKBytes);
      const int row = b * p.n_sel + key0;
      tma_load_2d(k_s, &tmap_kv, &k_bar, kh * kD, row);
      tma_load_2d(k_s + kKBytes / 2, &tmap_kv, &k_bar, kh * kD, row + 64);
      tma_load_2d(v_s, &tmap_kv, &k_bar, p.HK * kD + kh * kD, row);
      tma_load_2d(v_s + kKBytes / 2, &tmap_kv, &k_bar, p.HK * kD + kh * kD, row + 64);
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % kStages;
        if (!mbar_wait(&q_empty[s], ((it / kStages) & 1) ^ 1, &abort_flag, p.status)) break;
        const int h = kh * G + it / q_tiles, l0 = (it % q_tiles) * kQB;
        uint8_t* st = ring + s * kStageB;
        mbar_arrive_expect_tx(&q_full[s], kStageTx);
        tma_load_2d(st, &tmap_q, &q_full[s], h * kD, b * p.L + l0);
        tma_load_2d(st + kQTileBytes, &tmap_do, &q_full[s], h * kD, b * p.L + l0);
        const long long soff = (static_cast<long long>(b) * p.H + h) * p.L + l0;
        bulk_load_1d(stats + s * kStatBytes, p.statb + soff, kStatBytes, &q_full[s]);
      }
    }
  } else if (warp == 9) {
    {   // warp-uniform: every lane runs the loop, one elected lane issues
      const uint32_t idesc_s = umma_idesc_bf16(kKeysB, kQB, 0, 0);   // S^T, dP^T
      const uint32_t idesc_g = umma_idesc_bf16(kKeysB, kD, 0, 1);    // dV, dK: B = dO / Q tile, MN-major
      // descriptors are built once; a stage or K step only adds a constant to the address field
      const uint64_t k_desc = umma_desc_sw128(smem_u32(k_s), 16, 1024);
      const uint64_t v_desc = umma_desc_sw128(smem_u32(v_s), 16, 1024);
      const uint64_t pt_desc = umma_desc_sw128(smem_u32(pt_s), 16, 1024);                      // P^T, K-major
      const uint64_t q_desc0 = umma_desc_sw128(smem_u32(ring), 16, 1024);                      // Q tile, K-major
      const uint64_t do_desc0 = umma_desc_sw128(smem_u32(ring) + kQTileBytes, 16, 1024);       // dO tile, K-major
      const uint64_t qmn_desc0 = umma_desc_sw128(smem_u32(ring), 8192, 1024);                  // Q tile, MN-major
      const uint64_t domn_desc0 = umma_desc_sw128(smem_u32(ring) + kQTileBytes, 8192, 1024);   // dO tile, MN-major
      // rank-16 products that add the per-query constants: D[key, q] += sum_k sel[key, k] * stat[q, k]
      const uint64_t sel_s_desc = umma_desc_plain(smem_u32(sel_s), smem_u32(zeros) - smem_u32(sel_s), 128);
      const uint64_t sel_d_desc = umma_desc_plain(smem_u32(sel_d), smem_u32(zeros) - smem_u32(sel_d), 128);
      const uint64_t stat_desc0 = umma_desc_plain(smem_u32(stats), smem_u32(zeros) - smem_u32(stats), 128);
      constexpr uint64_t kStageOff = kStageB >> 4;
      constexpr uint64_t kStatOff = kStatBytes >> 4;
      // the zero block is addressed relative to each stage's constant rows
      constexpr uint64_t kStatLboStep = static_cast<uint64_t>(kStatBytes >> 4) << 16;
      bool ok = mbar_wait_w(&k_bar, 0, &abort_flag, p.status);
      if (ok && n_iter > 0) {
        ok = mbar_wait_w(&q_full[0], 0, &abort_flag, p.status);
        if (ok) {
          tc_fence_after();
          issue_ss_pair(tmem + kColST, tmem + kColDPT, k_desc, q_desc0, v_desc, do_desc0, idesc_s);
          issue_ss_k16(tmem + kColST, sel_s_desc, stat_desc0, idesc_s);
          issue_ss_k16(tmem + kColDPT, sel_d_desc, stat_desc0, idesc_s);
          tc_commit_w(&s_full);
          tc_commit_w(&dp_full);
        }
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % kStages;
        const bool more = it + 1 < n_iter;
        const int sn = (it + 1) % kStages;
        if (more) {
          ok = mbar_wait_w(&q_full[sn], ((it + 1) / kStages) & 1, &abort_flag, p.status);
          if (!ok) break;
          ok = mbar_wait_w(&s_free, it & 1, &abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          issue_ss_one<2>(tmem + kColST, k_desc, q_desc0 + sn * kStageOff, idesc_s, 0u);
          issue_ss_k16(tmem + kColST, sel_s_desc, stat_desc0 + sn * kStatOff - sn * kStatLboStep, idesc_s);
          tc_commit_w(&s_full);
        }
        ok = mbar_wait_w(&p_full, it & 1, &abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        issue_ss_one<128>(tmem + kColDV, pt_desc, domn_desc0 + s * kStageOff, idesc_g, it > 0 ? 1u : 0u);
        tc_commit_w(&p_free);
        ok = mbar_wait_w(&ds_full, it & 1, &abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        // dS^T for queries [32g, 32g+32) sits in the first 16 columns of column half g of dP^T
        issue_ts_one_hi(tmem + kColDK, tmem + kColDPT, 32, qmn_desc0 + s * kStageOff, idesc_g, it > 0 ? 1u : 0u);
        tc_commit_w(&q_empty[s]);
        if (more) {
          // strictly after dK_j: the first K step already overwrites all of dS^T_j's columns
          issue_ss_one<2>(tmem + kColDPT, v_desc, do_desc0 + sn * kStageOff, idesc_s, 0u);
          issue_ss_k16(tmem + kColDPT, sel_d_desc, stat_desc0 + sn * kStatOff - sn * kStatLboStep, idesc_s);
          tc_commit_w(&dp_full);
        }
      }
      tc_commit_w(&acc_bar);
    }
  } else {
    const int half = warp >> 2;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int row = (warp & 3) * 32 + lane;
    // this thread's 64 bytes of P^T row `row`: 16-byte chunks 4*half .. 4*half+3 under the 128-byte swizzle
    const uint32_t pt_row = smem_u32(pt_s) + row * 128;
    const uint32_t sw = static_cast<uint32_t>(row & 7);
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      ok = mbar_wait(&s_full, it & 1, &abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float pf[32];
      {
        uint32_t rs[32];
        tmem_ld32(tmem + lane_sel + kColST + half * 32, rs);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&s_free);          // S^T_j is in registers: its columns may take S^T_{j+1}
        // the tensor core already added -lse / scale to every column
#pragma unroll
        for (int c = 0; c < 32; ++c) pf[c] = ex2(__uint_as_float(rs[c]) * p.scale_log2);
      }
      if (it > 0) {
        ok = mbar_wait(&p_free, (it - 1) & 1, &abort_flag, p.status);   // dV_{j-1} has read the P^T tile
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t addr = pt_row + (((static_cast<uint32_t>(half) * 4 + c) ^ sw) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                     "r"(pack_bf16x2(pf[8 * c + 0], pf[8 * c + 1])), "r"(pack_bf16x2(pf[8 * c + 2], pf[8 * c + 3])),
                     "r"(pack_bf16x2(pf[8 * c + 4], pf[8 * c + 5])), "r"(pack_bf16x2(pf[8 * c + 6], pf[8 * c + 7]))
                     : "memory");
      }
      fence_proxy_async();
      mbar_arrive(&p_full);
      ok = mbar_wait(&dp_full, it & 1, &abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t rd[32], pd[16];
        tmem_ld32(tmem + lane_sel + kColDPT + half * 32, rd);
        tmem_wait_ld();
        // dS^T = P^T (dP^T - delta) without the softmax scale (applied once when dK is written); the
        // tensor core already subtracted delta from every column
#pragma unroll
        for (int c = 0; c < 32; c += 2)
          pd[c / 2] = pack_bf16x2(pf[c] * __uint_as_float(rd[c]), pf[c + 1] * __uint_as_float(rd[c + 1]));
        // this thread has read every fp32 value of its row in this column half: overwrite its first 16 columns
        tmem_st16(tmem + lane_sel + kColDPT + half * 32, pd);
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive(&ds_full);
    }
    if (ok) {
      ok = mbar_wait(&acc_bar, 0, &abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
    }
    float kv_dot_part = 0.f;        // this thread's share of sum_rows (<dK, K> + <dV, V>) for its key row and column half
    if (p.dkv_tma) {
      // One thread owns one key row, so direct stores would scatter 16-byte pieces over 32 rows per instruction.
      // The tile ring is idle now: each (lane quarter, dK | dV) gets a 32-row x 128-byte swizzled block there,
      // filled by the two warps that own its column halves, and leaves as one TMA store.
      const int quarter = warp & 3;
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int which = 0; which < 2; ++which) {      // 0: dK (carries the softmax scale), 1: dV
          uint32_t r[32];
          tmem_ld32(tmem + lane_sel + (which ? kColDV : kColDK) + half * 32, r);
          tmem_wait_ld();
          const int krow = key0 + quarter * 32 + lane;
          const float rsf = (p.row_scale != nullptr && krow < p.n_sel)
                                ? p.row_scale[static_cast<long long>(b) * p.n_sel + krow] : 1.f;
          const float f = (which ? 1.f : p.scale) * rsf;
          if (p.kv_dot != nullptr && krow < p.n_sel) {
            // the stationary K / V tile is still in shared memory (two 64-row boxes, 128-byte rows, swizzled)
            const int rr = quarter * 32 + lane;
            const uint8_t* tile = (which ? v_s : k_s) + (rr >> 6) * (kKBytes / 2) + (rr & 63) * 128;
            float acc = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint4 kvv = *reinterpret_cast<const uint4*>(tile + ((static_cast<uint32_t>(half * 4 + c) ^ (rr & 7)) << 4));
              const uint32_t w4[4] = {kvv.x, kvv.y, kvv.z, kvv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                acc = fmaf(__uint_as_float(r[8 * c + 2 * e]), __uint_as_float(w4[e] << 16), acc);
                acc = fmaf(__uint_as_float(r[8 * c + 2 * e + 1]), __uint_as_float(w4[e] & 0xFFFF0000u), acc);
              }
            }
            kv_dot_part = fmaf(acc, which ? 1.f : p.scale, kv_dot_part);
          }
          const uint32_t row_addr = smem_u32(ring) + (quarter * 2 + which) * 4096 + lane * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t addr = row_addr + ((static_cast<uint32_t>(half * 4 + c) ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                         "r"(pack_bf16x2(__uint_as_float(r[8 * c + 0]) * f, __uint_as_float(r[8 * c + 1]) * f)),
                         "r"(pack_bf16x2(__uint_as_float(r[8 * c + 2]) * f, __uint_as_float(r[8 * c + 3]) * f)),
                         "r"(pack_bf16x2(__uint_as_float(r[8 * c + 4]) * f, __uint_as_float(r[8 * c + 5]) * f)),
                         "r"(pack_bf16x2(__uint_as_float(r[8 * c + 6]) * f, __uint_as_float(r[8 * c + 7]) * f))
                         : "memory");
          }
        }
        fence_proxy_async();
      }
      if (p.kv_dot != nullptr) {
        // 64-key block c of this tile = lane quarters 2c, 2c+1 and both column halves: four warps; the sum is
        // formed in a fixed order (warp shuffle tree, then the four partials in warp order)
        const float wsum = warp_sum(ok ? kv_dot_part : 0.f);
        float* part = reinterpret_cast<float*>(stats);         // the constant rows are no longer read
        if (lane == 0) part[warp] = wsum;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (ok && warp < 2 && lane == 0) {
          const int blk = key0 / 64 + warp;
          if (blk * 64 < p.n_sel) {
            const float t = part[2 * warp] + part[2 * warp + 1] + part[4 + 2 * warp] + part[4 + 2 * warp + 1];
            p.kv_dot[(static_cast<long long>(b) * (p.n_sel / 64) + blk) * p.HK + kh] = t;
          }
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");     // the eight row-owning warps, whatever `ok` is
      if (ok && half == 0 && lane == 0 && key0 + quarter * 32 < p.n_sel) {
        const int grow = b * p.n_sel + key0 + quarter * 32;
        tma_store_2d(&tmap_dkv, ring + (quarter * 2) * 4096, kh * kD, grow);
        tma_store_2d(&tmap_dkv, ring + (quarter * 2 + 1) * 4096, p.HK * kD + kh * kD, grow);
        bulk_commit_group();
        bulk_wait_all();
      }
    } else if (ok) {
      tc_fence_after();
      const int key = key0 + row;
      __nv_bfloat16* dst = p.d_kv + (static_cast<long long>(b) * p.n_sel + key) * (2 * p.HK * kD) + kh * kD + half * 32;
#pragma unroll
      for (int which = 0; which < 2; ++which) {      // 0: dK (carries the softmax scale), 1: dV
        uint32_t r[32];
        tmem_ld32(tmem + lane_sel + (which ? kColDV : kColDK) + half * 32, r);
        tmem_wait_ld();
        const float rsf = (p.row_scale != nullptr && key < p.n_sel)
                              ? p.row_scale[static_cast<long long>(b) * p.n_sel + key] : 1.f;
        const float f = (which ? 1.f : p.scale) * rsf;
        if (key < p.n_sel) {
          __nv_bfloat16* d2 = dst + (which ? p.HK * kD : 0);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * c + 0]) * f, __uint_as_float(r[8 * c + 1]) * f);
            v.y = pack_bf16x2(__uint_as_float(r[8 * c + 2]) * f, __uint_as_float(r[8 * c + 3]) * f);
            v.z = pack_bf16x2(__uint_as_float(r[8 * c + 4]) * f, __uint_as_float(r[8 * c + 5]) * f);
            v.w = pack_bf16x2(__uint_as_float(r[8 * c + 6]) * f, __uint_as_float(r[8 * c + 7]) * f);
            *reinterpret_cast<uint4*>(d2 + c * 8) = v;
          }
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (abort_flag) { for (int i = 0; i < 200; ++i) __nanosleep(1000); }
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

}  // namespace

int launch_attn_tc_bwd(const moc_attn_shape* s, const void* q, const void* kv, const void* o, const float* lse,
                       const void* d_o, void* d_q, void* d_kv, float* scratch, int32_t* status,
                       cudaStream_t stream, int parts, const float* kv_row_scale, float* kv_dot) {
  MOC_REQUIRE(s->head_dim == kD, "bf16 attention needs head_dim 64");
  MOC_REQUIRE(s->seq % kQB == 0, "bf16 attention backward needs seq % 64 == 0");
  MOC_REQUIRE(s->num_heads % s->num_kv_heads == 0, "num_heads must be a multiple of num_kv_heads");
  const int B = s->batch, L = s->seq, H = s->num_heads, HK = s->num_kv_heads;
  float* delta = scratch;
  float* nlse2 = scratch + static_cast<long long>(B) * H * L;
  uint4* statb = reinterpret_cast<uint4*>(scratch + 2ll * B * H * L);
  MOC_REQUIRE((reinterpret_cast<uintptr_t>(statb) & 15) == 0, "attention backward scratch must be 16-byte aligned");
  if (parts & 1) {
    const long long total = static_cast<long long>(B) * L;
    const int blocks = static_cast<int>((total * 32 + 255) / 256);
    bwd_prep_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(o),
                                                static_cast<const __nv_bfloat16*>(d_o), lse, delta, nlse2, statb,
                                                1.0f / s->scale, B, L, H);
  }
  CUtensorMap tq128, tdo128, tq64, tdo64, tkv;
  const uint64_t qrows = static_cast<uint64_t>(B) * L, qcols = static_cast<uint64_t>(H) * kD;
  const uint64_t kvrows = static_cast<uint64_t>(B) * s->n_sel, kvcols = static_cast<uint64_t>(2 * HK) * kD;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tq128, q, qrows, qcols, qcols, kQ, kD)) != MOC_OK) return rc;
  if ((rc = make_tmap_bf16_2d(&tdo128, d_o, qrows, qcols, qcols, kQ, kD)) != MOC_OK) return rc;
  if ((rc = make_tmap_bf16_2d(&tq64, q, qrows, qcols, qcols, kQB, kD)) != MOC_OK) return rc;
  if ((rc = make_tmap_bf16_2d(&tdo64, d_o, qrows, qcols, qcols, kQB, kD)) != MOC_OK) return rc;
  if ((rc = make_tmap_bf16_2d(&tkv, kv, kvrows, kvcols, kvcols, 64, kD)) != MOC_OK) return rc;
  MOC_CUDA_OK(cudaFuncSetAttribute(attn_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqSmem));
  MOC_CUDA_OK(cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDkvSmem));
  if (parts & 2) {
    DqParams p;
    p.d_q = static_cast<__nv_bfloat16*>(d_q); p.delta = delta; p.nlse2 = nlse2;
    p.L = L; p.n_sel = s->n_sel; p.H = H; p.HK = HK;
    p.scale = s->scale; p.scale_log2 = s->scale * kLog2e; p.status = status;
    dim3 grid(ceil_div(L, kQ), H, B);
    attn_bwd_dq_tc_kernel<<<grid, kThreads, kDqSmem, stream>>>(tq128, tdo128, tkv, p);
  }
  if (parts & 4) {
    DkvParams p;
    CUtensorMap tdkv = tkv;      // placeholder when the TMA-store epilogue is not used
    p.dkv_tma = (s->n_sel % 32 == 0 && (reinterpret_cast<uintptr_t>(d_kv) & 15) == 0) ? 1 : 0;
    if (p.dkv_tma && (rc = make_tmap_bf16_2d(&tdkv, d_kv, kvrows, kvcols, kvcols, 32, kD)) != MOC_OK) return rc;
    p.d_kv = static_cast<__nv_bfloat16*>(d_kv); p.statb = statb; p.row_scale = kv_row_scale;
    p.kv_dot = kv_dot;
    if (kv_dot != nullptr)
      MOC_REQUIRE(p.dkv_tma && s->n_sel % 64 == 0, "the per-block <dKV, KV> sums need n_sel % 64 == 0 and an aligned d_kv");
    p.L = L; p.n_sel = s->n_sel; p.H = H; p.HK = HK;
    p.scale = s->scale; p.scale_log2 = s->scale * kLog2e; p.status = status;
    dim3 grid(ceil_div(s->n_sel, kKeysB), HK, B);
    attn_bwd_dkv_tc_kernel<<<grid, kThreads, kDkvSmem, stream>>>(tq64, tdo64, tkv, tdkv, p);
  }
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

}  // namespace moc
