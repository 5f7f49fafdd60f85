// bf16 joint-softmax cross attention, forward, for sm_100a.
//
// One CTA = 128 queries of one (batch, head); it streams the (S+k) gathered chapters as tiles of
// 64 keys:   S_j = Q K_j^T  (tcgen05.mma, operands in 128-byte-swizzled shared memory filled by TMA,
// accumulator in tensor memory) -> online softmax by 128 threads that each own one query row
// (tcgen05.ld, exp2 on the scaled scores, P written back to tensor memory as packed bf16) ->
// O += P_j V_j (tcgen05.mma with A = P from tensor memory, B = the V tile as an MN-major operand).
// A CTA holds 256 TMEM columns -- two 64-column score buffers (tile j uses buffer j & 1; P_j is written
// as packed bf16 over the first 32 columns of its own buffer) and the 64-column O accumulator -- about
// 65 KiB of shared memory and 192 threads, and two CTAs share an SM (__launch_bounds__(192, 2)).  S_{j+1}
// is issued before PV_j, so the tensor pipe computes the next scores while the row owners run the softmax
// of the current ones; the second CTA fills what is left of the strictly ordered chain.  The
// running maximum is only raised (and O rescaled) when it grows by more than 2^8, which keeps P
// within bf16 range while skipping almost every rescale.
#define MOC_KERNEL_TAG 2
#include "moc_common.cuh"

namespace moc {
namespace {

constexpr int kQ = 128;          // queries per CTA
constexpr int kKeys = 64;        // keys per tile
constexpr int kD = 64;           // head dim
constexpr int kStages = 3;       // K/V ring depth (K_j is read one tile before V_j)
constexpr int kThreads = 192;    // 4 softmax warps + TMA warp + MMA warp
constexpr int kQBytes = kQ * kD * 2;
constexpr int kTileBytes = kKeys * kD * 2;
constexpr int kSmemBytes = kQBytes + kStages * 2 * kTileBytes + 1024;
constexpr int kTmemCols = 256;
constexpr uint32_t kColS = 0;      // S buffers: columns [0,64) and [64,128), tile j uses buffer j & 1
constexpr uint32_t kColP = 0;      // P_j as packed bf16 over the first 32 columns of its S buffer
constexpr uint32_t kColO = 128;    // O accumulator: 64 columns
constexpr float kRescaleThreshold = 8.0f;

struct FwdParams {
  __nv_bfloat16* o;
  float* lse;
  int L, n_sel, H, HK;
  float scale_log2;   // softmax scale * log2(e)
  int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


// MMA groups issued as one instruction block by one elected lane (~3 instructions per MMA): the MMA warp
// shares its scheduler partition with busy row-owning warps, so instructions per MMA set the issue rate.
// [d] = A * B^T over 4 K steps, both operands K-major in shared memory.
__device__ __forceinline__ void issue_ss_single(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc) {
#define MOC_SS1_STEP(KK, PACC)                                                  \
  "add.s64 ta, %1, " #KK "*2;\n\t add.s64 tb, %2, " #KK "*2;\n\t"                \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, " PACC ";\n\t"
  asm volatile(
      "{\n\t.reg .pred q, pt, pf;\n\t.reg .b64 ta, tb;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      MOC_SS1_STEP(0, "pf") MOC_SS1_STEP(1, "pt") MOC_SS1_STEP(2, "pt") MOC_SS1_STEP(3, "pt")
      "}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc)
      : "memory");
#undef MOC_SS1_STEP
}
// [d] += A * B over 4 K steps: A packed bf16 in tensor memory (K step kk at column a + 8 kk), B MN-major.
__device__ __forceinline__ void issue_ts_single(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
#define MOC_TS1_STEP(KK, PACC)                                                  \
  "add.u32 ca, %1, " #KK "*8;\n\t add.s64 tb, %2, " #KK "*128;\n\t"               \
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

__global__ void __launch_bounds__(kThreads, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                   FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  // p_full is one barrier per score buffer: S_{j+1} is issued before the MMA warp waits for P_j, so the row owners
  // can finish tile j+1 (the other buffer) while that wait has not yet observed tile j's phase; with a single barrier
  // two completed phases would look like none to a parity wait and the warp would wait forever.
  __shared__ __align__(8) uint64_t q_bar, kv_full[kStages], kv_empty[kStages], s_full[2], p_full[2], pv_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = base;
  uint8_t* kv_s = base + kQBytes;

  const int q0 = blockIdx.x * kQ;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kh = h / (p.H / p.HK);
  const int n_tiles = (p.n_sel + kKeys - 1) / kKeys;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&q_bar, 1);
    for (int s = 0; s < kStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(&p_full[0], 128);
    mbar_init(&p_full[1], 128);
    mbar_init(&pv_bar, 1);
    fence_mbar_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_kv);
  }
  if (warp == 5) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_arrive_expect_tx(&q_bar, kQBytes);
      tma_load_2d(q_s, &tmap_q, &q_bar, h * kD, b * p.L + q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        if (!mbar_wait(&kv_empty[s], ph ^ 1, &abort_flag, p.status)) break;
        mbar_arrive_expect_tx(&kv_full[s], 2 * kTileBytes);
        uint8_t* k_s = kv_s + s * 2 * kTileBytes;
        const int row = b * p.n_sel + j * kKeys;
        tma_load_2d(k_s, &tmap_kv, &kv_full[s], kh * kD, row);
        tma_load_2d(k_s + kTileBytes, &tmap_kv, &kv_full[s], p.HK * kD + kh * kD, row);
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    {   // warp-uniform: every lane runs the loop, one elected lane issues
      const uint32_t idesc_s = umma_idesc_bf16(kQ, kKeys, 0, 0);
      const uint32_t idesc_o = umma_idesc_bf16(kQ, kD, 0, 1);
      // descriptors are built once; a stage or K step only adds a constant to the address field
      const uint64_t q_desc = umma_desc_sw128(smem_u32(q_s), 16, 1024);
      const uint64_t k_desc0 = umma_desc_sw128(smem_u32(kv_s), 16, 1024);
      const uint64_t v_desc0 = umma_desc_sw128(smem_u32(kv_s) + kTileBytes, 8192, 1024);
      constexpr uint64_t kStageOff = (2 * kTileBytes) >> 4;
      bool ok = mbar_wait_w(&q_bar, 0, &abort_flag, p.status);
      // Two S buffers: S_{j+1} is issued before PV_j, so the tensor pipe computes the next scores while the row
      // owners exponentiate the current ones.  S_{j+1} overwrites the buffer P_{j-1} lived in; tcgen05.mma
      // instructions of one thread execute in issue order, so PV_{j-1} has read it.
      if (ok && n_tiles > 0) {
        ok = mbar_wait_w(&kv_full[0], 0, &abort_flag, p.status);
        if (ok) {
          tc_fence_after();
          issue_ss_single(tmem + kColS, q_desc, k_desc0, idesc_s);
          tc_commit_w(&s_full[0]);
        }
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          const int sn = (j + 1) % kStages;
          ok = mbar_wait_w(&kv_full[sn], ((j + 1) / kStages) & 1, &abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          issue_ss_single(tmem + kColS + ((j + 1) & 1) * 64, q_desc, k_desc0 + sn * kStageOff, idesc_s);
          tc_commit_w(&s_full[(j + 1) & 1]);
        }
        const int s = j % kStages;
        ok = mbar_wait_w(&p_full[j & 1], (j >> 1) & 1, &abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        issue_ts_single(tmem + kColO, tmem + kColP + (j & 1) * 64, v_desc0 + s * kStageOff, idesc_o, j > 0 ? 1u : 0u);
        tc_commit_w(&kv_empty[s]);
        tc_commit_w(&pv_bar);
      }
    }
  } else {
    // ---------------- softmax: thread <-> query row ----------------
    const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;
    const int row = warp * 32 + lane;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, &abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_sel + kColS + (j & 1) * 64;
      const int valid = p.n_sel - j * kKeys;   // keys of this tile that exist
      uint32_t r0[32], r1[32];                 // the whole score row stays in registers
      tmem_ld32(s_addr, r0);
      tmem_ld32(s_addr + 32, r1);
      tmem_wait_ld();
      if (valid < kKeys) {                     // last, partial tile: columns past the end count as -inf
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          if (c >= valid) r0[c] = 0xFF800000u;
          if (32 + c >= valid) r1[c] = 0xFF800000u;
        }
      }
      float tmax = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) tmax = fmaxf(tmax, fmaxf(__uint_as_float(r0[c]), __uint_as_float(r1[c])));
      const float m_new = fmaxf(m_used, tmax * p.scale_log2);
      const bool need = (j == 0) || (m_new - m_used > kRescaleThreshold);
      const bool any_need = __any_sync(0xffffffffu, need);
      if (j > 0 && any_need) {
        ok = mbar_wait(&pv_bar, (j - 1) & 1, &abort_flag, p.status);   // O is complete up to tile j-1
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const float alpha = need ? ex2(m_used - m_new) : 1.f;
        uint32_t r[32];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          tmem_ld32(tmem + lane_sel + kColO + half * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
          tmem_st32(tmem + lane_sel + kColO + half * 32, r);
        }
        l_sum *= alpha;
      }
      if (need) m_used = m_new;
      uint32_t pk[32];
      float psum0 = 0.f, psum1 = 0.f;
      // exp2 of -inf is 0, so masked columns add nothing
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float e0 = ex2(fmaf(__uint_as_float(r0[c]), p.scale_log2, -m_used));
        const float e1 = ex2(fmaf(__uint_as_float(r0[c + 1]), p.scale_log2, -m_used));
        psum0 += e0;
        psum1 += e1;
        pk[c / 2] = pack_bf16x2(e0, e1);
      }
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float e0 = ex2(fmaf(__uint_as_float(r1[c]), p.scale_log2, -m_used));
        const float e1 = ex2(fmaf(__uint_as_float(r1[c + 1]), p.scale_log2, -m_used));
        psum0 += e0;
        psum1 += e1;
        pk[16 + c / 2] = pack_bf16x2(e0, e1);
      }
      l_sum += psum0 + psum1;
      // every S value of this row is in registers: P goes over the first 32 columns of this tile's S buffer
      tmem_st32(tmem + lane_sel + kColP + (j & 1) * 64, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[j & 1]);
    }
    if (ok) {
      ok = mbar_wait(&pv_bar, (n_tiles - 1) & 1, &abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l_sum;
      const int l = q0 + row;
      __nv_bfloat16* dst = p.o + (static_cast<long long>(b) * p.L + l) * (p.H * kD) + h * kD;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_sel + kColO + half * 32, r);
        tmem_wait_ld();
        if (l < p.L) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * c + 0]) * inv, __uint_as_float(r[8 * c + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(r[8 * c + 2]) * inv, __uint_as_float(r[8 * c + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(r[8 * c + 4]) * inv, __uint_as_float(r[8 * c + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(r[8 * c + 6]) * inv, __uint_as_float(r[8 * c + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + half * 32 + c * 8) = v;
          }
        }
      }
      if (l < p.L)
        p.lse[(static_cast<long long>(b) * p.H + h) * p.L + l] = (m_used + log2f(l_sum)) * 0.6931471805599453f;
    }
    tc_fence_before();
  }

  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

int launch_attn_tc_fwd(const moc_attn_shape* s, const void* q, const void* kv, void* o, float* lse,
                       int32_t* status, cudaStream_t stream) {
  MOC_REQUIRE(s->head_dim == kD, "bf16 attention needs head_dim 64");
  MOC_REQUIRE(s->num_heads % s->num_kv_heads == 0, "num_heads must be a multiple of num_kv_heads");
  MOC_REQUIRE((reinterpret_cast<uintptr_t>(o) & 15) == 0, "output must be 16-byte aligned");
  CUtensorMap tq, tkv;
  int rc = make_tmap_bf16_2d(&tq, q, static_cast<uint64_t>(s->batch) * s->seq,
                             static_cast<uint64_t>(s->num_heads) * kD, static_cast<uint64_t>(s->num_heads) * kD,
                             kQ, kD);
  if (rc != MOC_OK) return rc;
  rc = make_tmap_bf16_2d(&tkv, kv, static_cast<uint64_t>(s->batch) * s->n_sel,
                         static_cast<uint64_t>(2 * s->num_kv_heads) * kD,
                         static_cast<uint64_t>(2 * s->num_kv_heads) * kD, kKeys, kD);
  if (rc != MOC_OK) return rc;
  MOC_CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  FwdParams p;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.L = s->seq; p.n_sel = s->n_sel; p.H = s->num_heads; p.HK = s->num_kv_heads;
  p.scale_log2 = s->scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid(ceil_div(s->seq, kQ), s->num_heads, s->batch);
  attn_fwd_tc_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tq, tkv, p);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

}  // namespace moc
