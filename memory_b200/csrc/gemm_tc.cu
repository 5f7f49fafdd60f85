// bf16 tensor-core projection kernel for sm_100a: TMA -> shared memory (128-byte swizzle) ->
// tcgen05.mma with the fp32 accumulator tile in tensor memory -> tcgen05.ld epilogue.
//
//   C[M,N] (+)= op(A)[M,K] * op(B)[K,N], 128 x 256 (or 128 x 128) output tiles, 64-wide K stages.
//
// Persistent: one CTA per SM walks a static list of (tile, K-split) items.  Roles inside a CTA of 192
// threads: warp 0 issues the TMA loads, warp 1 owns tensor memory and issues the MMAs from one lane,
// warps 2-5 drain the accumulator (each warp may only touch the 32 TMEM lanes selected by
// warp_id % 4).  Two accumulator buffers in tensor memory let the epilogue of one tile run under the
// main loop of the next.  The A operand can be fetched through a row-block gather
// list, which is how selected chapters are read straight out of the memory bank.
#define MOC_KERNEL_TAG 1
#include "moc_common.cuh"

namespace moc {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kTmemCols = 512;          // two accumulator buffers of up to 256 columns

// MT = 128-row MMA tiles per CTA tile.  MT = 1: 128 x BN output tile, two accumulator buffers, so the epilogue of
// one tile runs under the main loop of the next.  MT = 2: 256 x 256 output tile, both accumulators live at once
// and the two MMAs of a K step share the B stage: a third fewer bytes from L2 per FLOP, which is what limits
// this kernel at K <= 1536.
template <int BN, int MT> struct Cfg {
  static constexpr int kStages = (MT == 2) ? 3 : ((BN == 256) ? 4 : 6);
  static constexpr int kThreads = 64 + 128 * MT;
  static constexpr int kABytes = BM * MT * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStoreBytes = 32 * 128;        // per epilogue warp: 32 rows x 64 bf16 staged for a TMA store
  static constexpr int kSmemBytes = kStages * kStageBytes + 4 * MT * kStoreBytes + 1024;
};

struct GemmTcParams {
  int m, n, k;
  int a_kmajor, b_kmajor;
  void* c;
  long long ldc;
  int c_bf16;
  int c_tma;               // bf16 C written through shared memory and TMA stores (rows 16-byte aligned)
  int accumulate;
  int atomic;
  const float* row_scale;
  int scale_block_rows;
  const float* residual;   // fp32 [m, n] added to the product by the first K split, or nullptr
  long long ldr;
  const int* a_row_blocks;
  int a_box_rows;          // rows per A box when A is K-major
  int a_num_blocks;        // entries in the gather list
  long long a_stored_rows;
  const int* b_row_blocks; // gather list over the K rows of an MN-major B ([K, N] row-major), or nullptr
  int b_block_rows;        // rows per listed block (a chapter)
  int b_box_rows;          // rows per TMA box of the gathered B: min(b_block_rows, 64)
  int b_num_blocks;
  long long b_stored_rows;
  int k_tiles_total;
  int k_tiles_per_split;
  int splits;
  int m_tiles, n_tiles;
  int num_items;           // m_tiles * n_tiles * splits
  int* status;
};

__device__ __forceinline__ void drain_after_abort() {
  // give bulk copies already in flight time to land before the CTA's shared memory is released
  for (int i = 0; i < 200; ++i) __nanosleep(1000);
}

// Persistent kernel: CTA i works on items i, i + gridDim.x, ...; an item is (output tile, K split).
template <int BN, int MT>
__global__ void __launch_bounds__(64 + 128 * MT, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_c, GemmTcParams p) {
  using C = Cfg<BN, MT>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[C::kStages];
  __shared__ __align__(8) uint64_t empty_bar[C::kStages];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4 * MT);
    }
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
        const int split = item % p.splits;
        const int tile = item / p.splits;
        const int n0 = (tile % p.n_tiles) * BN;
        const int m0 = (tile / p.n_tiles) * (BM * MT);
        const int kt_begin = split * p.k_tiles_per_split;
        int kt_count = p.k_tiles_total - kt_begin;
        if (kt_count > p.k_tiles_per_split) kt_count = p.k_tiles_per_split;
        // Gathered A: the stored rows of this tile's boxes depend on the tile only, so the list is read once per
        // item (up to 32 boxes: 256 rows of 8), not once per K step -- a dependent global load in front of every
        // copy would pace the whole pipeline.
        int a_rows[32];
        const int nbox_a = p.a_kmajor ? BM * MT / p.a_box_rows : 0;
        if (p.a_kmajor && p.a_row_blocks != nullptr) {
#pragma unroll 1
          for (int i = 0; i < nbox_a; ++i) {
            const int blk = m0 / p.a_box_rows + i;
            long long row = (blk < p.a_num_blocks) ? static_cast<long long>(p.a_row_blocks[blk]) * p.a_box_rows
                                                   : p.a_stored_rows;
            if (row < 0 || row > p.a_stored_rows) {
              atomicMax(p.status, MOC_DEV_BAD_INDEX);
              row = p.a_stored_rows;   // fully out of range: the copy zero-fills
            }
            a_rows[i] = static_cast<int>(row);
          }
        }
        // Gathered B: block ids are requested kIdAhead K steps before they are needed (a register ring), so the
        // latency of the list read (a dependent global load) is hidden behind the copies of the steps in between.
        constexpr int kIdAhead = 8;
        const int nsub_b = (p.b_row_blocks != nullptr) ? BK / p.b_box_rows : 0;
        auto blk_of = [&](long long kg) { return kg / p.b_block_rows; };
        auto ld_id = [&](long long kg) -> long long {
          const long long blk = blk_of(kg);
          return (blk < p.b_num_blocks) ? static_cast<long long>(p.b_row_blocks[blk]) : -1;
        };
        long long ring[kIdAhead];
        if (nsub_b == 1) {
#pragma unroll
          for (int i = 0; i < kIdAhead; ++i)
            ring[i] = (i < kt_count) ? ld_id(static_cast<long long>(kt_begin + i) * BK) : -1;
        }
        for (int kt = 0; kt < kt_count; ++kt, ++it) {
          const int s = it % C::kStages;
          const uint32_t ph = (it / C::kStages) & 1;
          long long b_rows[8];
          if (nsub_b > 0) {
#pragma unroll 1
            for (int i = 0; i < nsub_b; ++i) {
              const long long kg = static_cast<long long>(kt_begin + kt) * BK + i * p.b_box_rows;
              const long long blk = blk_of(kg);
              const long long id = (nsub_b == 1) ? ring[0] : ld_id(kg);
              long long row = p.b_stored_rows;      // fully out of range: the copy zero-fills
              if (blk < p.b_num_blocks) {
                if (id < 0 || (id + 1) * p.b_block_rows > p.b_stored_rows) atomicMax(p.status, MOC_DEV_BAD_INDEX);
                else row = id * p.b_block_rows + (kg - blk * p.b_block_rows);
              }
              b_rows[i] = row;
            }
            if (nsub_b == 1) {
#pragma unroll
              for (int i = 0; i + 1 < kIdAhead; ++i) ring[i] = ring[i + 1];
              ring[kIdAhead - 1] = (kt + kIdAhead < kt_count)
                                       ? ld_id(static_cast<long long>(kt_begin + kt + kIdAhead) * BK) : -1;
            }
          }
          ok = mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, p.status);
          if (!ok) break;
          mbar_arrive_expect_tx(&full_bar[s], C::kStageBytes);
          uint8_t* a_s = tiles + s * C::kStageBytes;
          uint8_t* b_s = a_s + C::kABytes;
          const int k0 = (kt_begin + kt) * BK;
          if (p.a_kmajor) {
            for (int i = 0; i < nbox_a; ++i) {
              const int row = (p.a_row_blocks != nullptr) ? a_rows[i] : m0 + i * p.a_box_rows;
              tma_load_2d(a_s + i * p.a_box_rows * 128, &tmap_a, &full_bar[s], k0, row);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 2 * MT; ++i) tma_load_2d(a_s + i * 8192, &tmap_a, &full_bar[s], m0 + 64 * i, k0);
          }
          if (p.b_kmajor) {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              tma_load_2d(b_s + j * 16384, &tmap_b, &full_bar[s], k0, n0 + j * 128);
          } else if (p.b_row_blocks == nullptr) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_s + j * 8192, &tmap_b, &full_bar[s], n0 + j * 64, k0);
          } else {
            // the K rows of this stage are rows of listed blocks (chapters of the bank): one box per run of rows
            // that is contiguous in the stored matrix
            for (int i = 0; i < nsub_b; ++i) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(b_s + j * 8192 + i * p.b_box_rows * 128, &tmap_b, &full_bar[s], n0 + j * 64,
                            static_cast<int>(b_rows[i]));
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    {   // warp-uniform: every lane runs the loop, one elected lane issues
      const uint32_t idesc = umma_idesc_bf16(BM, BN, p.a_kmajor ? 0 : 1, p.b_kmajor ? 0 : 1);
      // Descriptors are built once: a stage or K step only adds a constant to the 16-byte-unit address
      // field, so issuing an MMA costs two 64-bit adds instead of rebuilding both descriptors.
      const uint32_t tiles_addr = smem_u32(tiles);
      const uint64_t a_base = p.a_kmajor ? umma_desc_sw128(tiles_addr, 16, 1024) : umma_desc_sw128(tiles_addr, 8192, 1024);
      const uint64_t b_base = p.b_kmajor ? umma_desc_sw128(tiles_addr + C::kABytes, 16, 1024)
                                         : umma_desc_sw128(tiles_addr + C::kABytes, 8192, 1024);
      const uint64_t a_step = p.a_kmajor ? (32 >> 4) : (2048 >> 4);
      const uint64_t b_step = p.b_kmajor ? (32 >> 4) : (2048 >> 4);
      uint32_t it = 0, t = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x, ++t) {
        const int split = item % p.splits;
        const int kt_begin = split * p.k_tiles_per_split;
        int kt_count = p.k_tiles_total - kt_begin;
        if (kt_count > p.k_tiles_per_split) kt_count = p.k_tiles_per_split;
        const uint32_t buf = (MT == 1) ? (t & 1) : 0;
        ok = mbar_wait_w(&acc_empty[buf], (MT == 1 ? ((t >> 1) & 1) : (t & 1)) ^ 1, &abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * 256;
        for (int kt = 0; kt < kt_count; ++kt, ++it) {
          const int s = it % C::kStages;
          const uint32_t ph = (it / C::kStages) & 1;
          ok = mbar_wait_w(&full_bar[s], ph, &abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint64_t stage_off = static_cast<uint64_t>(s) * (C::kStageBytes >> 4);
          const uint64_t ad = a_base + stage_off, bd = b_base + stage_off;
          if (MT == 1) {
            umma_ss_w(tmem_acc, ad, bd, idesc, kt > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < BK / 16; ++kk) umma_ss_w(tmem_acc, ad + kk * a_step, bd + kk * b_step, idesc, 1u);
          } else {
            // rows [128, 256) of the A stage start 16 KiB further on in both layouts; two independent accumulators
            constexpr uint64_t kSub = 16384 >> 4;
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
              const uint32_t acc = (kt > 0 || kk > 0) ? 1u : 0u;
              umma_ss_w(tmem_base, ad + kk * a_step, bd + kk * b_step, idesc, acc);
              umma_ss_w(tmem_base + 256, ad + kSub + kk * a_step, bd + kk * b_step, idesc, acc);
            }
          }
          tc_commit_w(&empty_bar[s]);
        }
        if (!ok) break;
        tc_commit_w(&acc_full[buf]);
      }
    }
  } else {
    // epilogue: TMEM lanes [32*(warp%4), +32) <-> output rows
    const int lane_group = (warp & 3) * 32;
    const int sub = (MT == 2) ? (warp - 2) / 4 : 0;        // which 128-row half of the tile this warp drains
    // One thread owns one output row, so direct stores scatter 16-byte pieces over 32 rows per instruction.
    // bf16 tiles therefore go through a 128-byte-swizzled staging block and leave as TMA stores.
    uint8_t* stage_c = tiles + C::kStages * C::kStageBytes + (warp - 2) * C::kStoreBytes;
    const uint32_t stage_row = smem_u32(stage_c) + lane * 128;
    uint32_t t = 0;
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x, ++t) {
      const int split = item % p.splits;
      const int tile = item / p.splits;
      const int n0 = (tile % p.n_tiles) * BN;
      const int m0 = (tile / p.n_tiles) * (BM * MT) + sub * BM;
      const int kt_begin = split * p.k_tiles_per_split;
      const bool has_k = kt_begin < p.k_tiles_total;
      const uint32_t buf = (MT == 1) ? (t & 1) : 0;
      bool have_acc = mbar_wait(&acc_full[buf], MT == 1 ? ((t >> 1) & 1) : (t & 1), &abort_flag, p.status);
      have_acc = __all_sync(0xffffffffu, have_acc);   // tcgen05.ld below is warp-collective
      if (!have_acc) break;
      tc_fence_after();
      const uint32_t tmem_acc = tmem_base + (MT == 1 ? buf : static_cast<uint32_t>(sub)) * 256;
      const int row = m0 + lane_group + lane;
      float rs = 1.0f;
      if (p.row_scale != nullptr && row < p.m) rs = p.row_scale[row / p.scale_block_rows];
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        const int col0 = n0 + c * 32;
        if (col0 >= p.n) break;                       // uniform across the warp
        if (has_k) {
          tmem_ld32(tmem_acc + (static_cast<uint32_t>(lane_group) << 16) + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (p.c_tma) {
          if ((c & 1) == 0) {                          // the previous store must be done with the staging block
            if (lane == 0) bulk_wait_read_all();
            __syncwarp();
          }
          if (p.residual != nullptr && row < p.m) {
            const float* res = p.residual + static_cast<long long>(row) * p.ldr + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.n) r[j] = __float_as_uint(__uint_as_float(r[j]) * rs + res[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * rs);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t addr = stage_row + ((static_cast<uint32_t>((c & 1) * 4 + j) ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                         "r"(pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]))),
                         "r"(pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]))),
                         "r"(pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]))),
                         "r"(pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])))
                         : "memory");
          }
          if ((c & 1) || col0 + 32 >= p.n) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmap_c, stage_c, n0 + (c & ~1) * 32, m0 + lane_group);
              bulk_commit_group();
            }
          }
          continue;
        }
        if (row >= p.m) continue;
        if (p.residual != nullptr && split == 0) {
          // fold the row scale and the residual into the registers; the stores below then see rs = 1
          const float* res = p.residual + static_cast<long long>(row) * p.ldr + col0;
          const bool vec4 = ((p.ldr & 3) == 0) && (col0 + 32 <= p.n) &&
                            ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0);
          if (vec4) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 v = *reinterpret_cast<const float4*>(res + 4 * j);
              r[4 * j + 0] = __float_as_uint(__uint_as_float(r[4 * j + 0]) * rs + v.x);
              r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) * rs + v.y);
              r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) * rs + v.z);
              r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) * rs + v.w);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.n) r[j] = __float_as_uint(__uint_as_float(r[j]) * rs + res[j]);
          }
        } else if (!has_k && (p.atomic || p.accumulate)) {
          continue;
        }
        const float rs_store = (p.residual != nullptr && split == 0) ? 1.0f : rs;
        if (p.c_bf16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + static_cast<long long>(row) * p.ldc + col0;
          const bool vec = ((p.ldc & 7) == 0) && (col0 + 32 <= p.n) &&
                           ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0);
          if (vec) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]) * rs_store, __uint_as_float(r[8 * j + 1]) * rs_store);
              v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * rs_store, __uint_as_float(r[8 * j + 3]) * rs_store);
              v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * rs_store, __uint_as_float(r[8 * j + 5]) * rs_store);
              v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * rs_store, __uint_as_float(r[8 * j + 7]) * rs_store);
              *reinterpret_cast<uint4*>(dst + 8 * j) = v;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.n) dst[j] = __float2bfloat16(__uint_as_float(r[j]) * rs_store);
          }
        } else {
          float* dst = reinterpret_cast<float*>(p.c) + static_cast<long long>(row) * p.ldc + col0;
          if (p.atomic) {
            const bool vec4 = ((p.ldc & 3) == 0) && (col0 + 32 <= p.n) &&
                              ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0);
            if (vec4) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                atomicAdd(reinterpret_cast<float4*>(dst + 4 * j),
                          make_float4(__uint_as_float(r[4 * j + 0]) * rs_store, __uint_as_float(r[4 * j + 1]) * rs_store,
                                      __uint_as_float(r[4 * j + 2]) * rs_store, __uint_as_float(r[4 * j + 3]) * rs_store));
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.n) atomicAdd(dst + j, __uint_as_float(r[j]) * rs_store);
            }
          } else {
            const bool vec = ((p.ldc & 3) == 0) && (col0 + 32 <= p.n) &&
                             ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0);
            if (vec) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j + 0]) * rs_store, __uint_as_float(r[4 * j + 1]) * rs_store,
                                       __uint_as_float(r[4 * j + 2]) * rs_store, __uint_as_float(r[4 * j + 3]) * rs_store);
                float4* d4 = reinterpret_cast<float4*>(dst + 4 * j);
                if (p.accumulate) {
                  const float4 o = *d4;
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *d4 = v;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.n) {
                  const float v = __uint_as_float(r[j]) * rs_store;
                  dst[j] = p.accumulate ? dst[j] + v : v;
                }
            }
          }
        }
      }
      // this warp is done reading the accumulator buffer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (p.c_tma && lane == 0) bulk_wait_all();       // stores still in flight read this CTA's shared memory
    tc_fence_before();
  }

  __syncthreads();
  if (abort_flag) drain_after_abort();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

}  // namespace

int launch_gemm_tc(const moc_gemm_desc* g, const void* a, const void* b, void* c, const float* row_scale,
                   const int32_t* a_row_blocks, int32_t* status, cudaStream_t stream,
                   const int32_t* b_row_blocks, int32_t b_block_rows, int64_t b_stored_rows) {
  MOC_REQUIRE(g->k % 8 == 0, "bf16 projection needs K % 8 == 0");
  MOC_REQUIRE(g->lda % 8 == 0 && g->ldb % 8 == 0, "bf16 projection needs 16-byte aligned operand rows");
  MOC_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0,
              "operands must be 16-byte aligned");
  MOC_REQUIRE(g->c_dtype == MOC_BF16 || g->c_dtype == MOC_F32, "bad c_dtype");
  const int split = g->split_k > 1 ? g->split_k : 1;
  if (split > 1 || g->accumulate) MOC_REQUIRE(g->c_dtype == MOC_F32, "accumulate / split_k need an fp32 C");
  int a_box_rows = 64;
  int a_num_blocks = 0;
  long long a_stored_rows = g->a_kmajor ? g->m : g->k;
  if (a_row_blocks != nullptr) {
    MOC_REQUIRE(g->a_kmajor, "the gather list needs a K-major A");
    a_box_rows = g->a_block_rows;
    MOC_REQUIRE(a_box_rows >= 8 && a_box_rows <= 128 && (128 % a_box_rows) == 0 && (a_box_rows % 8) == 0,
                "a_block_rows must be a multiple of 8 that divides 128");
    // (up to 256 / 8 = 32 boxes per tile, the size of the per-item row table in the producer)
    MOC_REQUIRE(g->m % a_box_rows == 0, "M must be a multiple of a_block_rows");
    a_num_blocks = g->m / a_box_rows;
    a_stored_rows = g->a_stored_rows;
    MOC_REQUIRE(a_stored_rows > 0, "a_stored_rows missing");
  }
  int b_box_rows = 64, b_num_blocks = 0;
  if (b_row_blocks != nullptr) {
    MOC_REQUIRE(!g->b_kmajor, "the B gather list needs an MN-major B ([K, N] row-major)");
    MOC_REQUIRE(b_block_rows >= 8 && (b_block_rows % 8) == 0 && ((64 % b_block_rows) == 0 || (b_block_rows % 64) == 0),
                "b_block_rows must be a multiple of 8 that divides 64 or is a multiple of 64");
    MOC_REQUIRE(g->k % b_block_rows == 0, "K must be a multiple of b_block_rows");
    MOC_REQUIRE(b_stored_rows > 0, "b_stored_rows missing");
    b_box_rows = b_block_rows < 64 ? b_block_rows : 64;
    b_num_blocks = g->k / b_block_rows;
  }

  // Tile width.  The kernel is fed from L2 (~8.4 TB/s measured over all SMs), so a tile's time goes with the
  // bytes it loads per K step, (BM + BN) * 128: the cost of a width is rounds-of-items times that.
  const int sms = sm_count();
  const int m_tiles = ceil_div(g->m, BM);
  auto waves_cost = [&](int bn) {
    const long long items = static_cast<long long>(m_tiles) * ceil_div(g->n, bn) * split;
    const long long rounds = (items + sms - 1) / sms;
    return static_cast<double>(rounds) * (BM + bn);
  };
  const int bn = (g->n > 128 && waves_cost(256) <= waves_cost(128)) ? 256 : 128;
  // 256 x 256 tiles: single pass over K only (no split), and only where the rounds-times-bytes cost, with the
  // epilogue that is no longer hidden counted as 8 %, beats the 128-row tiles.
  bool tall = false;
  if (bn == 256 && split == 1 && g->m >= 2 * BM && (a_row_blocks == nullptr || 256 % a_box_rows == 0)) {
    const long long items = static_cast<long long>(ceil_div(g->m, 2 * BM)) * ceil_div(g->n, 256);
    const double cost_tall = static_cast<double>((items + sms - 1) / sms) * (2 * BM + 256) * 1.08;
    tall = cost_tall < waves_cost(256);
  }

  CUtensorMap tmap_a, tmap_b;
  int rc;
  if (g->a_kmajor) {
    rc = make_tmap_bf16_2d(&tmap_a, a, static_cast<uint64_t>(a_stored_rows), static_cast<uint64_t>(g->k),
                           static_cast<uint64_t>(g->lda), static_cast<uint32_t>(a_box_rows), 64);
  } else {
    rc = make_tmap_bf16_2d(&tmap_a, a, static_cast<uint64_t>(g->k), static_cast<uint64_t>(g->m),
                           static_cast<uint64_t>(g->lda), 64, 64);
  }
  if (rc != MOC_OK) return rc;
  if (g->b_kmajor) {
    rc = make_tmap_bf16_2d(&tmap_b, b, static_cast<uint64_t>(g->n), static_cast<uint64_t>(g->k),
                           static_cast<uint64_t>(g->ldb), 128, 64);
  } else if (b_row_blocks != nullptr) {
    rc = make_tmap_bf16_2d(&tmap_b, b, static_cast<uint64_t>(b_stored_rows), static_cast<uint64_t>(g->n),
                           static_cast<uint64_t>(g->ldb), static_cast<uint32_t>(b_box_rows), 64);
  } else {
    rc = make_tmap_bf16_2d(&tmap_b, b, static_cast<uint64_t>(g->k), static_cast<uint64_t>(g->n),
                           static_cast<uint64_t>(g->ldb), 64, 64);
  }
  if (rc != MOC_OK) return rc;

  const bool c_tma = g->c_dtype == MOC_BF16 && (g->ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(c) & 15) == 0;
  CUtensorMap tmap_c = tmap_a;      // placeholder when the TMA-store epilogue is not used
  if (c_tma) {
    rc = make_tmap_bf16_2d(&tmap_c, c, static_cast<uint64_t>(g->m), static_cast<uint64_t>(g->n),
                           static_cast<uint64_t>(g->ldc), 32, 64);
    if (rc != MOC_OK) return rc;
  }

  GemmTcParams p;
  p.c_tma = c_tma ? 1 : 0;
  p.m = g->m; p.n = g->n; p.k = g->k;
  p.a_kmajor = g->a_kmajor; p.b_kmajor = g->b_kmajor;
  p.c = c; p.ldc = g->ldc; p.c_bf16 = (g->c_dtype == MOC_BF16);
  p.accumulate = g->accumulate; p.atomic = split > 1;
  p.row_scale = row_scale; p.scale_block_rows = g->scale_block_rows > 0 ? g->scale_block_rows : 1;
  p.residual = g->residual; p.ldr = g->ldr;
  p.a_row_blocks = a_row_blocks; p.a_box_rows = a_box_rows; p.a_num_blocks = a_num_blocks;
  p.a_stored_rows = a_stored_rows;
  p.b_row_blocks = b_row_blocks; p.b_block_rows = b_block_rows; p.b_box_rows = b_box_rows;
  p.b_num_blocks = b_num_blocks; p.b_stored_rows = b_stored_rows;
  p.k_tiles_total = ceil_div(g->k, BK);
  p.k_tiles_per_split = ceil_div(p.k_tiles_total, split);
  p.splits = ceil_div(p.k_tiles_total, p.k_tiles_per_split);   // no empty splits
  p.m_tiles = tall ? ceil_div(g->m, 2 * BM) : m_tiles;
  p.n_tiles = ceil_div(g->n, bn);
  p.num_items = p.m_tiles * p.n_tiles * p.splits;
  p.status = status;

  const int grid = p.num_items < sms ? p.num_items : sms;
  if (tall) {
    using C2 = Cfg<256, 2>;
    MOC_CUDA_OK(cudaFuncSetAttribute(gemm_tc_kernel<256, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, C2::kSmemBytes));
    gemm_tc_kernel<256, 2><<<grid, C2::kThreads, C2::kSmemBytes, stream>>>(tmap_a, tmap_b, tmap_c, p);
  } else if (bn == 256) {
    using C1 = Cfg<256, 1>;
    MOC_CUDA_OK(cudaFuncSetAttribute(gemm_tc_kernel<256, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, C1::kSmemBytes));
    gemm_tc_kernel<256, 1><<<grid, C1::kThreads, C1::kSmemBytes, stream>>>(tmap_a, tmap_b, tmap_c, p);
  } else {
    using C0 = Cfg<128, 1>;
    MOC_CUDA_OK(cudaFuncSetAttribute(gemm_tc_kernel<128, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, C0::kSmemBytes));
    gemm_tc_kernel<128, 1><<<grid, C0::kThreads, C0::kSmemBytes, stream>>>(tmap_a, tmap_b, tmap_c, p);
  }
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

}  // namespace moc
