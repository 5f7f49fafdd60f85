// Host-side utilities shared by the entry points: last-error text and TMA tensor-map creation.
#include <string>

#define MOC_KERNEL_TAG 4
#include <cstdio>

#include "moc_common.cuh"

namespace moc {

static thread_local std::string g_last_error;

void set_last_error(const char* what, const char* detail) {
  g_last_error = std::string(what ? what : "") + ": " + (detail ? detail : "");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

int make_tmap_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                      uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_last_error("cuTensorMapEncodeTiled", "driver entry point not found");
    return MOC_ERR_CUDA;
  }
  MOC_REQUIRE(box_cols * 2 == 128, "tile rows must be 128 bytes for the 128-byte swizzle");
  MOC_REQUIRE(box_rows >= 1 && box_rows <= 256, "box rows out of range");
  MOC_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor base must be 16-byte aligned");
  MOC_REQUIRE((row_stride_elems * 2) % 16 == 0, "row stride must be a multiple of 16 bytes");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  // The encoder is a driver-API call and needs a context current on the calling thread.  A thread that has made no
  // runtime call yet has none -- e.g. an autograd worker thread whose first operation of a backward pass is one of
  // these projections on device 0 (the framework then has no reason to switch devices): bind the primary context of
  // the thread's current device once per thread.
  thread_local bool context_bound = false;
  if (!context_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) cudaFree(nullptr);
    context_bound = true;
  }
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    // say what was asked for, and whether an earlier asynchronous error is what the driver is reporting
    char msg[320];
    const cudaError_t pending = cudaPeekAtLastError();
    snprintf(msg, sizeof(msg), "encode failed (CUresult %d; base %p, rows %llu, cols %llu, row stride %llu, box %u x %u; "
             "pending runtime error: %s)", static_cast<int>(r), base, static_cast<unsigned long long>(rows),
             static_cast<unsigned long long>(cols), static_cast<unsigned long long>(row_stride_elems), box_rows,
             box_cols, cudaGetErrorString(pending));
    set_last_error("cuTensorMapEncodeTiled", msg);
    return MOC_ERR_CUDA;
  }
  return MOC_OK;
}

// One CTA whose first warp waits, with the library's bounded wait, on an mbarrier that `arrivals` of the
// other threads arrive at.  With arrivals below the barrier's count the wait can only run out: that is how
// the give-up path (status word, abort flag, normal return) is exercised without a hung kernel.
__global__ void wait_probe_kernel(int expected, int arrivals, uint32_t poll_limit, int* status, int* out) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, static_cast<uint32_t>(expected));
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x >= 32 && static_cast<int>(threadIdx.x) - 32 < arrivals) mbar_arrive(&bar);
  if (threadIdx.x < 32) {
    const bool ok = mbar_wait_limited(&bar, 0, &abort_flag, status, poll_limit);
    // a second wait after a give-up must return at once (the CTA-wide abort flag)
    const bool again = ok ? true : mbar_wait_limited(&bar, 0, &abort_flag, status, poll_limit);
    if (threadIdx.x == 0) { out[0] = ok ? 1 : 0; out[1] = again ? 1 : 0; out[2] = abort_flag; }
  }
}

// Barrier between the ranks of one node over flag words in each other's memory (plain peer stores and loads, one
// thread per peer, no SM held while nothing is due).  Rank r's flag array lives in r's own memory; word q of it is
// written by rank q only.  An arrival stores the epoch (a counter that only grows) with release semantics at system
// scope -- whatever this stream did before, e.g. copy-engine pushes into the peer's buffers, is complete and visible
// first -- and then polls its own word of that peer with acquire loads until it holds at least this epoch.  The
// poll is bounded: after `poll_limit` rounds the thread records MOC_DEV_TIMEOUT and returns.
struct PeerFlags { uint32_t* p[16]; };
__global__ void peer_barrier_kernel(PeerFlags flags, int rank, int world, uint32_t epoch, uint32_t poll_limit,
                                    int* status) {
  const int r = threadIdx.x;
  if (r >= world || r == rank) return;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[r] + rank), "r"(epoch) : "memory");
  const uint32_t* mine = flags.p[rank] + r;
  for (uint32_t it = 0; it < poll_limit; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) return;
    __nanosleep(100);
  }
  atomicMax(status, MOC_DEV_TIMEOUT | (MOC_KERNEL_TAG << 8) | (__LINE__ << 12));
}

}  // namespace moc

extern "C" int moc_peer_barrier(const void* const* flag_arrays, int32_t rank, int32_t world, uint32_t epoch,
                                uint32_t poll_limit, int32_t* status, void* stream_) {
  using namespace moc;
  MOC_REQUIRE(flag_arrays && status, "NULL buffer");
  MOC_REQUIRE(world >= 1 && world <= 16 && rank >= 0 && rank < world, "bad rank / world size");
  MOC_REQUIRE(poll_limit >= 1, "poll_limit must be positive");
  PeerFlags f;
  for (int r = 0; r < 16; ++r) f.p[r] = r < world ? static_cast<uint32_t*>(const_cast<void*>(flag_arrays[r])) : nullptr;
  for (int r = 0; r < world; ++r) MOC_REQUIRE(f.p[r] != nullptr, "NULL flag array");
  if (world == 1) return MOC_OK;
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(f, rank, world, epoch, poll_limit, status);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_wait_probe(int32_t expected, int32_t arrivals, uint32_t poll_limit, int32_t* status,
                              int32_t* out, void* stream_) {
  using namespace moc;
  MOC_REQUIRE(status && out, "NULL buffer");
  MOC_REQUIRE(expected >= 1 && expected <= 96 && arrivals >= 0 && arrivals <= expected, "bad arrival counts");
  MOC_REQUIRE(poll_limit >= 1 && poll_limit <= (1u << 20), "poll_limit must be in [1, 2^20]");
  wait_probe_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream_)>>>(expected, arrivals, poll_limit, status, out);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" const char* moc_last_error(void) { return moc::g_last_error.c_str(); }
extern "C" int moc_abi_version(void) { return 2; }
