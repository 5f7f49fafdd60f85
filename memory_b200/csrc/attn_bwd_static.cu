// Attention backward for callers that must not allocate device memory.
//
// moc_attn_bwd needs 6*B*H*L floats of scratch (the per-row <O,dO> sums, the rescaled log-sum-exp and
// their packed bf16 operand rows)
// that the caller normally allocates.  Some callers cannot: code running while a CUDA memory pool is
// frozen (a serving process that pre-sized its arena), code inside a library callback that forbids
// cudaMalloc, or a process whose allocator is owned by another framework and is not reachable from
// C.  For them this file keeps the scratch in a fixed array in device global memory that is part of
// the library image: every GPU that loads the library holds kStaticScratchFloats * 4 bytes of it
// until the process exits.
//
// The array's name is only a host-side handle.  Its device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and that pointer is what the kernels receive.
#include <mutex>

#include "moc_common.cuh"

namespace moc {
int launch_delta(int dtype, const void* o, const void* d_o, float* delta, int B, int L, int H, int D,
                 cudaStream_t stream);
int launch_attn_f32_bwd(const moc_attn_shape* s, const float* q, const float* kv, const float* d_o,
                        const float* lse, const float* delta, float* d_q, float* d_kv, cudaStream_t stream);
int launch_attn_tc_bwd(const moc_attn_shape* s, const void* q, const void* kv, const void* o, const float* lse,
                       const void* d_o, void* d_q, void* d_kv, float* scratch, int32_t* status,
                       cudaStream_t stream, int parts, const float* kv_row_scale = nullptr, float* kv_dot = nullptr);
}  // namespace moc

namespace {

constexpr size_t kStaticScratchFloats = MOC_ATTN_BWD_STATIC_MAX_FLOATS;     // 4 MiB
static __device__ __align__(256) float g_attn_bwd_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (looked up on the first call there).
int scratch_for_current_device(float** out) {
  int dev = -1;
  MOC_CUDA_OK(cudaGetDevice(&dev));
  MOC_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    MOC_CUDA_OK(cudaGetSymbolAddress(&p, g_attn_bwd_scratch));
    MOC_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned NULL");
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return MOC_OK;
}

}  // namespace

using namespace moc;

extern "C" int moc_attn_bwd_static(const moc_attn_shape* s, const void* q, const void* kv, const void* o,
                                   const float* lse, const void* d_o, void* d_q, void* d_kv, int32_t* status,
                                   void* stream_) {
  MOC_REQUIRE(s != nullptr, "shape is NULL");
  MOC_REQUIRE(s->batch > 0 && s->seq > 0 && s->n_sel > 0, "empty attention problem");
  MOC_REQUIRE(s->num_heads > 0 && s->num_kv_heads > 0 && s->num_heads % s->num_kv_heads == 0,
              "num_heads must be a positive multiple of num_kv_heads");
  MOC_REQUIRE(q && kv && o && lse && d_o && d_q && d_kv && status, "NULL attention buffer");
  const size_t need = size_t(6) * s->batch * s->num_heads * s->seq;
  MOC_REQUIRE(need <= kStaticScratchFloats,
              "6*batch*num_heads*seq exceeds the built-in scratch (1,048,576 floats): use moc_attn_bwd");
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != MOC_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // Nothing in the scratch has to start at zero: the preparation kernel overwrites every word the
  // other kernels read.  The previous call's contents are simply replaced.
  if (s->dtype == MOC_F32) {
    rc = launch_delta(MOC_F32, o, d_o, scratch, s->batch, s->seq, s->num_heads, s->head_dim, stream);
    if (rc != MOC_OK) return rc;
    return launch_attn_f32_bwd(s, static_cast<const float*>(q), static_cast<const float*>(kv),
                               static_cast<const float*>(d_o), lse, scratch, static_cast<float*>(d_q),
                               static_cast<float*>(d_kv), stream);
  }
  if (s->dtype == MOC_BF16) return launch_attn_tc_bwd(s, q, kv, o, lse, d_o, d_q, d_kv, scratch, status, stream, 7);
  set_last_error("dtype", "unknown dtype");
  return MOC_ERR_INVALID;
}
