// extern "C" dispatch of the projection and attention entry points onto the fp32 (FMA) and bf16
// (tcgen05) kernels.  There is no CPU path: a dtype / shape the kernels do not cover is an error.
#include "moc_common.cuh"

namespace moc {
int launch_gemm_tc(const moc_gemm_desc* g, const void* a, const void* b, void* c, const float* row_scale,
                   const int32_t* a_row_blocks, int32_t* status, cudaStream_t stream,
                   const int32_t* b_row_blocks = nullptr, int32_t b_block_rows = 0, int64_t b_stored_rows = 0);
int launch_sgemm(const moc_gemm_desc* g, const float* a, const float* b, float* c, const float* row_scale,
                 cudaStream_t stream);
int launch_delta(int dtype, const void* o, const void* d_o, float* delta, int B, int L, int H, int D,
                 cudaStream_t stream);
int launch_attn_f32_fwd(const moc_attn_shape* s, const float* q, const float* kv, float* o, float* lse,
                        cudaStream_t stream);
int launch_attn_f32_bwd(const moc_attn_shape* s, const float* q, const float* kv, const float* d_o,
                        const float* lse, const float* delta, float* d_q, float* d_kv, cudaStream_t stream);
int launch_attn_tc_fwd(const moc_attn_shape* s, const void* q, const void* kv, void* o, float* lse,
                       int32_t* status, cudaStream_t stream);
int launch_attn_tc_bwd(const moc_attn_shape* s, const void* q, const void* kv, const void* o, const float* lse,
                       const void* d_o, void* d_q, void* d_kv, float* scratch, int32_t* status,
                       cudaStream_t stream, int parts, const float* kv_row_scale = nullptr, float* kv_dot = nullptr);
}  // namespace moc

using namespace moc;

extern "C" int moc_gemm(const moc_gemm_desc* g, const void* a, const void* b, void* c, const float* row_scale,
                        const int32_t* a_row_blocks, int32_t* status, void* stream_) {
  MOC_REQUIRE(g && a && b && c && status, "NULL projection argument");
  MOC_REQUIRE(g->m > 0 && g->n > 0 && g->k > 0, "empty projection");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (g->dtype == MOC_F32) {
    MOC_REQUIRE(a_row_blocks == nullptr, "the fp32 projection takes gathered rows, not a gather list");
    return launch_sgemm(g, static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(c),
                        row_scale, stream);
  }
  if (g->dtype == MOC_BF16) return launch_gemm_tc(g, a, b, c, row_scale, a_row_blocks, status, stream);
  set_last_error("dtype", "unknown dtype");
  return MOC_ERR_INVALID;
}

static int check_attn(const moc_attn_shape* s) {
  MOC_REQUIRE(s != nullptr, "shape is NULL");
  MOC_REQUIRE(s->batch > 0 && s->seq > 0 && s->n_sel > 0, "empty attention problem");
  MOC_REQUIRE(s->num_heads > 0 && s->num_kv_heads > 0 && s->num_heads % s->num_kv_heads == 0,
              "num_heads must be a positive multiple of num_kv_heads");
  return MOC_OK;
}

extern "C" int moc_attn_fwd(const moc_attn_shape* s, const void* q, const void* kv, void* o, float* lse,
                            int32_t* status, void* stream_) {
  int rc = check_attn(s);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(q && kv && o && lse && status, "NULL attention buffer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (s->dtype == MOC_F32)
    return launch_attn_f32_fwd(s, static_cast<const float*>(q), static_cast<const float*>(kv),
                               static_cast<float*>(o), lse, stream);
  if (s->dtype == MOC_BF16) return launch_attn_tc_fwd(s, q, kv, o, lse, status, stream);
  set_last_error("dtype", "unknown dtype");
  return MOC_ERR_INVALID;
}

extern "C" int moc_attn_bwd_parts(const moc_attn_shape* s, const void* q, const void* kv, const void* o,
                                  const float* lse, const void* d_o, void* d_q, void* d_kv, float* delta,
                                  int32_t parts, int32_t* status, void* stream_) {
  int rc = check_attn(s);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(q && kv && o && lse && d_o && d_q && d_kv && delta && status, "NULL attention buffer");
  MOC_REQUIRE(s->dtype == MOC_BF16, "per-kernel launches exist for the bf16 kernels only");
  return launch_attn_tc_bwd(s, q, kv, o, lse, d_o, d_q, d_kv, delta, status, static_cast<cudaStream_t>(stream_),
                            parts);
}

extern "C" int moc_attn_bwd(const moc_attn_shape* s, const void* q, const void* kv, const void* o,
                            const float* lse, const void* d_o, void* d_q, void* d_kv, float* delta,
                            int32_t* status, void* stream_) {
  int rc = check_attn(s);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(q && kv && o && lse && d_o && d_q && d_kv && delta && status, "NULL attention buffer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (s->dtype == MOC_F32) {
    rc = launch_delta(MOC_F32, o, d_o, delta, s->batch, s->seq, s->num_heads, s->head_dim, stream);
    if (rc != MOC_OK) return rc;
    return launch_attn_f32_bwd(s, static_cast<const float*>(q), static_cast<const float*>(kv),
                               static_cast<const float*>(d_o), lse, delta, static_cast<float*>(d_q),
                               static_cast<float*>(d_kv), stream);
  }
  if (s->dtype == MOC_BF16) return launch_attn_tc_bwd(s, q, kv, o, lse, d_o, d_q, d_kv, delta, status, stream, 7);
  set_last_error("dtype", "unknown dtype");
  return MOC_ERR_INVALID;
}


extern "C" int moc_row_dot(const void* a, const void* b, int32_t dtype, float* out, int64_t rows, int32_t dim,
                           void* stream_) {
  MOC_REQUIRE(a && b && out && rows > 0 && dim > 0, "bad row-dot arguments");
  MOC_REQUIRE(dtype == MOC_F32 || dtype == MOC_BF16, "bad dtype");
  MOC_REQUIRE(rows <= 0x7fffffffLL, "too many rows");
  // one (batch, head) with `rows` positions: delta[l] = <a[l, :], b[l, :]>
  return launch_delta(dtype, a, b, out, 1, static_cast<int>(rows), 1, dim, static_cast<cudaStream_t>(stream_));
}


extern "C" int moc_gemm_gather_b(const moc_gemm_desc* g, const void* a, const void* b, void* c,
                                 const float* row_scale, const int32_t* b_row_blocks, int32_t b_block_rows,
                                 int64_t b_stored_rows, int32_t* status, void* stream_) {
  MOC_REQUIRE(g && a && b && c && status && b_row_blocks, "NULL projection argument");
  MOC_REQUIRE(g->m > 0 && g->n > 0 && g->k > 0, "empty projection");
  MOC_REQUIRE(g->dtype == MOC_BF16, "the gathered-B projection is a bf16 tensor-core kernel");
  return launch_gemm_tc(g, a, b, c, row_scale, nullptr, status, static_cast<cudaStream_t>(stream_), b_row_blocks,
                        b_block_rows, b_stored_rows);
}

extern "C" int moc_attn_bwd_scaled_parts(const moc_attn_shape* s, const void* q, const void* kv, const void* o,
                                         const float* lse, const void* d_o, void* d_q, void* d_kv, float* delta,
                                         const float* kv_row_scale, float* kv_dot, int32_t parts, int32_t* status,
                                         void* stream_) {
  int rc = check_attn(s);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(q && kv && o && lse && d_o && d_q && d_kv && delta && status, "NULL attention buffer");
  MOC_REQUIRE(s->dtype == MOC_BF16, "the row-scaled backward exists for the bf16 kernels only");
  return launch_attn_tc_bwd(s, q, kv, o, lse, d_o, d_q, d_kv, delta, status, static_cast<cudaStream_t>(stream_),
                            parts, kv_row_scale, kv_dot);
}

extern "C" int moc_attn_bwd_scaled(const moc_attn_shape* s, const void* q, const void* kv, const void* o,
                                   const float* lse, const void* d_o, void* d_q, void* d_kv, float* delta,
                                   const float* kv_row_scale, float* kv_dot, int32_t* status, void* stream_) {
  int rc = check_attn(s);
  if (rc != MOC_OK) return rc;
  MOC_REQUIRE(q && kv && o && lse && d_o && d_q && d_kv && delta && status && kv_row_scale, "NULL attention buffer");
  MOC_REQUIRE(s->dtype == MOC_BF16, "the row-scaled backward exists for the bf16 kernels only");
  return launch_attn_tc_bwd(s, q, kv, o, lse, d_o, d_q, d_kv, delta, status, static_cast<cudaStream_t>(stream_), 7,
                            kv_row_scale, kv_dot);
}
