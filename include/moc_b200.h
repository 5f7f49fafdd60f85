/* moc_b200 -- C ABI of the B200 (sm_100a) Mixture-of-Chapters memory cross-attention kernels.
 *
 * Conventions
 *   - every pointer named d_* or documented "device" is a CUDA device pointer owned by the caller;
 *     the library allocates nothing unless a function says so;
 *   - `stream` is a cudaStream_t passed as void*; every call only enqueues work on it;
 *   - return value: MOC_OK or a negative MOC_ERR_* (moc_last_error() gives the text); nothing aborts;
 *   - `status` is a device int32 the kernels raise (atomicMax) to a MOC_DEV_* code when a bounded device
 *     wait gives up or a chapter id is out of range; the caller clears and reads it;
 *   - tensors are row-major and contiguous unless a leading dimension is given;
 *   - dtype codes: MOC_F32 = 0, MOC_BF16 = 1.
 *
 * Each entry point names the reference interface (file:line inside the Memory project) it stands in for.
 */
#ifndef MOC_B200_H_
#define MOC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOC_OK 0
#define MOC_ERR_INVALID (-1)
#define MOC_ERR_CUDA (-2)
#define MOC_ERR_UNSUPPORTED (-3)

#define MOC_DEV_OK 0
#define MOC_DEV_TIMEOUT 1
#define MOC_DEV_BAD_INDEX 2

#define MOC_F32 0
#define MOC_BF16 1

#define MOC_NORM_NONE 0
#define MOC_NORM_RMS 1
#define MOC_NORM_LAYERNORM 2

/* Text of the last error raised on the calling thread ("" if none). */
const char* moc_last_error(void);
/* ABI version of this library. */
int moc_abi_version(void);

/* Self-test of the bounded device wait every kernel of this library uses on its barriers.  One CTA waits on a
 * barrier that expects `expected` arrivals while only `arrivals` are made; the wait polls at most `poll_limit`
 * times, then raises MOC_DEV_TIMEOUT in `status` and the kernel returns normally.  out[0] = 1 if the wait
 * succeeded, out[1] = result of a second wait, out[2] = the CTA's abort flag.  No counterpart in the reference
 * (its kernels have no device-side waits). */
int moc_wait_probe(int32_t expected, int32_t arrivals, uint32_t poll_limit, int32_t* status, int32_t* out,
                   void* stream);

/* Barrier between the ranks of one node through flag words in each other's memory (peer-mapped device pointers,
 * e.g. views of one symmetric-memory allocation): flag_arrays[r] points at rank r's array of `world` uint32 words,
 * zero before the first use; `epoch` must grow by one per call (the same on every rank).  The kernel stores the epoch
 * into every peer's array (release, system scope: work this stream did before -- copy-engine pushes into the peers'
 * buffers -- is visible first) and waits, at most poll_limit polls per peer, for the peers' stores into its own;
 * a wait that runs out raises MOC_DEV_TIMEOUT in `status` and the kernel returns.  Replaces the collective a DDP
 * bucket all-reduce provides as a side effect (the reference syncs gradients with torch DDP, training/trainer.py)
 * where the data itself travels by copy engine. */
int moc_peer_barrier(const void* const* flag_arrays, int32_t rank, int32_t world, uint32_t epoch, uint32_t poll_limit,
                     int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Router.  Replaces ChapterRouter.forward / _compute_losses (memory_transformer/router.py:94-156,
 * 197-260) and MemoryTransformer._prepend_shared_chapters (memory_transformer/model.py:356-391).
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t batch;         /* B */
  int32_t seq;           /* L */
  int32_t hidden_dim;    /* d */
  int32_t num_chapters;  /* C, shared prefix included */
  int32_t top_k;         /* requested k; k' = min(k, C - num_shared) chapters are returned */
  int32_t num_shared;    /* S, chapters [0,S) are always on and excluded from selection */
  float routed_scale;    /* rho, multiplies the routed weights before the joint renormalisation */
  int32_t h_dtype;       /* dtype of the hidden states */
} moc_router_shape;

/* Bytes of device scratch moc_router_fwd / moc_router_bwd need. */
size_t moc_router_workspace_bytes(const moc_router_shape* s);
/* The same for a call restricted to some parts (bit sets as in moc_router_fwd_parts / moc_router_bwd_parts; 0 = that
 * direction is not called with this workspace).  A token-level call (fwd bits 8 + 16, bwd bit 1 only) needs a few
 * hundred bytes where the sequence-level layout would reserve batch-sized pooling scratch. */
size_t moc_router_workspace_bytes_parts(const moc_router_shape* s, int32_t fwd_parts, int32_t bwd_parts);

/* Forward.  Outputs (device): pooled [B,d], logits [B,C], probs [B,C] (fp32);
 * idx [B,k'] int64 and weights [B,k'] (sorted by weight descending, ties to the lower chapter id);
 * comb_idx [B,S+k'] int32 and comb_w [B,S+k'] (shared prefix first);
 * row_stats [B,4] = {logsumexp, masked mass, top-k mass, combined mass};
 * chapter_stats [2,C] = {selection fraction f, mean squared probability};
 * losses [4] = {load_balance, auxiliary, z_loss, entropy}, or NULL to skip them. */
int moc_router_fwd(const moc_router_shape* s, const void* h, const float* w, const float* bias,
                   float* pooled, float* logits, float* probs, int64_t* idx, float* weights,
                   int32_t* comb_idx, float* comb_w, float* row_stats, float* chapter_stats, float* losses,
                   void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* moc_router_fwd in two pieces: parts bit 1 = pooling, logits, selection (everything the gather needs),
 * bit 2 = the loss terms (reads probs / idx / row_stats of bit 1), bit 8 (with bit 1) = `pooled` already holds
 * the pooled states, e.g. from moc_pool_weighted_fwd, and `h` is not read; bit 16 (with bit 1) = `logits` already
 * holds pooled x W^T from a projection kernel and only the bias is added before the selection.  Bits 8 + 16 with
 * batch = B*L rows and seq = 1 are ChapterRouter.route_token_level (memory_transformer/router.py:262-340): every
 * token is its own routing row.  A caller can wait for bit 1 only and let the
 * losses finish beside the gather.  moc_router_fwd is parts = 3.  No counterpart in the reference. */
int moc_router_fwd_parts(const moc_router_shape* s, const void* h, const float* w, const float* bias,
                         float* pooled, float* logits, float* probs, int64_t* idx, float* weights,
                         int32_t* comb_idx, float* comb_w, float* row_stats, float* chapter_stats, float* losses,
                         void* workspace, size_t workspace_bytes, int32_t parts, int32_t* status, void* stream);

/* Backward of the above (autograd of router.py:94-156,197-260 and model.py:356-391).
 * d_weights [B,k'] and d_comb_w [B,S+k'] are the incoming gradients of the two weight outputs (either
 * may be NULL); d_losses [4] (device) the incoming gradients of the four loss scalars (NULL = none).
 * Outputs: d_logits [B,C], d_w [C,d], d_bias [C], d_pooled [B,d]; d_h [B,L,d] in h_dtype receives
 * d_pooled / L on every position (added to its contents when accumulate_dh != 0; NULL to skip). */
int moc_router_bwd(const moc_router_shape* s, const float* w, const float* pooled, const float* probs,
                   const int64_t* idx, const float* weights, const float* comb_w, const float* row_stats,
                   const float* chapter_stats, const float* d_weights, const float* d_comb_w,
                   const float* d_losses, float* d_logits, float* d_w, float* d_bias, float* d_pooled,
                   void* d_h, int32_t accumulate_dh, void* workspace, size_t workspace_bytes,
                   int32_t* status, void* stream);

/* moc_router_bwd in pieces, so that a caller can put them on different streams: parts is a bit set of
 * 1 = d_logits, 2 = d_w and d_bias (reads d_logits), 4 = d_pooled and d_h (reads d_logits).  Same buffers in
 * every call; moc_router_bwd is parts = 7.  No counterpart in the reference. */
int moc_router_bwd_parts(const moc_router_shape* s, const float* w, const float* pooled, const float* probs,
                         const int64_t* idx, const float* weights, const float* comb_w, const float* row_stats,
                         const float* chapter_stats, const float* d_weights, const float* d_comb_w,
                         const float* d_losses, float* d_logits, float* d_w, float* d_bias, float* d_pooled,
                         void* d_h, int32_t accumulate_dh, void* workspace, size_t workspace_bytes, int32_t parts,
                         int32_t* status, void* stream);

/* Position-weighted pooling: pooled[b, :] = sum_t pos_weight[t] * h[b, t, :] (fp32 accumulation), and its
 * backward d_h[b, t, :] (+)= pos_weight[t] * d_pooled[b, :].  With the coefficients of the rolling-window rule this
 * replaces ChapterRouter._sequence_rolling_pool (memory_transformer/router.py:159-195): the average over t of the
 * window means mean(h[max(0, t-w+1) .. t]) is linear in h, so it is one coefficient per position.  Feed the result to
 * moc_router_fwd_parts with parts bit 8.  workspace: batch * 32 * dim floats. */
int moc_pool_weighted_fwd(const void* h, int32_t h_dtype, const float* pos_weight, float* pooled, int32_t batch,
                          int32_t seq, int32_t dim, void* workspace, size_t workspace_bytes, void* stream);
int moc_pool_weighted_bwd(const float* d_pooled, const float* pos_weight, void* d_h, int32_t h_dtype,
                          int32_t batch, int32_t seq, int32_t dim, int32_t accumulate, void* stream);

/* out[c] = sum over rows of x[r, c] (fp32, fixed summation order): the router bias gradient of the token-level
 * path, where the logit gradient has one row per token (autograd of router.py:294). */
int moc_col_sum(const float* x, float* out, int64_t rows, int32_t cols, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Chapter gather.  Replaces ChapteredMemoryBank.get_chapters_batched (memory_bank.py:244-293), the
 * optional per-row normalisation (model.py:393-432) and the weight multiply (model.py:689-692).
 * ---------------------------------------------------------------------------------------------- */
/* out[b, s*T + r, :] = comb_w[b,s] * norm(bank[comb_idx[b,s]*T + r, :]).
 * comb_w may be NULL (no scaling).  row_stats [B*K*T, 2] = {mean, 1/std or 1/rms} is written when
 * norm_type != MOC_NORM_NONE (may be NULL otherwise). */
int moc_gather_rows_fwd(const void* bank, int32_t bank_dtype, int64_t bank_rows, int32_t dim,
                        int32_t tokens_per_chapter, const int32_t* comb_idx, const float* comb_w,
                        int32_t batch, int32_t k_sel, int32_t norm_type, float eps, void* out,
                        int32_t out_dtype, float* row_stats, int32_t* status, void* stream);

/* Groups the B*K (batch, slot) pairs by chapter id, deterministically.
 * uniq [<=n_pairs] ascending chapter ids, seg_offsets [n_pairs+1], seg_pairs [n_pairs] pair ids grouped by
 * chapter and ascending inside a group, pair_to_uniq [n_pairs], num_unique [1].  One CTA; n_pairs <= 65536. */
int moc_chapter_segments(const int32_t* comb_idx, int32_t n_pairs, int32_t num_chapters, int32_t* uniq,
                         int32_t* seg_offsets, int32_t* seg_pairs, int32_t* pair_to_uniq,
                         int32_t* num_unique, int32_t* status, void* stream);

/* Backward of moc_gather_rows_fwd: the scatter-add that torch.gather's autograd performs densely
 * (memory_bank.py:291) done only on touched rows.
 * d_mem [B*K*T, dim] (fp32 or bf16) is the gradient of the scaled rows.
 * d_comb_w [B,K] <- sum over the slot's rows of <d_mem, norm(bank row)>.
 * bank_grad [num_unique*T, dim] fp32, compact: block u holds the gradient of chapter uniq[u];
 * bank_grad_bf16 (may be NULL): the same rows once more in bf16, for a gradient exchange that sends half the bytes. */
int moc_gather_rows_bwd(const void* d_mem, int32_t d_mem_dtype, const void* bank, int32_t bank_dtype,
                        int64_t bank_rows, int32_t dim, int32_t tokens_per_chapter, const int32_t* comb_idx,
                        const float* comb_w, int32_t batch, int32_t k_sel, int32_t norm_type, float eps,
                        const float* row_stats, const int32_t* uniq, const int32_t* seg_offsets,
                        const int32_t* seg_pairs, const int32_t* num_unique, float* d_comb_w,
                        float* bank_grad, void* bank_grad_bf16, int32_t* status, void* stream);

/* ---- Fused gather-and-project path (no gathered rows are materialised) ----------------------------------------
 * Forward: moc_gemm with the TMA gather list over a bf16 copy of the bank and row_scale[pair*T + r] = u~[pair]
 * (times 1/rms of the bank row when the rows are RMS-normalised, model.py:423-425) -- get_chapters_batched, the
 * normalisation, the weight multiply and k_proj / v_proj (memory_bank.py:263-293, model.py:393-432, 689-692,
 * memory_attention.py:241-243) in one kernel.  Backward: moc_attn_bwd_scaled writes dK / dV already multiplied by
 * the same row scale; g' = dKV' x [Wk; Wv] is then s_r * dM~_r, from which moc_gather_rows_bwd_prescaled derives the
 * chapter-weight gradient and the compact bank gradient, and moc_gemm_gather_b forms the Wk / Wv gradient reading the
 * bank rows through the same list.
 * moc_row_inv_rms: out[row] = 1 / sqrt(mean(row^2) + eps) for every bank row (refresh after an update).
 * moc_chapter_row_scale: scale [n_pairs*T]; inv_rms may be NULL (no normalisation). */
int moc_row_inv_rms(const void* bank, int32_t bank_dtype, int64_t rows, int32_t dim, float eps, float* out,
                    void* stream);
int moc_chapter_row_scale(const int32_t* comb_idx, const float* comb_w, const float* inv_rms, int64_t bank_rows,
                          int32_t n_pairs, int32_t tokens_per_chapter, float* scale, int32_t* status, void* stream);
/* g [n_pairs*T, dim] = s_r * dM~_r (fp32 or bf16); bank: the rows the forward read (its bf16 copy, or fp32);
 * inv_rms [bank_rows] or NULL.  d_comb_w [n_pairs] = (1/u~) sum_r <g_r, m_r>; bank_grad compact fp32 as in
 * moc_gather_rows_bwd (bank_grad_bf16 optional second copy). */
int moc_gather_rows_bwd_prescaled(const void* g, int32_t g_dtype, const void* bank, int32_t bank_dtype,
                                  int64_t bank_rows, int32_t dim, int32_t tokens_per_chapter,
                                  const int32_t* comb_idx, const float* comb_w, int32_t n_pairs,
                                  const float* inv_rms, const int32_t* uniq, const int32_t* seg_offsets,
                                  const int32_t* seg_pairs, const int32_t* num_unique, float* d_comb_w,
                                  float* bank_grad, void* bank_grad_bf16, int32_t* status, void* stream);

/* Consumer of a data-parallel gradient exchange: the ranks' compact bank-gradient rows summed over the UNION of
 * their chapter lists (the sum DDP's dense all-reduce of the bank gradient produces, training/trainer.py:873, on
 * the touched chapters only).  rank_rows: host array of `world` device pointers, rank r's rows [per_rank*T, dim]
 * (fp32 or bf16); ids_all [world, per_rank] int32 chapter ids, of which the first counts[r] of rank r are filled.
 * Outputs: uniq (ascending union) / num_unique, seg_offsets / seg_pairs / pair_to_uniq (scratch, world*per_rank (+1)
 * ints each), rows_out fp32 [num_unique*T, dim] = scale * sum over the ranks holding each chapter, added in
 * ascending (rank, slot) order, so every rank computes identical bits.  rows_out_capacity (rows) must cover
 * min(world*per_rank, num_chapters) chapters. */
int moc_bank_grad_merge(const void* const* rank_rows, int32_t rows_dtype, int32_t world, const int32_t* ids_all,
                        const int32_t* counts, int32_t per_rank, int32_t tokens_per_chapter, int32_t dim,
                        int32_t num_chapters, float scale, int32_t* uniq, int32_t* seg_offsets, int32_t* seg_pairs,
                        int32_t* pair_to_uniq, int32_t* num_unique, float* rows_out, int64_t rows_out_capacity,
                        int32_t* status, void* stream);
/* The same with the output dtype chosen by the caller (MOC_F32 or MOC_BF16; sums are formed in fp32 either way):
 * bf16 mean rows halve what the consumer of an exchange writes at a rounding of 2^-9 relative. */
int moc_bank_grad_merge_to(const void* const* rank_rows, int32_t rows_dtype, int32_t world, const int32_t* ids_all,
                           const int32_t* counts, int32_t per_rank, int32_t T, int32_t dim, int32_t num_chapters,
                           float scale, int32_t* uniq, int32_t* seg_offsets, int32_t* seg_pairs,
                           int32_t* pair_to_uniq, int32_t* num_unique, void* rows_out, int32_t rows_out_dtype,
                           int64_t rows_out_capacity, int32_t* status, void* stream);

/* bank_dense[uniq[u]*T + r, :] += bank_grad[u*T + r, :]  (fp32). */
int moc_scatter_bank_grad(const float* bank_grad, const int32_t* uniq, const int32_t* num_unique,
                          int32_t max_unique, int32_t tokens_per_chapter, int32_t dim, float* bank_dense,
                          int64_t bank_rows, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Dense projections.  Replaces the nn.Linear calls of MemoryCrossAttention._compute_qkv and
 * _project_output (memory_attention.py:241-243, 456) and their autograd.
 *   C[M,N] (+)= op(A)[M,K] * op(B)[K,N]
 *   a_kmajor != 0: A is stored [M,K] (lda = row stride), else stored [K,M];
 *   b_kmajor != 0: B is stored [N,K] (the nn.Linear weight layout), else stored [K,N].
 * dtype MOC_F32: fp32 FMA kernel, any shape.  dtype MOC_BF16: tcgen05 kernel, bf16 operands, fp32
 * accumulation in tensor memory, K % 8 == 0 and 16-byte aligned rows; c_dtype is the output type.
 * row_scale (device, may be NULL): C row m is multiplied by row_scale[m / scale_block_rows].
 * a_row_blocks (device int32, may be NULL; bf16, a_kmajor only): gather list -- rows
 * [i*block, (i+1)*block) of op(A) are rows [a_row_blocks[i]*block, ...) of the stored A, block =
 * a_block_rows (8..128, divides 128): this is the fused chapter gather + Wk/Wv projection, with the
 * chapter rows fetched by TMA straight from the bank.
 * accumulate != 0 adds into C (fp32 C only); split_k > 1 splits K over CTAs with fp32 atomics
 * (fp32 C only, C must be pre-zeroed or accumulate set).
 * residual (device fp32 [M,N], row stride ldr, may be NULL): added to the product before it is stored,
 * C = row_scale * (A B) + residual -- the residual add that follows the output projection in the
 * reference's block (memory_block.py:558) done in the projection's epilogue. */
typedef struct {
  int32_t dtype, c_dtype;
  int32_t m, n, k;
  int32_t a_kmajor, b_kmajor;
  int64_t lda, ldb, ldc;
  int32_t accumulate, split_k;
  int32_t scale_block_rows;
  int32_t a_block_rows;
  int64_t a_stored_rows;   /* rows of the stored A when a gather list is used */
  const float* residual;
  int64_t ldr;
} moc_gemm_desc;

int moc_gemm(const moc_gemm_desc* g, const void* a, const void* b, void* c, const float* row_scale,
             const int32_t* a_row_blocks, int32_t* status, void* stream);

/* moc_gemm with a gather list over the K rows of an MN-major B ([K, N] row-major, g->b_kmajor = 0): logical K row
 * j*b_block_rows + r is stored row b_row_blocks[j]*b_block_rows + r of a matrix with b_stored_rows rows.  This is
 * how the Wk / Wv weight gradient dKV'^T x (selected bank rows) reads the bank without a gathered copy.  bf16 only;
 * b_block_rows a multiple of 8 that divides 64 or is a multiple of 64. */
int moc_gemm_gather_b(const moc_gemm_desc* g, const void* a, const void* b, void* c, const float* row_scale,
                      const int32_t* b_row_blocks, int32_t b_block_rows, int64_t b_stored_rows, int32_t* status,
                      void* stream);

/* ------------------------------------------------------------------------------------------------
 * Normalisation in front of the memory cross-attention.  Replaces `memory_layernorm` of
 * MemoryTransformerBlock (memory_block.py:475, 551, 578): RMSNorm (memory_block.py:18-28,
 * x / sqrt(mean(x^2) + eps) * weight) when kind = MOC_NORM_RMS, torch.nn.LayerNorm when kind =
 * MOC_NORM_LAYERNORM (bias may be NULL).
 *   x [rows, dim] fp32, dim % 4 == 0; y_f32 and / or y_bf16 [rows, dim] receive the result (either may be
 *   NULL, not both): the bf16 copy is the operand of the query projection, so no separate cast runs;
 *   stats [rows, 2] fp32 = (mean, 1 / sqrt(var + eps)) per row, kept for the backward pass.
 * moc_norm_bwd: dy is the gradient of the normalised rows; dx = norm-gradient + residual_grad (fp32
 * [rows, dim] or NULL: the gradient that reaches x through the residual connection, memory_block.py:558);
 * dweight / dbias [dim] (may be NULL; dbias only for LayerNorm); workspace of
 * moc_norm_bwd_workspace_bytes(rows, dim) bytes holds per-block column sums.
 * ---------------------------------------------------------------------------------------------- */
size_t moc_norm_bwd_workspace_bytes(int64_t rows, int32_t dim);
int moc_norm_fwd(const float* x, const float* weight, const float* bias, int32_t kind, float eps,
                 int64_t rows, int32_t dim, float* y_f32, void* y_bf16, float* stats, void* stream);
int moc_norm_bwd(const float* dy, const float* x, const float* weight, const float* stats,
                 const float* residual_grad, int32_t kind, int64_t rows, int32_t dim, float* dx,
                 float* dweight, float* dbias, void* workspace, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Joint-softmax cross attention over the gathered chapters.  Replaces MemoryCrossAttention._attention
 * (memory_attention.py:298-316) and its autograd.
 *   q  [B, L, H*D]; kv [B, n_sel, 2*HK*D] = K heads then V heads per row; o [B, L, H*D];
 *   lse [B, H, L] fp32 (natural log of the softmax denominator of the scaled scores).
 * dtype MOC_F32: FMA kernels, D in {16,32,64,128}.  dtype MOC_BF16: tcgen05 kernels, D = 64.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t batch, seq, n_sel, num_heads, num_kv_heads, head_dim;
  float scale;
  int32_t dtype;
} moc_attn_shape;

int moc_attn_fwd(const moc_attn_shape* s, const void* q, const void* kv, void* o, float* lse,
                 int32_t* status, void* stream);
/* delta is scratch of 6*B*H*L floats, 16-byte aligned (per-row <O,dO>, rescaled log-sum-exp, and the packed
 * bf16 rows the dK/dV kernel feeds to the tensor cores).  d_q like q, d_kv like kv. */
int moc_attn_bwd(const moc_attn_shape* s, const void* q, const void* kv, const void* o, const float* lse,
                 const void* d_o, void* d_q, void* d_kv, float* delta, int32_t* status, void* stream);

/* Measurement aid for the bf16 backward, same arguments as moc_attn_bwd: runs only the kernels selected by
 * `parts` (1 = delta / log-sum-exp preparation, 2 = dQ kernel, 4 = dK/dV kernel), so each can be timed
 * alone.  moc_attn_bwd is parts = 7.  No counterpart in the reference. */
int moc_attn_bwd_parts(const moc_attn_shape* s, const void* q, const void* kv, const void* o, const float* lse,
                       const void* d_o, void* d_q, void* d_kv, float* delta, int32_t parts, int32_t* status,
                       void* stream);

/* moc_attn_bwd (bf16 only) whose dK / dV rows leave multiplied by kv_row_scale [B*n_sel]: the backward half of the
 * fused gather-and-project path described at moc_row_inv_rms.  kv_dot (may be NULL; needs n_sel % 64 == 0):
 * [B, n_sel/64, HK] fp32, per 64-key block and KV head the sum over its rows of <dK, K> + <dV, V> with the unscaled
 * dK / dV -- for 64-row chapters, summed over the heads and divided by the chapter weight, this is the chapter-weight
 * gradient (d u~ = sum_r <dM~_r, M~_r> / u~ and <dM~_r, M~_r> = <dKV_r, KV_r>), taken while the K / V tile is
 * still in shared memory.  No counterpart in the reference. */
int moc_attn_bwd_scaled(const moc_attn_shape* s, const void* q, const void* kv, const void* o, const float* lse,
                        const void* d_o, void* d_q, void* d_kv, float* delta, const float* kv_row_scale,
                        float* kv_dot, int32_t* status, void* stream);
/* The same in pieces (parts as in moc_attn_bwd_parts: 1 = per-row constants, 2 = dQ, 4 = dK/dV; kv_row_scale may be
 * NULL): lets a caller run the dQ kernel and the dK/dV kernel on different streams once the constants are there. */
int moc_attn_bwd_scaled_parts(const moc_attn_shape* s, const void* q, const void* kv, const void* o, const float* lse,
                              const void* d_o, void* d_q, void* d_kv, float* delta, const float* kv_row_scale,
                              float* kv_dot, int32_t parts, int32_t* status, void* stream);

/* moc_attn_bwd without caller-provided scratch and without any allocation.  It has no counterpart in the
 * reference.  It exists for callers that are not allowed to allocate device memory when they run the
 * backward pass (a serving process whose memory pool is frozen, a callback in which cudaMalloc is
 * forbidden, a host program whose allocator cannot be reached from C).  The delta / log-sum-exp scratch
 * lives in a fixed 4 MiB array inside the library image, so 6 * batch * num_heads * seq must not exceed
 * MOC_ATTN_BWD_STATIC_MAX_FLOATS; larger problems are rejected with MOC_ERR_INVALID.
 * The first call on each device looks the array's device address up (with that device current): make
 * that first call outside any stream capture.  All calls on a device share the one array: two calls
 * whose kernels can overlap on the GPU (different streams, no dependency) race on it and must be
 * serialised by the caller.  Results equal moc_attn_bwd's. */
#define MOC_ATTN_BWD_STATIC_MAX_FLOATS 1048576
int moc_attn_bwd_static(const moc_attn_shape* s, const void* q, const void* kv, const void* o, const float* lse,
                        const void* d_o, void* d_q, void* d_kv, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Decode-time memory attention over a cache of projected bank rows.  The reference re-gathers and
 * re-projects (S+k)*T bank rows per sequence at every generated token (inference/generate.py:194-210 ->
 * model.py:624-692 -> memory_attention.py:241-243); it has no such cache.  Because the chapter weight
 * multiplies a row before the linear projection, K = u_c * (norm(m) Wk^T): the per-layer cache
 *   kv_bank [C*T, 2*HK*64] bf16 = norm(M) [Wk; Wv]^T   (built once per weight state with moc_gemm)
 * gives the same attention from a gather of cached rows:
 *   s_r = scale * u_c * <q, K_bank[r]>,  out = sum_r softmax_r(s) * u_c * V_bank[r]   (one joint softmax).
 *   q, out [B, n_q, H*64] bf16; comb_idx [B, n_chapters] int32 (shared prefix first), comb_w [B, n_chapters]
 *   fp32 as produced by moc_router_fwd; lse [B, n_q, H] fp32 (may be NULL).  Chapter ids outside the cache
 *   raise MOC_DEV_BAD_INDEX in the status word and are skipped.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t batch, n_q, num_heads, num_kv_heads, head_dim, n_chapters, tokens_per_chapter;
  float scale;
} moc_decode_shape;

int moc_decode_attn(const moc_decode_shape* s, const void* q, const void* kv_bank, int64_t bank_rows,
                    const int32_t* comb_idx, const float* comb_w, void* out, float* lse, int32_t* status,
                    void* stream);

/* ------------------------------------------------------------------------------------------------
 * Per-token chapter-sparse attention: the contract of memory_cross_attn(q, k, v, block_indices,
 * block_size, scale) (kernels-final/memory_cross_attn.py:1310-1366, 1387-1603, 1639-1652).
 *   q [B,TQ,HQ,D], k/v [B,TK,H,D], block_indices [B,TQ,H,S] int32, o [B,TQ,HQ,D], lse [B,TQ,HQ].
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t batch, tq, tk, hq, h, head_dim, n_select, block_size;
  float scale;
  int32_t dtype;
} moc_sparse_attn_shape;

int moc_sparse_attn_fwd(const moc_sparse_attn_shape* s, const void* q, const void* k, const void* v,
                        const int32_t* block_indices, void* o, float* lse, int32_t* status, void* stream);
/* d_k / d_v are fp32 [B,TK,H,D] accumulators the call zeroes and fills (atomic adds). */
int moc_sparse_attn_bwd(const moc_sparse_attn_shape* s, const void* q, const void* k, const void* v,
                        const int32_t* block_indices, const void* o, const float* lse, const void* d_o,
                        void* d_q, float* d_k, float* d_v, int32_t* status, void* stream);

/* out[r] = <a[r, :], b[r, :]> in fp32 for contiguous [rows, dim] operands: the per-(token, head) delta = <o, do> of
 * memory_cross_attn_preprocess_delta (kernels-final/memory_cross_attn.py:1369-1384). */
int moc_row_dot(const void* a, const void* b, int32_t dtype, float* out, int64_t rows, int32_t dim, void* stream);

/* Weighted mixture rule: every selected chapter has its own softmax and the per-chapter outputs are mixed by
 * router weights, o = base + out_scale * sum_s w[b,t,s] * softmax(q K_s^T * scale) V_s -- the contract of
 * FSA_topk_sparse_attention_weighted_bthd (kernels-final/kernel_v4.py:972-1027, 1313-1340) and, with base = the
 * dense shared-chapter branch and out_scale = routed_scale, the routed branch of
 * MemoryCrossAttention._forward_token_routed_attention (memory_transformer/memory_attention.py:550-551, 596-714).
 *   weights fp32 [B,TQ,S]; base like o or NULL; lse_slots fp32 [B,TQ,HQ,S] (every chapter's own log-sum-exp);
 *   kv_row_stride: elements between consecutive rows of k (and of v), H*D when contiguous -- larger when K and V
 *   of one bank row share a projected row. */
int moc_sparse_attn_weighted_fwd(const moc_sparse_attn_shape* s, const void* q, const void* k, const void* v,
                                 int64_t kv_row_stride, const int32_t* block_indices, const float* weights,
                                 const void* base, float out_scale, void* o, float* lse_slots, int32_t* status,
                                 void* stream);
/* Backward (kernels-final/kernel_v4.py:1029-1231).  d_o is the gradient of o.  d_q is written, or added to when
 * accumulate_dq != 0; d_k / d_v are fp32 accumulators with row stride dkv_row_stride that the CALLER has zeroed
 * (atomic adds); d_w_heads fp32 [B,TQ,HQ,S] holds every head's share of the weight gradient (sum over HQ). */
int moc_sparse_attn_weighted_bwd(const moc_sparse_attn_shape* s, const void* q, const void* k, const void* v,
                                 int64_t kv_row_stride, const int32_t* block_indices, const float* weights,
                                 float out_scale, const float* lse_slots, const void* d_o, void* d_q,
                                 int32_t accumulate_dq, float* d_k, float* d_v, int64_t dkv_row_stride,
                                 float* d_w_heads, int32_t* status, void* stream);

/* The same weighted mixture on the tensor cores (bf16, head_dim 64, block_size 64 only): an inverted index
 * chapter -> (token, slot) pairs is built on the device and each chapter's K / V tile stays in shared memory while
 * the query rows that selected it are gathered against it (tcgen05 products, accumulators in tensor memory).
 *   index_heads: 1 when block_indices is [B,TQ,1,S] (one chapter list per token, every head uses it -- the module
 *   path, memory_transformer/memory_attention.py:596-714) or H for [B,TQ,H,S] (kernels-final/kernel_v4.py:972-1027).
 *   workspace: moc_token_mix_workspace_bytes() bytes; moc_token_mix_index fills it, forward and backward read it.
 *   partial / dq_partial: bf16 scratch [B,TQ,S,HQ,D].  Chapter ids outside [0, TK/64) raise MOC_DEV_BAD_INDEX in
 *   the status word and contribute nothing. */
size_t moc_token_mix_workspace_bytes(const moc_sparse_attn_shape* s, int32_t index_heads);
int moc_token_mix_index(const moc_sparse_attn_shape* s, int32_t index_heads, const int32_t* block_indices,
                        void* workspace, int32_t* status, void* stream);
int moc_token_mix_fwd(const moc_sparse_attn_shape* s, int32_t index_heads, const void* q, const void* k, const void* v,
                      int64_t kv_row_stride, const int32_t* block_indices, const float* weights, const void* base,
                      float out_scale, const void* workspace, void* partial, void* o, float* lse_slots,
                      int32_t* status, void* stream);
/* d_q = d_q_base (or 0 when NULL) + the routed branch's gradient; d_k / d_v are bf16 with row stride
 * dkv_row_stride and are WRITTEN in full: the 64 rows of every selected chapter by the one CTA that owns the chapter
 * (pairs in ascending order), zeros for chapters nobody selected -- the caller need not clear them. */
int moc_token_mix_bwd(const moc_sparse_attn_shape* s, int32_t index_heads, const void* q, const void* k, const void* v,
                      int64_t kv_row_stride, const int32_t* block_indices, const float* weights, float out_scale,
                      const float* lse_slots, const void* d_o, const void* workspace, void* dq_partial,
                      const void* d_q_base, void* d_q, void* d_k, void* d_v, int64_t dkv_row_stride,
                      float* d_w_heads, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Optimizer step of the bank from a compact gradient.  Replaces torch.optim.AdamW over the bank parameter
 * (training/trainer.py:372-378, param group "memory_bank" :338-347) fed by the dense gradient of torch.gather's
 * backward: same update for EVERY row (rows of untouched chapters see a zero gradient: moments decay, decoupled
 * weight decay and the remaining momentum still apply), computed in one pass without a dense gradient tensor.
 *   param / exp_avg / exp_avg_sq fp32 [bank_rows, dim], updated in place; uniq / num_unique / grad_rows: the
 *   compact gradient (block u of grad_rows = chapter uniq[u]); grad_scale multiplies the gradient first (1 / world,
 *   a clipping coefficient); step counts from 1 (bias correction); shadow_bf16 (may be NULL) receives the updated
 *   parameter as bf16 -- the working copy the TMA-gather projection reads.
 *   workspace: moc_bank_adamw_workspace_bytes(num_chapters). */
size_t moc_bank_adamw_workspace_bytes(int32_t num_chapters);
int moc_bank_adamw_step(float* param, float* exp_avg, float* exp_avg_sq, int64_t bank_rows, int32_t dim,
                        int32_t tokens_per_chapter, const int32_t* uniq, const int32_t* num_unique,
                        int32_t max_unique, const float* grad_rows, float grad_scale, float lr, float beta1,
                        float beta2, float eps, float weight_decay, int64_t step, void* shadow_bf16,
                        void* workspace, size_t workspace_bytes, int32_t* status, void* stream);
/* out[0] = sum of squares of the first num_unique*T rows of a compact gradient: the bank's share of the global
 * gradient norm that the reference clips by (training/trainer.py:876-880).  workspace: 592 floats. */
int moc_rows_sqnorm(const float* rows, const int32_t* num_unique, int32_t tokens_per_chapter, int32_t dim,
                    float* out, void* workspace, size_t workspace_bytes, void* stream);

/* Element-wise helpers used by the host layer (device pointers, n elements). */
int moc_cast_f32_to_bf16(const float* src, void* dst, int64_t n, void* stream);
int moc_cast_bf16_to_f32(const void* src, float* dst, int64_t n, void* stream);
/* dst bf16 [terms, n]: term t is the bf16 rounding of what terms 0..t-1 left of src (terms <= 3; three terms carry
 * 24 mantissa bits).  Lets an fp32 projection run as sums of exact bf16 tensor-core products -- the per-token
 * router projection nn.Linear(hidden, num_chapters) of ChapterRouter.route_token_level
 * (memory_transformer/router.py:262-340) at [B*L, hidden] x [hidden, C]. */
int moc_split_bf16(const float* src, void* dst, int64_t n, int32_t terms, void* stream);
/* dst[r, c] = bias[c] + sum_t src[r, t * ld + c] (bias may be NULL): folds the column blocks that one product against
 * the stacked terms of a split weight leaves side by side, and adds the router's bias (router.py:294). */
int moc_sum_terms(const float* src, const float* bias, float* dst, int64_t rows, int32_t cols, int32_t ld,
                  int32_t terms, void* stream);
/* dst[c, r] = src[r, c] for a row-major [rows, cols] matrix, converting between the dtype codes.  Used to
 * keep the nn.Linear weights (memory_attention.py:140-143) in the K-major layout the input-gradient
 * projections want. */
int moc_transpose(const void* src, int32_t src_dtype, void* dst, int32_t dst_dtype, int32_t rows, int32_t cols,
                  void* stream);
/* One launch for up to four weight matrices (host arrays of n device pointers / sizes): dst[i] (may be NULL) receives
 * src[i] as bf16 in the same [rows, cols] layout, dst_t[i] (may be NULL) its transpose [cols, rows] with row stride
 * ldt[i] (0 = rows[i]; a larger stride lets Wk^T and Wv^T share one [d, 2*dkv] matrix).  This is the bf16 working
 * copy of the q/k/v/o nn.Linear weights (memory_attention.py:140-143) for one step. */
int moc_pack_weights(int32_t n, const void* const* src, int32_t src_dtype, void* const* dst, void* const* dst_t,
                     const int32_t* rows, const int32_t* cols, const int32_t* ldt, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOC_B200_H_ */
