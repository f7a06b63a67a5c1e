/* C ABI of libflash_msa_b200.so: hand-written sm_100a kernels for the Flash-MSA training path.
 *
 * Conventions
 *  - Every entry point returns an int status: FMSA_OK, or a negative FMSA_ERR_* for a rejected
 *    call (nothing was launched).  Kernels report device-side trouble (a bounded wait that ran
 *    out, an out-of-range index in metadata) in a caller-provided int32 status word on the
 *    device, never by trapping.
 *  - All pointers are device pointers unless stated otherwise.  The library never allocates or
 *    frees device memory; the caller owns every buffer, including workspaces whose size the
 *    *_workspace_bytes functions report.
 *  - Launches go to the given stream and never synchronise with the host.
 *  - Activations are bf16 or fp16 (one type per call) with head dimension 128 and 128-token blocks.  A 4-D activation
 *    (B, H, S, 128) is described by its base pointer and element strides for B, H and S; the
 *    last dimension must be contiguous and rows 16-byte aligned.
 *
 * File:line citations refer to the reference project nanduruganesh/flash-msa.
 */
#ifndef FLASH_MSA_B200_H
#define FLASH_MSA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FMSA_OK 0
#define FMSA_ERR_ARGUMENT (-1)    /* shape / alignment / null pointer */
#define FMSA_ERR_UNSUPPORTED (-2) /* valid request outside the implemented envelope */
#define FMSA_ERR_WORKSPACE (-3)   /* workspace too small */
#define FMSA_ERR_CUDA (-4)        /* the CUDA runtime refused the launch */

#define FMSA_MAX_TOPK_BLOCKS 128

/* Activation types.  The reference accepts both (flash_msa/msa_backward_cutedsl.py:169-183). */
#define FMSA_DTYPE_BF16 0
#define FMSA_DTYPE_FP16 1

/* Strided (B, H, S, 128) bf16 activation. */
typedef struct {
    const void* ptr;
    int64_t stride_b, stride_h, stride_s; /* in elements */
} fmsa_tensor;

/* Head configuration of one call.  Hq main query heads, Hkv key/value heads, Hp proxy query heads,
 * Hpkv proxy key heads; Hq % Hp == 0, Hq % Hkv == 0, Hp % Hkv == 0, Hp % Hpkv == 0.
 * top_k_blocks = top_k / 128 (ignored by the dense warmup paths). */
typedef struct {
    int32_t B, S, Hq, Hkv, Hp, Hpkv, top_k_blocks;
    float scale;
    int32_t dtype; /* FMSA_DTYPE_BF16 or FMSA_DTYPE_FP16: the type of every activation, partial row and gradient */
    /* Document masking of packed sequences (no counterpart in the reference, whose README lists variable-length
     * batches as missing): NULL, or int32 [B,S] on the device holding, for every token, the position of the first
     * token of its document (cu_seqlens[i] for the tokens of document i).  A query then sees only the keys of its own
     * document: block scores, selection, forward and backward (sparse and dense warmup) all honour it. */
    const int32_t* doc_start;
} fmsa_problem;

/* Library ABI version (bumped on any signature change). */
int fmsa_abi_version(void);

/* Test hook: one 128x128x128 tcgen05 product D = A_eff * B_eff^T computed exactly the way the
 * attention kernels do it (cp.async or TMA staging into the swizzled tile layout, one TMEM
 * accumulator, tcgen05.ld read-back).  a/b: row-major [128][128] bf16; d: [128][128] fp32.
 * a_mn / b_mn = 1 uses the stored matrix transposed (MN-major operand).  use_tma = 1 stages A
 * and B with cp.async.bulk.tensor instead of cp.async.  status: int32[1].
 * No counterpart in the reference (its kernels use warp-level mma.sync). */
int fmsa_umma_selftest(const void* a, const void* b, float* d, int a_mn, int b_mn, int use_tma, int* status,
                       void* stream);

/* Test hook for the staging and operand forms that only the attention kernels use: the A tile is
 * gathered row by row with TMA (tile::gather4; row ids outside [0, src_rows) read as zeros), D1 = A_g B^T;
 * bf16(D1/16) goes back into TMEM with tcgen05.st as a packed A operand and feeds D2 = A2 * B (B used
 * MN-major); the same bf16 rows leave through a swizzled staging tile and TMA tile stores into
 * part[slot][1][:] of a [128][2][128] bf16 buffer.
 *   src bf16 [src_rows][128];  rows int32[128];  b bf16 [128][128];  d1, d2 fp32 [128][128];  status int32[1].
 * withhold = 1 leaves out the completion signal of the second product: the wait for it, bounded by
 * limit_ns, runs out, status becomes 1 and the kernel returns normally (how the tests reach the
 * timeout path).  No counterpart in the reference. */
int fmsa_pipeline_selftest(const void* src, int64_t src_rows, const int32_t* rows, const void* b, float* d1, float* d2,
                           void* part, int withhold, int64_t limit_ns, int* status, void* stream);

/* Per-row top-k over materialised block scores.
 * Replaces the running top-k of the reference select kernel
 * (flash_msa/msa_select_cutedsl.py:310-329, 370-392): total order (score descending, block
 * index ascending), the row's own block forced first, slots without a causally valid block set
 * to the sentinel NB.
 *   block_scores  fp32 [rows_bh, S, NB]   (rows_bh = B*Hp; entries with block > q/128 are ignored)
 *   block_indices int32 [rows_bh, S, Kb]
 * Kb <= FMSA_MAX_TOPK_BLOCKS. */
int fmsa_select_topk(const float* block_scores, int32_t* block_indices, int64_t rows_bh, int32_t S,
                     int32_t top_k_blocks, void* stream);

/* Deterministic reverse index (CSR) of the selection.
 * Replaces build_reverse_index_cuda / build_sparse_attention_metadata_cuda
 * (flash_msa/reverse_index_cuda.py:139-270; flash_msa/csrc/reverse_index_cuda.cu:19-233):
 * an entry (q, slot) is an edge iff 0 <= kb < NB and kb <= q/128 (reverse_index_cuda.cu:41).
 *   row_ptr  int32 [rows_bh*NB + 1]   CSR row (bp*NB + kb) lists the queries that chose kb
 *   col_q    int32 [rows_bh*S*Kb]     query positions, ascending inside a row; first row_ptr[last] used
 *   edge_pos int32 [rows_bh, S, Kb]   CSR position of each slot, -1 when the slot is not an edge
 * Unlike the reference no host synchronisation happens and the order inside a row is fixed. */
size_t fmsa_reverse_index_workspace_bytes(int64_t rows_bh, int32_t S);
int fmsa_reverse_index(const int32_t* block_indices, int32_t* row_ptr, int32_t* col_q, int32_t* edge_pos,
                       int64_t rows_bh, int32_t S, int32_t top_k_blocks, void* workspace, size_t workspace_bytes,
                       void* stream);

/* Reverse index for callers that cannot hand the library any device memory of their own.
 * (No counterpart in the reference, whose wrappers allocate their workspaces with torch.)
 * Some hosts own nothing but the input and output tensors: a thin FFI binding without a device
 * allocator, or a runtime whose memory plan is frozen before the step runs, so that neither it nor
 * this library may call cudaMalloc.  For them the scratch of fmsa_reverse_index is a fixed array of
 * FMSA_STATIC_SCRATCH_BYTES inside the library image (each GPU that loads the library keeps it
 * until the process ends).  Same inputs, outputs and results as fmsa_reverse_index.
 *  - Problems whose scratch need (fmsa_reverse_index_workspace_bytes) exceeds
 *    FMSA_STATIC_SCRATCH_BYTES are refused with FMSA_ERR_WORKSPACE; nothing is launched.
 *  - The call allocates and frees nothing.  Its first call on a device looks the array's device
 *    address up once (cudaGetSymbolAddress, with that device current) and keeps it; make that first call
 *    before any stream capture begins.  The kept address does not survive cudaDeviceReset: a process that
 *    resets a device must not call this entry point on it afterwards.
 *  - All calls on a device share the one array: two calls whose kernels may overlap on the GPU
 *    (different streams without an ordering) race and give wrong results.  Calls ordered on one
 *    stream are safe; nothing needs clearing between them. */
#define FMSA_STATIC_SCRATCH_BYTES (8 << 20)
int fmsa_reverse_index_static(const int32_t* block_indices, int32_t* row_ptr, int32_t* col_q, int32_t* edge_pos,
                              int64_t rows_bh, int32_t S, int32_t top_k_blocks, void* stream);

/* Proxy block scores: block_scores[b,p,q,j] = max over the causally visible keys k of block j of
 * scale * Qp[b,p,q] . Kp[b,p/pg,k], fp32, for every j <= q/128 (entries with j > q/128 are not
 * written).  Replaces the scoring half of the reference select kernel
 * (flash_msa/msa_select_cutedsl.py:149-306) and follows the eager definition
 * (flash_msa/tests/testing_model.py:75-88); scores are NOT rounded to bf16.
 *   q_proxy (B,Hp,S,128), k_proxy (B,Hpkv,S,128) bf16;  block_scores fp32 [B,Hp,S,S/128];  status int32[1]. */
int fmsa_select_scores(const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, float* block_scores, int32_t B,
                       int32_t Hp, int32_t Hpkv, int32_t S, float scale, int32_t dtype, const int32_t* doc_start,
                       int32_t* status, void* stream);

/* Scores and top-k in one kernel, for top_k_blocks <= FMSA_FUSED_SELECT_MAX_BLOCKS: the thread that owns a query row
 * keeps the row's best blocks in registers while the block scores come out of the tensor core, and writes
 * block_indices [B,Hp,S,top_k_blocks] (int32) itself; the fp32 block scores are never materialised.  Same result,
 * bit for bit, as fmsa_select_scores followed by fmsa_select_topk; larger top_k_blocks return FMSA_ERR_UNSUPPORTED.
 * Replaces the whole reference select kernel (flash_msa/msa_select_cutedsl.py:149-329, 481-538). */
#define FMSA_FUSED_SELECT_MAX_BLOCKS 64
int fmsa_select_fused(const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, int32_t* block_indices, int32_t B, int32_t Hp,
                      int32_t Hpkv, int32_t S, int32_t top_k_blocks, float scale, int32_t dtype, const int32_t* doc_start,
                      int32_t* status, void* stream);

/* Sparse forward, stage 1: per-edge partial attention (key-block stationary).
 * Replaces sparse_flash_varlen_forward (flash_msa/sparse_flash_varlen.py:92-261: local-block
 * FlashAttention call + chunked paged-varlen calls + torch gathers) and, with with_proxy = 1, the
 * second pass of the same machinery that the reference runs for the proxy log-sum-exp
 * (flash_msa/msa_select_cutedsl.py:541-581).
 * Work is restricted to the (batch, KV head) groups g_begin .. g_begin+g_count-1 (g = b*Hkv + kvh)
 * so that the partial buffers can be bounded: fmsa_fwd_partial_slots() gives the number of edge
 * slots the pass needs;
 *   o_part   bf16 [slots, Hq/Hp, 128]   unnormalised partial rows (sum over the block of exp(s - max) * V)
 *   lse_part fp32 [slots, Hq/Hp + 1, 2] per partial row: (row max in the log2 domain, row sum)
 * dense = 1 ignores row_ptr/col_q and runs every causal (query block, key block) pair: the warmup
 * forward (flash_msa/warmup/msa_forward_cutedsl_warmup.py:22-67).
 * counter: int32[1] scratch (reset by the call);  status: int32[1]. */
int64_t fmsa_fwd_partial_slots(const fmsa_problem* pb, int32_t g_count, int32_t dense);
int fmsa_sparse_fwd(const fmsa_problem* pb, const fmsa_tensor* q, const fmsa_tensor* k, const fmsa_tensor* v,
                    const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, const int32_t* row_ptr,
                    const int32_t* col_q, void* o_part, float* lse_part, int64_t part_slots, int32_t g_begin,
                    int32_t g_count, int32_t with_proxy, int32_t dense, int32_t* counter, int32_t* status, void* stream);

/* Sparse forward, stage 2: merge the partials of each query row (the job of the reference's
 * merge_attention_chunk / merge_lse_chunk kernels, flash_msa/csrc/reverse_index_cuda.cu:235-354).
 *   out bf16 [B, S, Hq*128]   lse fp32 [B, Hq, S]   lse_proxy fp32 [B, Hp, S] or NULL
 * Two launches for Hq/Hp <= 8 (the rows' log-sum-exp from the statistics, then the weighted sum of the partial rows,
 * which reads lse back), one otherwise. */
int fmsa_sparse_fwd_combine(const fmsa_problem* pb, const void* o_part, const float* lse_part,
                            const int32_t* edge_pos, const int32_t* row_ptr, void* out, float* lse, float* lse_proxy,
                            int32_t g_begin, int32_t g_count, int32_t dense, void* stream);

/* delta[b,h,q] = sum_d out[b,q,h,d] * d_out[b,q,h,d], fp32 [B,Hq,S].
 * Replaces the torch expression at flash_msa/flash_msa.py:99.  out is the contiguous
 * [B,S,Hq*128] forward output; d_out is described as a (B,Hq,S,128) view. */
int fmsa_bwd_delta(const void* out, const fmsa_tensor* d_out, float* delta, int32_t B, int32_t S, int32_t Hq,
                   int32_t dtype, void* stream);

/* Fused backward over the selected edges (dense = 1: over every causal block pair, the warmup
 * backward).  Replaces run_fused_backward (flash_msa/msa_backward_cutedsl.py:944-1114) and
 * run_warmup_backward (flash_msa/warmup/msa_backward_cutedsl_warmup.py:117-191).
 * Restricted, like fmsa_sparse_fwd, to the (batch, KV head) groups g_begin .. g_begin+g_count-1.
 *   d_out      (B,Hq,S,128) view of the upstream gradient
 *   lse, delta fp32 [B,Hq,S];  lse_proxy fp32 [B,Hp,S]
 *   dq_part    bf16 [slots, Hq/Hp, 128], dqp_part bf16 [slots, 128]: per-edge contributions to dQ and
 *              dQp (part_slots = slots >= fmsa_fwd_partial_slots); fmsa_sparse_bwd_combine sums them per row.
 *              Both are unscaled; the combine applies scale and scale/(B*Hp*S).
 *   split      0: one bf16 value per element, as above.  1: both buffers hold TWO planes of part_slots slots
 *              (so twice the size): plane 0 the contribution rounded to bf16, plane 1 the remainder of that
 *              rounding, and the combine adds both.  The sum over the edges of a row then keeps fp32-like
 *              accuracy however many blocks a row selects (the reference accumulates in fp32 atomics,
 *              flash_msa/msa_backward_cutedsl.py:738-836); use it when a row has more than ~32 edges.
 *   dkp_acc fp32 [B,Hpkv,S,128], dk_acc, dv_acc fp32 [B,Hkv,S,128]: ZEROED by the caller,
 *              accumulated with atomics (long reverse-index rows are split over several CTAs),
 *              unscaled; cast to the activation dtype with fmsa_cast_scaled (which applies the factors).
 * with_kl = 0 skips the proxy work (the reference does the same when no gradient reaches kl_loss,
 * flash_msa/flash_msa.py:104-106) and ignores q_proxy, k_proxy, lse_proxy, dqp_part, dkp_acc, kl_value.
 * kl_value: NULL, or fp32[1] that the kernel ADDS this launch's share of the KL loss value to:
 *              sum over the launch's (batch, proxy head, row) of KL(teacher || proxy distribution), divided by
 *              B*Hp*S -- the number the reference's eager model returns as kl_loss
 *              (flash_msa/tests/testing_model.py:158-167).  The reference kernels return a zero placeholder
 *              (flash_msa/msa_forward_cutedsl.py:69); this output has no counterpart there.  The caller zeroes
 *              it before the first pass.
 * counter: int32[1] scratch;  status: int32[1]. */
int fmsa_sparse_bwd(const fmsa_problem* pb, const fmsa_tensor* q, const fmsa_tensor* k, const fmsa_tensor* v,
                    const fmsa_tensor* q_proxy, const fmsa_tensor* k_proxy, const fmsa_tensor* d_out, const float* lse,
                    const float* lse_proxy, const float* delta, const int32_t* row_ptr, const int32_t* col_q,
                    void* dq_part, void* dqp_part, int64_t part_slots, int32_t split, float* dkp_acc, float* dk_acc,
                    float* dv_acc, int32_t g_begin, int32_t g_count, int32_t with_kl, int32_t dense, float* kl_value,
                    int32_t* counter, int32_t* status, void* stream);

/* Sums the per-edge contributions of every query row:
 *   dq (B,Hq,S,128) view, written through its `ptr`;  dq_proxy (B,Hp,S,128) view (or NULL), multiplied by *grad_kl (device
 *   scalar, the upstream gradient of kl_loss: flash_msa/flash_msa.py:122-125; NULL = 1).
 * Takes the place of the reference's fp32 atomic accumulation + cast
 * (flash_msa/msa_backward_cutedsl.py:738-836, 1075-1081). */
int fmsa_sparse_bwd_combine(const fmsa_problem* pb, const void* dq_part, const void* dqp_part, int64_t part_slots,
                            int32_t split, const int32_t* edge_pos, const int32_t* row_ptr, const fmsa_tensor* dq,
                            const fmsa_tensor* dq_proxy, const float* grad_kl, int32_t g_begin, int32_t g_count,
                            int32_t dense, void* stream);

/* dst[i] = bf16 or fp16 (dtype) of (src[i] * const_scale * f), f = *scale_ptr (a device scalar, e.g. the upstream
 * gradient of kl_loss: flash_msa/flash_msa.py:122-125) or 1 when scale_ptr is NULL.  n % 4 == 0.
 * Replaces the fp32 -> input-dtype casts at flash_msa/msa_backward_cutedsl.py:1075-1081.
 * fmsa_sparse_bwd leaves these factors to the cast: dv_acc needs 1, dk_acc needs scale, dkp_acc
 * needs scale/(B*Hp*S) times the upstream kl gradient. */
int fmsa_cast_scaled(const float* src, void* dst, int64_t n, const float* scale_ptr, float const_scale, int32_t dtype,
                     void* stream);
/* The same cast from a contiguous fp32 [B,H,S,128] accumulator into a (B,H,S,128) VIEW given by element strides, so
 * that dK, dV and dKp can be written straight into (B,S,H,128) storage, the layout the reference's callers hold
 * their activations in (flash_msa/tests/testing_model.py:173-185): no transposing copy after the backward. */
int fmsa_cast_scaled_rows(const float* src, const fmsa_tensor* dst, int32_t B, int32_t H, int32_t S,
                          const float* scale_ptr, float const_scale, int32_t dtype, void* stream);

/* Asynchronous strided copy between pinned host memory and the device (either direction; inferred
 * from the pointers): `rows` pieces of `width` bytes, source pieces `src_pitch` bytes apart, destination
 * pieces `dst_pitch` bytes apart.  No counterpart in the reference, whose API takes device tensors only:
 * it serves the host-buffer pipeline (flash_msa_b200/host.py), which moves one (batch, head range)
 * chunk of a [B,S,H*128] host tensor at a time while the previous chunk computes. */
int fmsa_copy2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width, size_t rows,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASH_MSA_B200_H */
