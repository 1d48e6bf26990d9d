/*
 * speed3r_b200 — C ABI of the B200 (sm_100a) implementation of Speed3R's dual-branch sparse
 * global attention (the attention inside Pi3_Sparse's global decoder blocks).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its name ends in _host.  The caller owns every
 *     buffer; no entry point allocates or frees device memory unless its comment says so.
 *   - Activations are bf16 (uint16 storage); lse / delta are fp32; index tables are int32.
 *   - Tensors are dense row-major with the shape written in the comment.
 *   - `stream` is a cudaStream_t passed as void*.  Work is enqueued, never synchronised.
 *   - Return value: 0 = ok, <0 = argument error (S3R_ERR_*; message via s3r_last_error),
 *     >0 = a CUDA runtime error code from the launch.
 *   - Kernels never spin without a limit: if an internal wait runs out they set a bit in a
 *     per-device status word (s3r_device_status) and return early.
 *
 * Each entry point cites the reference interface it replaces, by path inside the reference
 * project (Visual-AI/speed3r).
 */
#ifndef SPEED3R_B200_H_
#define SPEED3R_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define S3R_OK 0
#define S3R_ERR_SHAPE (-1)       /* a size is zero, negative or inconsistent */
#define S3R_ERR_UNSUPPORTED (-2) /* head_dim / block / top-k outside what the kernels implement */
#define S3R_ERR_ALIGNMENT (-3)   /* a pointer is not 16-byte aligned */
#define S3R_ERR_NULL (-4)        /* a required pointer is NULL */
#define S3R_ERR_DRIVER (-5)      /* tensor-map creation through the driver failed */
#define S3R_ERR_TOO_LARGE (-6)   /* exceeds the capacity of a fixed-size buffer */

#define S3R_STATUS_WAIT_TIMEOUT 1u /* a bounded device-side wait gave up */
#define S3R_STATUS_BAD_INDEX 2u    /* s3r_qkv_prologue_fwd met a position outside its cos/sin tables (row clamped) */

/* Library version (major*10000 + minor*100 + patch). */
int s3r_version(void);

/* Copies the calling thread's last error message (NUL-terminated) into buf; returns its length. */
int s3r_last_error(char* buf, int n);

/* Reads (and clears when `clear` != 0) the status word of the current device.  Synchronises
 * the device.  0 means no kernel reported a problem. */
int s3r_device_status(uint32_t* status_host, int clear);

/* ------------------------------------------------------------------------------------------
 * Compression (block pooling).
 * Replaces the rearrange + F.avg_pool1d + rearrange + unbind of
 * pi3/models/layers/sparse_attention.py:97-102 for ONE of q/k/v (call three times).
 *
 *   in  : element (b, h, t, c) at  in + b*stride_b + h*stride_h + t*stride_t + c   (elements)
 *         — the packed qkv projection [B,T,3,H,d] is read in place with
 *           stride_b = T*3*H*d, stride_h = d, stride_t = 3*H*d and base = qkv + {0,1,2}*H*d
 *   out : [B,H,Nc,d] with Nc = floor((T-kernel)/stride)+1 ; out[j] = mean(in[j*stride : j*stride+kernel])
 * The mean is accumulated in fp32 and rounded once to bf16.
 * ------------------------------------------------------------------------------------------ */
int s3r_pool_fwd(const void* in, int64_t stride_b, int64_t stride_h, int64_t stride_t,
                 void* out, int B, int H, int T, int d, int kernel, int stride, void* stream);

/* Backward of s3r_pool_fwd (autograd of F.avg_pool1d, same lines):
 *   d_out [B,H,Nc,d];  d_in element (b,h,t,c) at d_in + b*stride_b + h*stride_h + t*stride_t + c
 *   d_in[b,h,t,:] = sum over windows j containing t of d_out[b,h,j,:] / kernel.
 * When `accumulate` is non-zero the result is added to d_in (fp32 add, one rounding) instead of
 * overwriting it, which folds the pooled-branch gradient into the token-branch gradient. */
int s3r_pool_bwd(const void* d_out, void* d_in, int64_t stride_b, int64_t stride_h, int64_t stride_t,
                 int B, int H, int T, int d, int kernel, int stride, int accumulate, void* stream);

/* ------------------------------------------------------------------------------------------
 * Prologue of the module in one pass over the packed projection.  Replaces the PyTorch code between
 * `qkv = self.qkv(x)` and the two attention calls of SparseFlashAttentionRope.forward
 * (pi3/models/layers/sparse_attention.py:95-123): F.avg_pool1d of the raw q,k,v, q_norm/k_norm
 * (nn.LayerNorm over the head dimension, fp32 under autocast, result rounded to bf16), the 2-D
 * rotary embedding RoPE2D (pi3/models/layers/pos_embed.py:112-159) at the token positions and at
 * the truncated mean position of every block, and the `[B,N,3,H,d] -> 3 x [B,H,N,d]` split.
 *   qkv            : [B,N,3,H,d] bf16, contiguous (the output of the qkv Linear)
 *   pos            : [B,N,2] int64 (y,x) or NULL (no rotary embedding)
 *   cos_tab/sin_tab: [tab_rows, d/2] bf16, row p = cos/sin of bf16(p * inv_freq) duplicated over the two
 *                    halves (what RoPE2D caches); a position outside the table is clamped and
 *                    raises S3R_STATUS_BAD_INDEX in the device status word
 *   q_weight..k_bias: fp32 [d] LayerNorm affine parameters, or all NULL (Identity norms)
 *   q,k,v          : [B,H,N,d] bf16 out;  q_c,k_c,v_c : [B,H,N/block,d] bf16 out
 * N must be a multiple of `block`; d = 64; at most 42 heads.  Forward only: a caller that
 * needs gradients runs the separate steps (s3r_pool_fwd/bwd and its own LayerNorm and rotary code). */
int s3r_qkv_prologue_fwd(const void* qkv, const int64_t* pos, const void* cos_tab, const void* sin_tab,
                         int tab_rows, const float* q_weight, const float* q_bias, const float* k_weight,
                         const float* k_bias, float eps, void* q, void* k, void* v, void* q_c, void* k_c,
                         void* v_c, int B, int H, int N, int d, int block, void* stream);

/* ------------------------------------------------------------------------------------------
 * Compression attention with fused top-k block selection.
 * Replaces flash_attn_topk_func / FlashAttnTopkFunc.forward / forward_with_topk /
 * _fwd_kernel_with_topk (pi3/models/sparse_attn/flash_attention_topk.py:22-200, 633-650) and
 * the key order of pi3/models/sparse_attn/topk_utils.py:19-23.
 *
 *   q_c [B,H,Nq,d], k_c / v_c [B,H,Nc,d]   (d = 64)
 *   o_c [B,H,Nq,d] bf16 = softmax(scale * q_c k_c^T) v_c          (non-causal)
 *   lse [B,H,Nq] fp32   = log-sum-exp of scale * q_c k_c^T
 *   idx [B,H,Nq,topk] int32 = columns of the `topk` largest RAW logits q_c k_c^T (fp32
 *         accumulation) of each row, ordered by (logit descending, column ascending); when
 *         Nc < topk the tail holds Nc-1, as the reference's zero-initialised running set does.
 *   Rows [q_row0, q_row0+Nq) of a longer query sequence can be processed against all Nc keys
 *   by passing q_c/o_c/lse/idx pointers of that slice (sequence-partitioned use).
 *   topk <= 32.  The running top-k sets live in shared memory; the call needs no scratch and keeps no
 *   state between calls.
 * ------------------------------------------------------------------------------------------ */
int s3r_cmp_attn_topk_fwd(const void* q_c, const void* k_c, const void* v_c, void* o_c, float* lse,
                          int32_t* idx, int B, int H, int Nq, int Nc, int d, int topk, float scale,
                          void* stream);

/* The same kernel for settings in which compressed keys are finer than selection blocks (windows of Lc
 * tokens every Sc tokens, selection blocks of Bs = group*Sc tokens).  No counterpart in the reference,
 * whose three sizes are equal.  Queries are pooled per selection block by the caller.
 *   idx [B,H,Nq,topk] = the `topk` selection BLOCKS of each row by the softmax probability mass of the
 *         block's own compressed keys, i.e. of columns group*n .. group*n+take-1 (take = (Bs-Lc)/Sc + 1
 *         windows lie inside a block), ranked through log2 sum_j 2^(scale*log2(e)*s_j) - monotone in the
 *         mass, no row normaliser needed - with the same order rules (score descending, block
 *         ascending) and the same padding (Nb-1 when fewer than topk blocks exist).  Only blocks with
 *         all `take` columns present are ranked: Nb = (Nc-take)/group + 1.
 *   group must be 4; 1 <= take <= 4.  o_c and lse as above. */
int s3r_cmp_attn_blocktopk_fwd(const void* q_c, const void* k_c, const void* v_c, void* o_c, float* lse,
                               int32_t* idx, int B, int H, int Nq, int Nc, int d, int topk, float scale,
                               int group, int take, void* stream);

/* Backward of the compression attention.  Replaces FlashAttnTopkFunc.backward /
 * _flash_attn_backward and its three kernels (flash_attention_topk.py:204-630).  No gradient
 * flows through idx (:665).
 *   delta [B,H,Nq] fp32 is scratch written by the call (sum_d o_c*do_c).
 *   dq_c [B,H,Nq,d], dk_c / dv_c [B,H,Nc,d] bf16 are overwritten. */
int s3r_cmp_attn_bwd(const void* q_c, const void* k_c, const void* v_c, const void* o_c, const float* lse,
                     const void* do_c, float* delta, void* dq_c, void* dk_c, void* dv_c, int B, int H, int Nq,
                     int Nc, int d, float scale, void* stream);

/* ------------------------------------------------------------------------------------------
 * Selection attention (block-sparse flash attention) with the gated merge fused in.
 * Replaces topk_blocksparse_attention / TopkBlockSparseAttention.forward /
 * _topk_blocksparse_attention_fwd / block_sparse_forward_kernel
 * (pi3/models/sparse_attn/topk_blocksparse_attention.py:35-128, 852-904, 1041-1121) and, when
 * `y` is given, the gate * branch merge and head-interleaving rearrange of
 * pi3/models/layers/sparse_attention.py:127-136.
 *
 *   q [B,H,Tq,d]; k, v: Tk tokens per (b,h), stored as `kv_chunks` chunks of Tk/kv_chunks tokens,
 *        chunk c at  k + c*kv_chunk_stride  (elements) holding [B,H,Tk/kv_chunks,d].  A single
 *        dense [B,H,Tk,d] tensor is kv_chunks = 1.  (An all-gather over the sequence leaves the
 *        keys in exactly this chunked form, one chunk per rank.)
 *   idx [B,H,ceil(Tq/block),topk] int32: key-block numbers; an entry n with n < 0 or
 *        n*block >= Tk is skipped; a block listed twice is counted twice.
 *   o_s [B,H,Tq,d] bf16 and lse_s [B,H,Tq] fp32: selection-branch output and log-sum-exp
 *        (either may be NULL when not needed, e.g. inference with the merge fused).
 *   Merge (all three NULL to disable):
 *        gate: element (b,h,t,g) at gate + b*gate_stride_b + h*gate_stride_h + t*gate_stride_t + g
 *              (g=0 weights the compression branch, g=1 the selection branch; already sigmoid-ed)
 *        o_c  [B,H,ceil(Tq/block),d] compression-branch output, one row per query block
 *        y    [B,Tq,H*d] bf16 = g0 * o_c[t/block] + g1 * o_s[t]
 *   block in {16,32,64}; topk <= 64; d = 64.
 * ------------------------------------------------------------------------------------------ */
int s3r_sel_attn_fwd(const void* q, const void* k, const void* v, int kv_chunks, int64_t kv_chunk_stride,
                     const int32_t* idx, void* o_s, float* lse_s,
                     const void* gate, int64_t gate_stride_b, int64_t gate_stride_h, int64_t gate_stride_t,
                     const void* o_c, void* y,
                     int B, int H, int Tq, int Tk, int d, int block, int topk, float scale, void* stream);

/* Key-centric index of the selection table, built on the device without any host
 * synchronisation.  Replaces count_query_fixedlen + reorder_topk_idx_fixedlen +
 * save_topk_idx_kernel_fixedlen (topk_blocksparse_attention.py:172-213, 368-555), including
 * their torch.argsort / cumsum / two .item() round trips.
 *   idx     [B,H,Nq,topk]
 *   offsets [B,H,Nkb+1] int32 : CSR row pointers per (b,h)
 *   qids    [B,H,Nq*topk] int32: for key block n, qids[offsets[n] : offsets[n+1]] are the query
 *           blocks that list n, ascending (a query block listing n twice appears twice);
 *           entries of idx outside [0,Nkb) are dropped.
 *   workspace: s3r_csr_workspace_bytes(...) bytes of scratch, 256-byte aligned (per-key-block
 *           cursors and an unsorted copy of qids); contents need not be initialised. */
size_t s3r_csr_workspace_bytes(int B, int H, int Nq, int topk, int Nkb);
int s3r_build_key_csr(const int32_t* idx, int32_t* offsets, int32_t* qids, int B, int H, int Nq, int topk,
                      int Nkb, void* workspace, size_t workspace_bytes, void* stream);

/* The same index build with NO caller-provided workspace and no allocation of any kind.
 * It has no counterpart in the reference.  It is for hosts that cannot allocate device memory
 * when the call is made (all memory was handed to another runtime up front, or a cudaMalloc, which
 * synchronises the device, is not acceptable where the call sits).  The scratch is a fixed buffer
 * of S3R_CSR_STATIC_SCRATCH_BYTES inside the library image; every GPU that loads the library
 * holds it until the process exits.
 *   - Same arguments, outputs and ordering guarantees as s3r_build_key_csr.
 *   - Tables whose scratch (s3r_csr_workspace_bytes) exceeds the buffer are refused with
 *     S3R_ERR_TOO_LARGE and a message; nothing is launched.
 *   - The first call on each device resolves the buffer's device address (cudaGetSymbolAddress
 *     with that device current); under lazy module loading that may load the library's device
 *     code then, which synchronises.  Make that first call during set-up.  The address is cached
 *     per device ordinal and is valid for the life of that device's primary context.
 *   - The buffer is 256-byte aligned, as the workspace of s3r_build_key_csr has to be.
 *   - All calls on a device share the one buffer, which keeps whatever the previous call left; the
 *     kernels overwrite every slot they later read, so nothing needs clearing.  Two calls that
 *     overlap on the GPU (different streams) race on it: serialise them.
 *   - Calls cudaMemsetAsync on `offsets` and launches kernels; no cudaMalloc/cudaFree. */
#define S3R_CSR_STATIC_SCRATCH_BYTES (8u << 20)
int s3r_build_key_csr_static(const int32_t* idx, int32_t* offsets, int32_t* qids, int B, int H, int Nq,
                             int topk, int Nkb, void* stream);

/* Backward of the gated merge (autograd of sparse_attention.py:127-136), producing what the
 * selection backward needs in one pass over dy:
 *   dy [B,Tq,H*d] ; gate / o_c / o_s as in the forward
 *   do_s  [B,H,Tq,d] bf16 = g1 * dy
 *   dgate [B,H,Tq,2] fp32 : dg0 = sum_d dy*o_c[t/block], dg1 = sum_d dy*o_s
 *   do_c  [B,H,ceil(Tq/block),d] bf16 = sum over the block's tokens of g0 * dy
 *   delta_s [B,H,Tq] fp32 = sum_d o_s*do_s = g1*dg1 */
int s3r_merge_bwd(const void* dy, const void* gate, int64_t gate_stride_b, int64_t gate_stride_h,
                  int64_t gate_stride_t, const void* o_c, const void* o_s, void* do_s, float* dgate,
                  void* do_c, float* delta_s, int B, int H, int Tq, int d, int block, void* stream);

/* Row-wise delta = sum_d o*do for [rows,d] bf16 tensors (backward_sum_o_do,
 * topk_blocksparse_attention.py:132-170); used when the merge is not fused. */
int s3r_delta(const void* o, const void* d_o, float* delta, int64_t rows, int d, void* stream);

/* Backward of the selection attention.  Replaces TopkBlockSparseAttention.backward /
 * _topk_blocksparse_attention_bwd and the kernels backward_dkdv / backward_dq
 * (topk_blocksparse_attention.py:557-849, 907-1038).
 *   q,k,v,idx as in the forward (kv_chunks = 1 only); lse_s, delta_s [B,H,Tq] fp32; do_s [B,H,Tq,d]
 *   offsets/qids from s3r_build_key_csr
 *   dq [B,H,Tq,d], dk / dv [B,H,Tk,d] bf16, overwritten (key blocks nobody selected get zeros).
 * Entries of idx that the forward skips are skipped here too (the reference's dq kernel reads out
 * of bounds for negative entries, :804-807). */
int s3r_sel_attn_bwd(const void* q, const void* k, const void* v, const int32_t* idx, const int32_t* offsets,
                     const int32_t* qids, const float* lse_s, const float* delta_s, const void* do_s,
                     void* dq, void* dk, void* dv, int B, int H, int Tq, int Tk, int d, int block, int topk,
                     float scale, void* stream);

/* ------------------------------------------------------------------------------------------
 * Multi-GPU helper of the sequence-partitioned op (the reference is single-GPU: no counterpart).
 * Copies `nseg` (<= 16) segments src[s] -> dst[s] of bytes[s] bytes (multiples of 16, 16-byte aligned)
 * with one kernel of `ctas` CTAs.  The sources are meant to be PEER memory mapped into this process
 * (CUDA IPC); they are only read, with plain loads.  A small `ctas` (16..32) keeps the copy on a few
 * SMs so that it can run beside a kernel that fills all the others.
 * ------------------------------------------------------------------------------------------ */
int s3r_peer_pull(const void* const* src, void* const* dst, const int64_t* bytes, int nseg, int ctas, void* stream);

/* Strided copy between host and device (rows of `width_bytes` at the two pitches) on `stream`:
 * cudaMemcpy2DAsync with the direction inferred from the pointers.  No counterpart in the reference;
 * the pinned-host pipeline uses it to place one head group's columns of y [B,T,H*d] in the caller's
 * buffer (PyTorch stages such a copy through pageable memory and blocks). */
int s3r_copy2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                     size_t rows, void* stream);

/* CUDA IPC for those sources.  s3r_ipc_export: the 64-byte handle of the allocation that holds `ptr` and
 * `ptr`'s offset in it (the owner keeps the buffer alive).  s3r_ipc_import: opens such a handle in another
 * process of the same node WITH THE IMPORTER'S DEVICE CURRENT (lazy peer access), so that kernels of that
 * device may dereference the returned address; the mapping lasts until the process exits. */
int s3r_ipc_export(const void* ptr, void* handle64, int64_t* offset);
int s3r_ipc_import(const void* handle64, int64_t offset, void** ptr);

#ifdef __cplusplus
}
#endif
#endif /* SPEED3R_B200_H_ */
