/* speed3r_b200_check.h - C ABI of libspeed3r_b200_check.so, a TESTS-ONLY companion of libspeed3r_b200.so.
 *
 * Nothing in the product path links, loads or calls this library.  It holds
 *   - plain SIMT restatements of the two forward attentions (one thread per query row, fp32
 *     arithmetic), so that the tensor-core kernels can be cross-checked ON THE DEVICE at sizes a
 *     CPU check cannot reach;
 *   - a probe of the bounded device-side wait every kernel of the product library uses.
 * Conventions (return codes, s3r_last_error, explicit stream) are those of speed3r_b200.h; the
 * library carries its own copy of the per-device status word, read with its own s3r_device_status.
 */
#ifndef SPEED3R_B200_CHECK_H_
#define SPEED3R_B200_CHECK_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same arguments and semantics as s3r_cmp_attn_topk_fwd / s3r_sel_attn_fwd (o_s, lse_s only) of
 * speed3r_b200.h, i.e. restatements of flash_attention_topk.py:22-152 and
 * topk_blocksparse_attention.py:35-128 of the reference. */
int s3r_check_cmp_attn_topk_fwd(const void* q_c, const void* k_c, const void* v_c, void* o_c, float* lse,
                                int32_t* idx, int B, int H, int Nq, int Nc, int d, int topk, float scale,
                                void* stream);
int s3r_check_sel_attn_fwd(const void* q, const void* k, const void* v, const int32_t* idx, void* o_s,
                           float* lse_s, int B, int H, int Tq, int Tk, int d, int block, int topk, float scale,
                           void* stream);

/* Launches one warp that waits, with the library's bounded wait and a limit of `limit_ns`
 * nanoseconds, on a barrier that nothing ever arrives on.  The wait must give up: the kernel then
 * returns normally, writes the nanoseconds it waited to *waited_ns (device memory, 8 bytes) and
 * raises S3R_STATUS_WAIT_TIMEOUT in this library's status word.  No counterpart in the reference
 * (which has no device-side waits); it exists so that the give-up path is exercised without
 * leaving anything waiting on the GPU. */
int s3r_check_wait_gives_up(uint64_t limit_ns, uint64_t* waited_ns, void* stream);

/* This library's copies of the two helpers of speed3r_b200.h. */
int s3r_last_error(char* buf, int n);
int s3r_device_status(uint32_t* status_host, int clear);

#ifdef __cplusplus
}
#endif
#endif /* SPEED3R_B200_CHECK_H_ */
