/* C ABI of the DSA top-k indexer (definition dsa_topk_indexer_fp8_h64_d128_topk2048_ps64), the sibling operator of
 * the MoE layer in the same shared library (libsyfi_moe.so).
 *
 * Replaces the reference's entry points for that definition: the configured one,
 * dsa_indexer/solution/python/dsa_topk_indexer.py::run (:64-112, pure torch), and the CUDA one,
 * run_dsa_topk_indexer (dsa_indexer/solution/cuda/dsa_topk_indexer.cu:468-557, exported at :557).
 * Same tensors, same order, destination-passing (dsa_indexer/config.toml:10); plain device pointers and sizes. */
#ifndef SYFI_DSA_H_
#define SYFI_DSA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SYFI_DSA_OK 0
#define SYFI_DSA_ERR_INVALID 1   /* bad argument */
#define SYFI_DSA_ERR_CUDA 2      /* a CUDA call failed, no CUDA device, or not an sm_100 device */
#define SYFI_DSA_ERR_DEVICE 3    /* a kernel gave up on a bounded wait (syfi_dsa_check) */
#define SYFI_DSA_TOPK 2048

/* For every sequence b of the batch: score[t] = sum_h weights[b, h] * relu(q[b, h, :] . key[t, :]) over the
 * sequence's tokens, key[t] = the token's 128 e4m3 values times its f32 scale; writes the cache token ids
 * (page * 64 + offset) of the 2048 best tokens, best first (ties by position in the sequence), -1 beyond the
 * sequence's length.  All pointers are DEVICE pointers, 16-byte aligned:
 *   q_index_fp8        e4m3 [batch, 64, 128]
 *   k_index_cache_fp8  bytes [num_pages, 64, 1, 132]: per page 64 x 128 e4m3 bytes, then 64 f32 scales
 *                      (dsa_topk_indexer.py:38-58)
 *   weights            f32 [batch, 64]
 *   seq_lens           int32 [batch]
 *   block_table        int32 [batch, max_pages]: cache page of every 64 tokens of a sequence
 *   topk_indices       int32 [batch, 2048] (output)
 * Work is enqueued on `stream` (a cudaStream_t) of the CURRENT device; the call does not synchronise.  A scratch
 * buffer of batch * max_pages * 64 floats per device is kept by the library and grows on demand.  Returns
 * SYFI_DSA_OK or an error code; syfi_moe_last_error() (syfi_moe.h) has the message.  The reference checks nothing
 * (dsa_topk_indexer.cu:476-494). */
int syfi_dsa_topk_indexer(const void* q_index_fp8, const void* k_index_cache_fp8, const float* weights,
                          const int32_t* seq_lens, const int32_t* block_table, int32_t batch, int64_t num_pages,
                          int32_t max_pages, int32_t* topk_indices, void* stream);

/* Synchronises `stream` and reports whether a kernel of this operator gave up on a bounded wait on the current
 * device since the last check (status 201). */
int syfi_dsa_check(void* stream);

#ifdef __cplusplus
}
#endif

#endif  /* SYFI_DSA_H_ */
