/*
 * adaptq_runtime.h -- C ABI over the device implementation of upstream's
 * second stack, the "V2" plugin runtime: adaptq::RuntimeContext with its
 * default HARFixedStrategy + ContiguousSlabStorage (runtime/runtime_context.h,
 * strategies/har_fixed.cpp, storage/contiguous_slab.h), the compute primitives
 * of adaptq::IKernelBackend (include/adaptq/kernel.h), and session snapshots in
 * the AQSS v2 file format (replay/session_snapshot.h, .cpp).
 *
 * It is the same arithmetic as the AttentionHead path of adaptq.h -- one
 * Quantizer per (layer, head), a single bit width for keys and values, FIFO
 * ring -- so every function below runs on the same CUDA kernels.  Differences
 * that upstream's stack has and that are kept:
 *   - head seeds are layer * 65537 + head      (runtime_context.cpp:128);
 *   - no FP32 window;
 *   - sparse V (v_mass > 0) adds rows one at a time until the mass is reached,
 *     not in blocks of four                    (har_fixed.cpp:258-264).
 *
 * Pointers may be host or device memory unless stated.  Functions return -1
 * (or NULL) and set adaptq_last_error() on failure; nothing throws.
 */
#ifndef ADAPTQ_RUNTIME_H
#define ADAPTQ_RUNTIME_H

#include "adaptq.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void *adaptq_runtime_t;

/* RuntimeContext::init(cfg) with the default factories
 * (runtime/runtime_context.cpp:85-152): n_layers x n_heads independent caches
 * of `capacity` tokens, `bits` in {2,3,4} for keys and values. */
adaptq_runtime_t adaptq_runtime_create(int n_layers, int n_heads, int dim,
                                       int bits, int capacity, float v_mass);
void adaptq_runtime_destroy(adaptq_runtime_t rt);

/* RuntimeContext::append (runtime_context.cpp:229-288): one K/V pair for
 * (layer, head).  The token position advances after the last head of the last
 * layer, as upstream's does.  Returns 0. */
int adaptq_runtime_append(adaptq_runtime_t rt, int layer, int head,
                          const float *k_vec, const float *v_vec);

/* RuntimeContext::compute (runtime_context.cpp:294-444), quantized branch =
 * HARFixedStrategy::compute_full (har_fixed.cpp:197-289).  out: float[dim].
 * Returns the number of cached tokens used (upstream's
 * ComputeMetrics::n_tokens_used); zeros and 0 for an empty cache. */
int adaptq_runtime_compute(adaptq_runtime_t rt, int layer, int head,
                           const float *q_vec, float *out);

/* The same for every (layer, head) in one call -- additions, no counterpart
 * upstream.  k, v, q, out: float [n_layers][n_heads][dim].  append_token
 * equals the double loop over adaptq_runtime_append in layer-major order. */
int adaptq_runtime_append_token(adaptq_runtime_t rt, const float *k,
                                const float *v);
int adaptq_runtime_compute_token(adaptq_runtime_t rt, const float *q,
                                 float *out);

/* RuntimeContext::reset / token_pos / n_layers ... (runtime_context.h) */
int adaptq_runtime_reset(adaptq_runtime_t rt);
int adaptq_runtime_token_pos(adaptq_runtime_t rt);
/* The multi-head handle underneath ((layer, head) is head layer*n_heads+head):
 * for adaptq_mha_info / adaptq_mha_export_head / adaptq_mha_synchronize.
 * Owned by the runtime; do not destroy it. */
adaptq_mha_t adaptq_runtime_handle(adaptq_runtime_t rt);

/* SessionSnapshot::capture + save (replay/session_snapshot.cpp:108-268): the
 * device cache of every head written as an AQSS v2 file -- 40-byte header,
 * then per head {layer, head, cache_size, slot_bytes, storage data (K rows of
 * the live slots, then V rows, each padded to slot_bytes =
 * max(packed row, dim*4) as upstream sizes its slots, runtime_context.cpp:
 * 113-116), scales (K then V), format tags (= bits, har_fixed.cpp:40-50)},
 * then the strategy-state blobs upstream's HARReplayHooks write (one uint32 1
 * per head, flags bit 1).  No token log (flags bit 0 clear).  For a full cache
 * the file equals, byte for byte, what upstream writes for the same tokens. */
int adaptq_runtime_snapshot_save(adaptq_runtime_t rt, const char *path);

/* SessionSnapshot::load (replay/session_snapshot.cpp:271-400) with the same
 * validation (magic, version <= 2, sizes against the remaining file, counts),
 * then a new runtime whose device caches hold the snapshot's rows and scales.
 * capacity = 0 sizes the rings to the largest cache_size in the file.  The ring
 * position of a full cache is n_tokens mod capacity (every token reaches every
 * head once); a token log, if present, is skipped. */
adaptq_runtime_t adaptq_runtime_snapshot_load(const char *path, int capacity,
                                              float v_mass);

/* Counterpart of adaptq_mha_export_head: overwrite head `head_idx` of a
 * multi-head handle with n_rows packed rows (k_rows: n_rows x k_row_bytes,
 * v_rows likewise, upstream's row layout), their scales, and the ring state
 * (ring_head = next slot to be written, ring_size = live tokens <= n_rows).
 * The FP32 window of that head is marked invalid, as after an eviction.
 * Host pointers.  Returns 0. */
int adaptq_mha_import_head(adaptq_mha_t mha, int head_idx,
                           const uint8_t *k_rows, const uint8_t *v_rows,
                           const float *k_scale, const float *v_scale,
                           int n_rows, int ring_head, int ring_size);

/* adaptq::IKernelBackend on the device (include/adaptq/kernel.h:24-94).
 * Compressed vectors are passed as `n` rows at a fixed stride -- the layout of
 * upstream's slab storage, where CompressResult::data of slot i is
 * base + i * slot_bytes -- with their scales in a parallel array.
 *   fwht_forward / fwht_inverse : in place on n_vectors x padded floats
 *   kdot_batch   : logits_out[i] = dot(q_rot, centroids(k_row_i)) * scale_i / padded
 *                  (kernels/scalar/kdot_scalar.cpp:35-49)
 *   vaccum_batch : acc[j] = sum_i weights[i] * scale_i * centroid(v_row_i)[j]
 *                  (kdot_scalar.cpp:53-67; acc is overwritten, zero weights skipped)
 * padded: a power of two <= 1024; bits in {2,3,4}. */
int adaptq_kernel_fwht_forward(float *x, const int8_t *D, int padded, int n_vectors);
int adaptq_kernel_fwht_inverse(float *x, const int8_t *D, int padded, int n_vectors);
int adaptq_kernel_kdot_batch(const float *q_rot, const uint8_t *k_rows,
                             size_t row_stride, const float *k_scales, int n,
                             int padded, int bits, float *logits_out);
int adaptq_kernel_vaccum_batch(float *acc, const uint8_t *v_rows,
                               size_t row_stride, const float *v_scales,
                               const float *weights, int n, int padded, int bits);
/* IKernelBackend::name() */
const char *adaptq_kernel_backend_name(void);

#ifdef __cplusplus
}
#endif
#endif /* ADAPTQ_RUNTIME_H */
