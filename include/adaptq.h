/*
 * adaptq.h -- C ABI of the B200 (sm_100a) AdapTQ engine.
 *
 * Symbol-for-symbol replacement for the C interface that the upstream CPU
 * library declares in include/adaptq.h and implements in
 * core/adaptq_c_api.cpp; a program linked against upstream's libadaptq can be
 * relinked against libadaptq_b200.so unchanged.  Each declaration names the
 * upstream line it replaces as  [h:<line in include/adaptq.h>
 * c:<line in core/adaptq_c_api.cpp>].
 *
 * What is the same: argument meaning, return values (handle or NULL, token
 * count or -1), the per-thread error string and its exact texts, the
 * per-head seed rule of the multi-head handle, ring-buffer (FIFO) eviction,
 * the hybrid FP32 window, sparse-V, K/V FP32 passthrough (bits == 16).
 *
 * What differs: the cache lives in GPU memory and every call runs CUDA
 * kernels; there is no CPU path.  `key`, `val`, `query`, `out` may be host
 * pointers (staged through a copy, as upstream callers pass them) or device
 * pointers (used in place).  Calls on one handle are ordered on that
 * handle's CUDA stream; calls that return data to a host pointer return
 * after the data has arrived.  Construction failures that upstream lets
 * escape as C++ exceptions (padded dimension above 1024, allocation
 * failure) come back as NULL with the error string set.
 *
 * The batched entry points that reach HBM bandwidth are in adaptq_b200.h.
 */
#ifndef ADAPTQ_B200_ADAPTQ_H
#define ADAPTQ_B200_ADAPTQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error classes [h:17-23].  As upstream, no function returns them; they
 * classify what adaptq_last_error() describes. */
typedef enum {
  ADAPTQ_OK = 0,
  ADAPTQ_ERR_ALLOC = 1,
  ADAPTQ_ERR_INVALID_ARG = 2,
  ADAPTQ_ERR_OUT_OF_BOUNDS = 3,
  ADAPTQ_ERR_UNSUPPORTED = 4
} adaptq_error_t;

/* Text of the last error raised on the calling thread, "" if none
 * [h:30 c:21]. */
const char *adaptq_last_error(void);

typedef void *adaptq_ctx_t; /* one head    [h:32] */
typedef void *adaptq_mha_t; /* many heads  [h:33] */

/* ---- one head ---------------------------------------------------------- */

/* [h:47 c:63]  dim > 0; k_bits, v_bits in {2,3,4,16}; capacity >= 0 tokens
 * (ring size); seed = Rademacher seed; v_mass <= 0 accumulates every V row,
 * v_mass > 0 only the heaviest rows until that softmax mass is covered;
 * hybrid_thresh > 0 keeps an FP32 copy of the first hybrid_thresh tokens and
 * answers from it while the cache holds no more than that.  NULL on bad
 * arguments ("adaptq_create: invalid dimensions or capacity"). */
adaptq_ctx_t adaptq_create(int dim, int k_bits, int v_bits, int capacity,
                           uint64_t seed, float v_mass, int hybrid_thresh);

/* [h:51 c:76]  NULL is a no-op. */
void adaptq_destroy(adaptq_ctx_t ctx);

/* [h:54 c:82]  key, val: float[dim]. */
void adaptq_append(adaptq_ctx_t ctx, const float *key, const float *val,
                   int token_pos);

/* [h:64 c:96]  query, out: float[dim].  Returns tokens attended (0 = empty
 * cache, out zeroed), -1 on a NULL argument. */
int adaptq_compute(adaptq_ctx_t ctx, const float *query, float *out);

/* [h:75 c:109]  queries, outs: float[num_queries*dim].  One launch serves all
 * queries; the cache comes from HBM once (re-reads are served by L2). */
int adaptq_compute_batch(adaptq_ctx_t ctx, const float *queries,
                         int num_queries, float *outs);

/* [h:79 c:128]  Forget all tokens, keep the configuration. */
void adaptq_reset(adaptq_ctx_t ctx);

/* [h:82 c:139]  tokens * (K row bytes + V row bytes); scales not counted. */
size_t adaptq_kv_bytes(adaptq_ctx_t ctx);

/* ---- many heads -------------------------------------------------------- */

/* [h:91 c:149]  Head i uses seed  base_seed ^ (i * 0xDEADBEEFCAFE)  [c:160].
 * NULL on bad arguments ("adaptq_mha_create: invalid parameters"). */
adaptq_mha_t adaptq_mha_create(int n_heads, int dim, int k_bits, int v_bits,
                               int capacity, uint64_t base_seed, float v_mass,
                               int hybrid_thresh);

void adaptq_mha_destroy(adaptq_mha_t mha); /* [h:95 c:167] */

/* [h:98 c:177]  0 <= head_idx < n_heads, else "...: head_idx out of range". */
void adaptq_mha_append(adaptq_mha_t mha, int head_idx, const float *key,
                       const float *val, int token_pos);

int adaptq_mha_compute(adaptq_mha_t mha, int head_idx, const float *query,
                       float *out); /* [h:102 c:197] */

int adaptq_mha_compute_batch(adaptq_mha_t mha, int head_idx,
                             const float *queries, int num_queries,
                             float *outs); /* [h:106 c:217] */

void adaptq_mha_reset(adaptq_mha_t mha);            /* [h:111 c:243] */
size_t adaptq_mha_total_kv_bytes(adaptq_mha_t mha); /* [h:114 c:252] */

/* ---- identity ---------------------------------------------------------- */

#define ADAPTQ_FEAT_AVX2 (1u << 0)     /* never set by this library */
#define ADAPTQ_FEAT_HYBRID (1u << 1)
#define ADAPTQ_FEAT_SPARSE_V (1u << 2)
#define ADAPTQ_FEAT_CUDA_SM100 (1u << 8) /* addition: always set here */

unsigned int adaptq_features(void); /* [h:123 c:267] */
const char *adaptq_version(void);   /* [h:126 c:275]  "<x.y.z>-sm100a" */

#ifdef __cplusplus
}
#endif
#endif /* ADAPTQ_B200_ADAPTQ_H */
