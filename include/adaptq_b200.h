/*
 * adaptq_b200.h -- batched entry points of the B200 AdapTQ engine.
 *
 * The upstream interface (adaptq.h) moves one float[dim] vector of one head
 * per call; upstream's own callers loop over heads in Python
 * (adaptq/core.py:53-57, :70-72).  That shape cannot keep a GPU busy, so the
 * same two operations are also offered over ALL heads of a handle at once.
 * They are additions: upstream has no counterpart, and they compute exactly
 * what a loop over adaptq_mha_append / adaptq_mha_compute(_batch) computes.
 *
 * Pointers may be host or device memory (the library asks the CUDA runtime
 * which); device pointers are used in place, host pointers are staged.
 * All functions return -1 and set adaptq_last_error() on failure.
 */
#ifndef ADAPTQ_B200_EXT_H
#define ADAPTQ_B200_EXT_H

#include "adaptq.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Like adaptq_mha_create (upstream core/adaptq_c_api.cpp:149-165) but every
 * head-instance gets its own seed, so one handle can hold the heads of many
 * layers and sequences (upstream builds one Engine per layer with seed
 * 42 ^ layer and lets the handle derive head seeds from it). */
adaptq_mha_t adaptq_mha_create_seeded(int n_heads, const uint64_t *seeds,
                                      int dim, int k_bits, int v_bits,
                                      int capacity, float v_mass,
                                      int hybrid_thresh);

/* Append n_tokens tokens to every head.  keys, vals: float
 * [n_tokens][n_heads][dim].  Equals, for t in order and every head h,
 * adaptq_mha_append(mha, h, keys[t][h], vals[t][h], token_pos0 + t)
 * (upstream attention/attention.cpp:338-366).  Returns 0. */
int adaptq_mha_append_batch(adaptq_mha_t mha, const float *keys,
                            const float *vals, int n_tokens, int token_pos0);

/* Attention for every head, queries_per_head queries each.  queries, outs:
 * float [n_heads][queries_per_head][dim].  Equals adaptq_mha_compute_batch
 * on every head (upstream attention/attention.cpp:480-677).  The queries of
 * a head are processed side by side, so the head's cache comes from HBM
 * once and the other queries find it in L2.  Returns the largest per-head
 * token count. */
int adaptq_mha_compute_all(adaptq_mha_t mha, const float *queries,
                           int queries_per_head, float *outs);

/* One decode step for every head: append one token per head, then attend
 * with one query per head.  keys, vals, queries, outs: float [n_heads][dim].
 * Equals adaptq_mha_append_batch(mha, keys, vals, 1, token_pos) followed by
 * adaptq_mha_compute_all(mha, queries, 1, outs) -- what upstream's
 * AdaptQAttention.forward does per token (adaptq/torch_adapter.py:100-108,
 * Engine.append then Engine.compute).  When all four buffers are page-locked
 * host memory (and the handle has at least 4096 heads moving in lockstep,
 * dense V) the heads are processed in chunks whose uploads, kernels and
 * downloads overlap on separate CUDA streams, so the host transfers hide
 * behind the kernels; otherwise the two calls run one after the other.
 * Returns the token count after the append, or -1. */
int adaptq_mha_decode_step(adaptq_mha_t mha, const float *keys,
                           const float *vals, const float *queries,
                           float *outs, int token_pos);

/* Sequence sharding.  When the tokens of ONE logical cache are spread over
 * several handles (for instance token t on GPU t mod G), each handle
 * produces un-normalised softmax partials in the rotated domain:
 *   partials: float [n_heads][queries_per_head][adaptq_mha_partial_floats()]
 *   = { running max m, sum l = sum_i exp(logit_i - m), acc[padded] }.
 * adaptq_mha_merge_partials combines n_parts of them (laid out
 * [n_parts][n_heads][queries_per_head][...]; gathered by the caller, e.g.
 * with an NCCL all-gather), applies the single inverse transform and
 * writes outs [n_heads][queries_per_head][dim].  Dense V and quantized K
 * only (v_mass <= 0, hybrid_thresh == 0, k_bits != 16, v_bits != 16). */
int adaptq_mha_partial_floats(adaptq_mha_t mha);
int adaptq_mha_compute_partial(adaptq_mha_t mha, const float *queries,
                               int queries_per_head, float *partials);
int adaptq_mha_merge_partials(adaptq_mha_t mha, const float *partials,
                              int n_parts, int queries_per_head, float *outs);

/* The same exchange without a collective-library call, for GPUs that can map
 * each other's memory (NVLink peers, e.g. torch symmetric memory or CUDA IPC):
 * the streaming kernel itself stores each head's combined partial into EVERY
 * rank's gather buffer as soon as that head is done, so the transfer overlaps
 * the rest of the kernel, and the receiving side's merge kernel waits on
 * per-rank arrival counts.
 *   peer_bufs[r]  : rank r's gather buffer, float [world][n_heads*queries_per_head]
 *                   [adaptq_mha_partial_floats()], as mapped in THIS process;
 *                   this rank fills slice [rank] of every buffer.
 *   peer_flags[r] : rank r's unsigned[world] arrival counts (zero before the
 *                   first step, never reset); this rank adds 1 to
 *                   peer_flags[r][rank] per (head, query) delivered, with
 *                   release semantics at system scope.
 * adaptq_mha_merge_from_peers(mha, own gather buffer, own counts, world,
 * expected, ...) waits until every count has reached `expected` (the running
 * total: step number x n_heads x queries_per_head, compared modulo 2^32),
 * merges and writes outs [n_heads][queries_per_head][dim].  The wait is
 * bounded (about a quarter of a second): if a peer never delivers, the outputs
 * are zeros and adaptq_mha_synchronize() reports the failure.  Use two gather
 * buffers in turn (step parity): a rank's next step may deliver while a slower
 * peer still merges the previous one.  Streaming-kernel shapes only, device
 * pointers only, at most 8 ranks.  No counterpart upstream. */
int adaptq_mha_compute_partial_to_peers(adaptq_mha_t mha, const float *queries,
                                        int queries_per_head,
                                        float *const *peer_bufs,
                                        unsigned int *const *peer_flags,
                                        int world, int rank);
int adaptq_mha_merge_from_peers(adaptq_mha_t mha, const float *gather_buf,
                                const unsigned int *flags, int world,
                                unsigned int expected, int queries_per_head,
                                float *outs);

/* Decode attention for every head WITHOUT any device or host allocation.
 * This entry point has no counterpart in upstream; it exists for callers
 * that must not reach the CUDA allocator after start-up -- an inference
 * server whose memory pool already owns all free HBM (a late cudaMalloc
 * fails there), or a decode loop that cannot afford the device-wide stall
 * an allocation or free can cause.  Same result as adaptq_mha_compute_all.
 *
 *  - queries, outs: DEVICE memory, float [n_heads][queries_per_head][dim].
 *  - Shapes of the streaming kernel only: K and V at 2, 3 or 4 bits with
 *    head dim 128 (3- or 4-bit K at dim 64), v_mass <= 0,
 *    hybrid_thresh == 0, all heads holding the same number of tokens.
 *    Anything else returns -1.
 *  - The split-KV partials live in a 4 MiB array inside the library image
 *    (held on every GPU that loads the library, until the process exits)
 *    instead of a cudaMalloc buffer.  A call needing more -- spans x n_heads
 *    x queries_per_head x (2 + padded) floats -- is refused with -1 and an
 *    error text; nothing is truncated.
 *  - The first call made on a device looks up the array's device address
 *    (cudaGetSymbolAddress); make that first call outside any stream
 *    capture.  Later calls do no set-up.
 *  - All handles and all calls on a device share the one array and it keeps
 *    the previous call's contents.  Nothing in it needs clearing (every slot
 *    read is written first by the same call), but two such calls that
 *    overlap on the GPU -- different streams or handles -- race on it:
 *    serialise them.
 * Returns the token count, or -1 with adaptq_last_error() set. */
int adaptq_mha_compute_all_static(adaptq_mha_t mha, const float *queries,
                                  int queries_per_head, float *outs);

/* Layer stacks.  Upstream keeps one Engine per transformer layer (seed
 * 42 ^ layer, its README and benchmarks) and walks layers and heads in Python,
 * one C call per head (adaptq/core.py:53-57, :70-72): 2 x layers x heads calls
 * per token.  A stack holds the caches of ALL layers -- layer l is what
 * Engine(dim, n_heads, k_bits[l], v_bits[l], capacity, seed ^ l, v_mass,
 * hybrid_thresh) holds -- and moves a token through every layer in one call.
 * Consecutive layers with the same (k_bits, v_bits) share one multi-head handle
 * (a "part"); the parts run on CUDA streams of their own, so e.g. the FP32-key
 * first layer of a layer-aware policy overlaps the quantized layers behind it.
 * Buffers are float [n_layers][n_heads][dim] (append: [n_tokens][n_layers]
 * [n_heads][dim]), host or device; with device buffers nothing synchronises.
 * Additions without a counterpart upstream; results equal the per-layer loop. */
typedef void *adaptq_stack_t;
adaptq_stack_t adaptq_stack_create(int n_layers, int n_heads, int dim,
                                   const int *k_bits, const int *v_bits,
                                   int capacity, uint64_t seed, float v_mass,
                                   int hybrid_thresh);
void adaptq_stack_destroy(adaptq_stack_t st);
int adaptq_stack_append(adaptq_stack_t st, const float *keys, const float *vals,
                        int n_tokens, int token_pos0);
int adaptq_stack_compute(adaptq_stack_t st, const float *queries, float *outs);
/* append(keys, vals, 1) + compute(queries) for every layer: 2 launches per part */
int adaptq_stack_decode_step(adaptq_stack_t st, const float *keys,
                             const float *vals, const float *queries,
                             float *outs, int token_pos);
int adaptq_stack_reset(adaptq_stack_t st);
size_t adaptq_stack_kv_bytes(adaptq_stack_t st);
/* number of parts; the multi-head handle that holds `layer` and the index of the
 * layer's first head inside it (for adaptq_mha_export_head, adaptq_mha_info) */
int adaptq_stack_parts(adaptq_stack_t st);
adaptq_mha_t adaptq_stack_layer_handle(adaptq_stack_t st, int layer, int *first_head);
int adaptq_stack_set_stream(adaptq_stack_t st, void *cuda_stream);
/* wait for the stack's work and report a kernel that gave up waiting (see
 * adaptq_mha_synchronize) */
int adaptq_stack_synchronize(adaptq_stack_t st);

/* Test hook: make the nth upcoming host-side call of one kind report failure
 * without touching the device -- kind 1: device allocation, 2: page-locked host
 * allocation, 3: kernel launch (the check after a launch sees an error; the
 * kernel itself still runs).  nth = 0 switches the kind off.  Lets tests walk
 * every error path of this library (NULL / -1 returns, error text, no leaked
 * memory, handle still usable) on a healthy GPU; nothing faults.  Upstream has
 * no counterpart (its allocation failures throw through the C ABI,
 * cache/ring_buffer.cpp:71-76). */
int adaptq_inject_failure(int kind, int nth);

/* Use `cuda_stream` (a cudaStream_t; NULL = the default stream) for all
 * further work of this handle. */
int adaptq_mha_set_stream(adaptq_mha_t mha, void *cuda_stream);
/* Wait until everything queued on the handle's stream has finished; returns
 * -1 and sets the error string if a kernel reported a fault. */
int adaptq_mha_synchronize(adaptq_mha_t mha);

typedef struct {
  int n_heads, dim, padded, k_bits, v_bits, capacity, hybrid_thresh;
  int k_row_bytes, v_row_bytes; /* as upstream cache/ring_buffer.cpp:52-53 */
  int device;                   /* CUDA device ordinal holding the cache */
  float v_mass;
  size_t device_bytes;          /* GPU memory owned by the handle */
} adaptq_mha_info_t;
int adaptq_mha_info(adaptq_mha_t mha, adaptq_mha_info_t *info);

/* Copy one head's cache to HOST buffers in upstream's memory layout
 * (include/ring_buffer.h:61-66): k_rows capacity*k_row_bytes bytes, v_rows
 * capacity*v_row_bytes bytes, k_scale/v_scale capacity floats, signs
 * `padded` int8 (+1/-1).  Any output pointer may be NULL.  ring_head /
 * ring_size / mirror_tokens receive the ring state. */
int adaptq_mha_export_head(adaptq_mha_t mha, int head_idx, uint8_t *k_rows,
                           uint8_t *v_rows, float *k_scale, float *v_scale,
                           int8_t *signs, int *ring_head, int *ring_size,
                           int *mirror_tokens);

/* Number of CUDA kernels this library has launched in this process. */
unsigned long long adaptq_kernel_launches(void);

/* Force a code path, for tests: 0 = automatic, 1 = general-purpose kernels
 * only, 2 = refuse shapes the specialised kernels do not cover. */
int adaptq_set_kernel_policy(int policy);

#ifdef __cplusplus
}
#endif
#endif /* ADAPTQ_B200_EXT_H */
