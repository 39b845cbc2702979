// ref_shim.cpp -- TEST INFRASTRUCTURE.  Linked together with the UPSTREAM
// sources (never copied into this repository) by oracle/build_ref.sh.  It
// gives C linkage to the upstream AttentionHead struct
// (include/attention.h:9-35) so that tests can read the packed K/V slabs and
// scales, which the upstream C API does not expose, and adds bulk loops so a
// timing harness does not pay one foreign-function call per token.
#include "attention.h"
#include "codebook.h"
#include "fwht.h"
#include "quantizer.h"
#include <chrono>
#include <cstdint>
#include <cstring>
#include <exception>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

void *ref_head_create(int dim, int k_bits, int v_bits, int capacity,
                      uint64_t seed, float v_mass, int hybrid_thresh) {
  try {
    auto *h = new AttentionHead();
    h->init(dim, k_bits, v_bits, capacity, seed, v_mass, hybrid_thresh);
    return h;
  } catch (const std::exception &) {
    return nullptr;
  }
}
void ref_head_destroy(void *p) { delete static_cast<AttentionHead *>(p); }
void ref_head_append(void *p, const float *k, const float *v, int pos) {
  static_cast<AttentionHead *>(p)->append_kv(k, v, pos);
}
void ref_head_append_many(void *p, const float *keys, const float *vals,
                          int n_tokens, int pos0) {
  auto *h = static_cast<AttentionHead *>(p);
  for (int t = 0; t < n_tokens; ++t)
    h->append_kv(keys + (size_t)t * h->dim, vals + (size_t)t * h->dim, pos0 + t);
}
int ref_head_compute(void *p, const float *q, float *out) {
  return static_cast<AttentionHead *>(p)->compute(q, out);
}
int ref_head_compute_batch(void *p, const float *qs, int nq, float *outs) {
  return static_cast<AttentionHead *>(p)->compute_batch(qs, nq, outs);
}
void ref_head_reset(void *p) { // what adaptq_reset does, core/adaptq_c_api.cpp:128-137
  auto *h = static_cast<AttentionHead *>(p);
  h->kv_buf.size = 0;
  h->kv_buf.head = 0;
  h->raw_kv.clear();
}
const uint8_t *ref_head_k_data(void *p) { return static_cast<AttentionHead *>(p)->kv_buf.k_data; }
const uint8_t *ref_head_v_data(void *p) { return static_cast<AttentionHead *>(p)->kv_buf.v_data; }
const float *ref_head_k_scale(void *p) { return static_cast<AttentionHead *>(p)->kv_buf.k_scale.data(); }
const float *ref_head_v_scale(void *p) { return static_cast<AttentionHead *>(p)->kv_buf.v_scale.data(); }
const int8_t *ref_head_signs(void *p) { return static_cast<AttentionHead *>(p)->quant.D.data(); }
int ref_head_ring_head(void *p) { return static_cast<AttentionHead *>(p)->kv_buf.head; }
int ref_head_size(void *p) { return static_cast<AttentionHead *>(p)->kv_buf.size; }
int ref_head_padded(void *p) { return static_cast<AttentionHead *>(p)->padded; }
int ref_head_k_row_bytes(void *p) { return static_cast<AttentionHead *>(p)->kv_buf.k_packed_bytes; }
int ref_head_v_row_bytes(void *p) { return static_cast<AttentionHead *>(p)->kv_buf.v_packed_bytes; }
int ref_head_mirror_tokens(void *p) {
  auto *h = static_cast<AttentionHead *>(p);
  return (int)(h->raw_kv.size() / (2 * (size_t)h->dim));
}
size_t ref_head_kv_bytes(void *p) { return static_cast<AttentionHead *>(p)->kv_bytes(); }

// Free functions of the math layer, for known-answer tests.
int ref_next_pow2(int n) { return next_pow2(n); }
void ref_gen_rademacher(int8_t *D, int d, uint64_t seed) { gen_rademacher(D, d, seed); }
int ref_fwht_forward(float *x, const int8_t *D, int d) {
  try { fwht_forward(x, D, d); return 0; } catch (const std::exception &) { return -1; }
}
int ref_fwht_inverse(float *x, const int8_t *D, int d) {
  try { fwht_inverse(x, D, d); return 0; } catch (const std::exception &) { return -1; }
}
int ref_quantize_fast(float v, int bits) { return quantize_fast(v, bits); }
int ref_quantize_scalar(float v, int bits) { return quantize_scalar(v, get_codebook(bits), codebook_size(bits)); }
const float *ref_codebook(int bits) { return get_codebook(bits); }
int ref_codebook_size(int bits) { return codebook_size(bits); }
int ref_pack_indices(const uint8_t *idx, int d, int bits, uint8_t *dst) {
  try { pack_indices(idx, d, bits, dst); return 0; } catch (const std::exception &) { return -1; }
}
int ref_unpack_indices(const uint8_t *src, int d, int bits, uint8_t *idx) {
  try { unpack_indices(src, d, bits, idx); return 0; } catch (const std::exception &) { return -1; }
}
float ref_quantize_into(const float *x, int dim, uint64_t seed, int bits, uint8_t *packed) {
  Quantizer qz;
  qz.init(dim, seed);
  return qz.quantize_into(x, bits, packed);
}
void ref_dequantize_raw(const uint8_t *packed, float scale, int dim, uint64_t seed, int bits, float *out) {
  Quantizer qz;
  qz.init(dim, seed);
  qz.dequantize_raw(packed, scale, qz.padded, bits, out);
}

int ref_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Timing harness: `n_heads` independent heads (one worker per head, handles
// are independent), each appended with `n_tokens` tokens from keys/vals
// [n_heads][n_tokens][dim]; then `n_steps` decode steps, each one append of one
// more token per head (row step % n_tokens again; with capacity == n_tokens the
// ring is full and evicts) followed by one query per head from
// queries[n_heads][dim].  Returns seconds for the fill in *t_append and for the
// decode steps in *t_compute.  outs is [n_heads][dim] (last step).
int ref_time_heads(int n_heads, int dim, int k_bits, int v_bits, int capacity,
                   uint64_t base_seed, float v_mass, int hybrid_thresh,
                   const float *keys, const float *vals, int n_tokens,
                   const float *queries, int n_steps, float *outs,
                   int n_threads, double *t_append, double *t_compute) {
  std::vector<AttentionHead *> heads(n_heads, nullptr);
  try {
    for (int i = 0; i < n_heads; ++i) {
      heads[i] = new AttentionHead();
      heads[i]->init(dim, k_bits, v_bits, capacity,
                     base_seed ^ ((uint64_t)i * 0xDEADBEEFCAFEULL), v_mass, hybrid_thresh);
    }
  } catch (const std::exception &) {
    for (auto *h : heads) delete h;
    return -1;
  }
  (void)n_threads;
  auto t0 = std::chrono::steady_clock::now();
#pragma omp parallel for schedule(dynamic, 1) num_threads(n_threads)
  for (int i = 0; i < n_heads; ++i) {
    const float *k = keys + (size_t)i * n_tokens * dim;
    const float *v = vals + (size_t)i * n_tokens * dim;
    for (int t = 0; t < n_tokens; ++t)
      heads[i]->append_kv(k + (size_t)t * dim, v + (size_t)t * dim, t);
  }
  auto t1 = std::chrono::steady_clock::now();
  for (int s = 0; s < n_steps; ++s) {
#pragma omp parallel for schedule(dynamic, 1) num_threads(n_threads)
    for (int i = 0; i < n_heads; ++i) {
      const size_t row = ((size_t)i * n_tokens + (size_t)(s % n_tokens)) * dim;
      heads[i]->append_kv(keys + row, vals + row, n_tokens + s);
      heads[i]->compute(queries + (size_t)i * dim, outs + (size_t)i * dim);
    }
  }
  auto t2 = std::chrono::steady_clock::now();
  *t_append = std::chrono::duration<double>(t1 - t0).count();
  *t_compute = std::chrono::duration<double>(t2 - t1).count();
  for (auto *h : heads) delete h;
  return 0;
}

} // extern "C"
