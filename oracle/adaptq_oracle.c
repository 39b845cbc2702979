/*
 * adaptq_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C, single-threaded restatement of the AdapTQ quantized KV-cache
 * append / decode-attention algorithm as the l3tchupkt/adaptq CPU core
 * computes it.  It exists so the CUDA library can be checked on a machine
 * that does not have the upstream sources.  Only tests/, the smoke check and
 * the CPU-baseline leg of bench.py may load it; the product path never does.
 *
 * Parity status: PINNED.  oracle/build_ref.sh compiles the upstream sources
 * themselves (with the one-line template fix described there) into
 * oracle/_ref/, and tests/test_oracle_vs_ref.py checks this file against that
 * build bit-for-bit (packed bytes, scales AND attention outputs); the golden
 * fixtures under tests/golden/ were produced by that upstream build.
 *
 * Build: gcc -O2 -ffp-contract=off -shared -fPIC (see oracle/Makefile).
 * -ffp-contract=off matters: the upstream scalar loops are written as
 * separate multiply and add, and packed indices are only reproducible when
 * the compiler does not fuse them.  Where upstream uses explicit AVX2 FMA
 * intrinsics this file calls fmaf() so the rounding is the same.
 *
 * Every function cites the upstream file:line it follows (paths are relative
 * to the upstream project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_MAX_PADDED 1024 /* core/quantizer.cpp:12-13, core/fwht.cpp:10 */

/* ------------------------------------------------------------------ */
/* core/fwht.cpp                                                        */
/* ------------------------------------------------------------------ */

/* core/fwht.cpp:13-19 */
int orc_next_pow2(int n) {
  if (n <= 1) return 1;
  if (n > (1 << 30)) return (1 << 30);
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

/* core/fwht.cpp:21-27 -- xorshift64, sign = low bit */
void orc_gen_rademacher(int8_t *D, int d, uint64_t seed) {
  uint64_t s = seed ? seed : 0xdeadbeefcafe1234ULL;
  for (int i = 0; i < d; ++i) {
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    D[i] = (s & 1) ? 1 : -1;
  }
}

/* Butterfly passes len = first .. n/2; lower index gets a+b, upper a-b.
 * core/fwht.cpp:43-57 (forward, starts at len 2) and :69-86 (inverse, len 1) */
static void butterflies(float *x, int n, int first_len) {
  for (int len = first_len; len < n; len <<= 1)
    for (int i = 0; i < n; i += len << 1)
      for (int j = 0; j < len; ++j) {
        float a = x[i + j], b = x[i + j + len];
        x[i + j] = a + b;
        x[i + j + len] = a - b;
      }
}

/* core/fwht.cpp:33-66 -- sign flip fused with the len=1 pass, then the
 * remaining passes, then one multiply by 1/sqrt(n). */
static void fwht_fused(float *x, const int8_t *D, int d, int n) {
  for (int i = 0; i < n; i += 2) {
    float a = x[i] * (i < d ? (float)D[i] : 1.0f);
    float b = x[i + 1] * (i + 1 < d ? (float)D[i + 1] : 1.0f);
    x[i] = a + b;
    x[i + 1] = a - b;
  }
  butterflies(x, n, 2);
  float inv = 1.0f / sqrtf((float)n);
  for (int i = 0; i < n; ++i) x[i] *= inv;
}

/* core/fwht.cpp:88-104 (zero-pads to the next power of two, copies d back) */
void orc_fwht_forward(float *x, const int8_t *D, int d) {
  if (!x || !D || d <= 0) return;
  int p = orc_next_pow2(d);
  if (p > ORC_MAX_PADDED) return;
  float pad[ORC_MAX_PADDED];
  float *work = x;
  if (p != d) {
    memcpy(pad, x, (size_t)d * sizeof(float));
    memset(pad + d, 0, (size_t)(p - d) * sizeof(float));
    work = pad;
  }
  if (p == 1) { /* the upstream len=1 loop would touch x[1]; p==1 is identity*sign */
    work[0] = work[0] * (float)D[0];
  } else {
    fwht_fused(work, D, d, p);
  }
  if (p != d) memcpy(x, work, (size_t)d * sizeof(float));
}

/* core/fwht.cpp:106-134 -- butterflies from len 1, then work*scale*D */
void orc_fwht_inverse(float *x, const int8_t *D, int d) {
  if (!x || !D || d <= 0) return;
  int p = orc_next_pow2(d);
  if (p > ORC_MAX_PADDED) return;
  float pad[ORC_MAX_PADDED];
  float *work = x;
  if (p != d) {
    memcpy(pad, x, (size_t)d * sizeof(float));
    memset(pad + d, 0, (size_t)(p - d) * sizeof(float));
    work = pad;
  }
  butterflies(work, p, 1);
  float scale = 1.0f / sqrtf((float)p);
  for (int i = 0; i < p; ++i)
    work[i] = work[i] * scale * (i < d ? (float)D[i] : 1.0f);
  if (p != d) memcpy(x, work, (size_t)d * sizeof(float));
}

/* ------------------------------------------------------------------ */
/* core/codebook.cpp                                                    */
/* ------------------------------------------------------------------ */

/* Lloyd-Max N(0,1) centroids, core/codebook.cpp:32-62 */
static const float CB2[4] = {-1.5104f, -0.4528f, 0.4528f, 1.5104f};
static const float CB3[8] = {-2.1529f, -1.3439f, -0.7560f, -0.2451f,
                             0.2451f,  0.7560f,  1.3439f,  2.1529f};
static const float CB4[16] = {-2.4008f, -1.8944f, -1.5105f, -1.2016f,
                              -0.9138f, -0.6402f, -0.3795f, -0.1258f,
                              0.1258f,  0.3795f,  0.6402f,  0.9138f,
                              1.2016f,  1.5105f,  1.8944f,  2.4008f};

/* core/codebook.cpp:102-109 */
const float *orc_codebook(int bits) {
  switch (bits) {
  case 2: return CB2;
  case 3: return CB3;
  default: return CB4;
  }
}

/* core/codebook.cpp:111-115 */
int orc_codebook_size(int bits) {
  if (bits <= 2) return 4;
  if (bits == 3) return 8;
  return 16;
}

/* Decision thresholds = fp32 midpoints (a+b)*0.5f with an exact 0 in the
 * middle, core/codebook.cpp:67-100.  Computed, not typed in, so the rounding
 * is the expression's own. */
static float thresh(const float *cb, int n, int i) { /* i in [0, n-2] */
  if (i == n / 2 - 1) return 0.0f;
  return (cb[i] + cb[i + 1]) * 0.5f;
}

float orc_threshold(int bits, int i) {
  return thresh(orc_codebook(bits), orc_codebook_size(bits), i);
}

/* core/codebook.cpp:119-144 -- NaN goes to the centroid just below zero;
 * otherwise a binary search with `v >= t` decisions. */
int orc_quantize_fast(float v, int bits) {
  if (isnan(v)) {
    if (bits <= 2) return 1;
    if (bits == 3) return 3;
    return 7;
  }
  if (bits >= 4) {
    int i = (v >= thresh(CB4, 16, 7)) ? 8 : 0;
    i += (v >= thresh(CB4, 16, i + 3)) ? 4 : 0;
    i += (v >= thresh(CB4, 16, i + 1)) ? 2 : 0;
    i += (v >= thresh(CB4, 16, i)) ? 1 : 0;
    return i;
  }
  if (bits == 3) {
    int i = (v >= thresh(CB3, 8, 3)) ? 4 : 0;
    i += (v >= thresh(CB3, 8, i + 1)) ? 2 : 0;
    i += (v >= thresh(CB3, 8, i)) ? 1 : 0;
    return i;
  }
  int i = (v >= thresh(CB2, 4, 1)) ? 2 : 0;
  i += (v >= thresh(CB2, 4, i)) ? 1 : 0;
  return i;
}

/* core/codebook.cpp:147-159 -- nearest centroid by linear scan */
int orc_quantize_scalar(float val, const float *cb, int n) {
  if (!cb || n <= 0) return 0;
  if (isnan(val)) return 0;
  if (val >= cb[n - 1]) return n - 1;
  if (val <= cb[0]) return 0;
  int best = 0;
  float bd = fabsf(val - cb[0]);
  for (int i = 1; i < n; ++i) {
    float d = fabsf(val - cb[i]);
    if (d < bd) { bd = d; best = i; }
  }
  return best;
}

/* ------------------------------------------------------------------ */
/* core/quantizer.cpp                                                   */
/* ------------------------------------------------------------------ */

/* MSB-first bit packing, core/quantizer.cpp:156-194 */
int orc_pack_indices(const uint8_t *idx, int d, int bits, uint8_t *dst) {
  if (bits == 4) {
    for (int i = 0; i < d / 2; ++i)
      dst[i] = (uint8_t)((idx[2 * i] << 4) | (idx[2 * i + 1] & 0xF));
  } else if (bits == 2) {
    for (int i = 0; i < d / 4; ++i)
      dst[i] = (uint8_t)((idx[4 * i] << 6) | (idx[4 * i + 1] << 4) |
                         (idx[4 * i + 2] << 2) | idx[4 * i + 3]);
  } else if (bits == 3) {
    for (int g = 0; g < d / 8; ++g) {
      const uint8_t *s = idx + g * 8;
      uint8_t *p = dst + g * 3;
      p[0] = (uint8_t)((s[0] << 5) | (s[1] << 2) | (s[2] >> 1));
      p[1] = (uint8_t)((s[2] << 7) | (s[3] << 4) | (s[4] << 1) | (s[5] >> 2));
      p[2] = (uint8_t)((s[5] << 6) | (s[6] << 3) | s[7]);
    }
  } else {
    return -1; /* upstream throws, core/quantizer.cpp:222-224 */
  }
  return 0;
}

int orc_unpack_indices(const uint8_t *src, int d, int bits, uint8_t *idx) {
  if (bits == 4) {
    for (int i = 0; i < d / 2; ++i) {
      idx[2 * i] = src[i] >> 4;
      idx[2 * i + 1] = src[i] & 0xF;
    }
  } else if (bits == 2) {
    for (int i = 0; i < d / 4; ++i) {
      idx[4 * i] = (src[i] >> 6) & 3;
      idx[4 * i + 1] = (src[i] >> 4) & 3;
      idx[4 * i + 2] = (src[i] >> 2) & 3;
      idx[4 * i + 3] = src[i] & 3;
    }
  } else if (bits == 3) {
    for (int g = 0; g < d / 8; ++g) {
      const uint8_t *p = src + g * 3;
      uint8_t *s = idx + g * 8;
      s[0] = (p[0] >> 5) & 7;
      s[1] = (p[0] >> 2) & 7;
      s[2] = (uint8_t)(((p[0] & 3) << 1) | (p[1] >> 7));
      s[3] = (p[1] >> 4) & 7;
      s[4] = (p[1] >> 1) & 7;
      s[5] = (uint8_t)(((p[1] & 1) << 2) | (p[2] >> 6));
      s[6] = (p[2] >> 3) & 7;
      s[7] = p[2] & 7;
    }
  } else {
    return -1;
  }
  return 0;
}

/* core/quantizer.cpp:53-101 -- returns the L2 norm (the stored scale);
 * idx_out receives `padded` indices.  The norm is a strictly sequential
 * mul-then-add chain over x[0..dim-1]. */
float orc_quantize_core(const float *x, int dim, int padded, const int8_t *D,
                        int bits, uint8_t *idx_out) {
  float buf[ORC_MAX_PADDED];
  float norm = 0.f;
  for (int i = 0; i < dim; ++i) {
    buf[i] = x[i];
    norm += x[i] * x[i];
  }
  for (int i = dim; i < padded; ++i) buf[i] = 0.f;
  norm = sqrtf(norm + 1e-12f);
  float inv = 1.f / norm;
  for (int i = 0; i < padded; ++i) buf[i] *= inv;

  orc_fwht_forward(buf, D, padded);
  float sp = sqrtf((float)padded);
  for (int i = 0; i < padded; ++i) buf[i] *= sp;

  float sum2 = 0.f;
  for (int i = 0; i < padded; ++i) sum2 += buf[i] * buf[i];
  float sigma = sqrtf(sum2 / (float)padded + 1e-12f);
  float clip = 3.0f * sigma;
  for (int i = 0; i < padded; ++i) {
    if (buf[i] > clip) buf[i] = clip;
    if (buf[i] < -clip) buf[i] = -clip;
  }
  for (int i = 0; i < padded; ++i)
    idx_out[i] = (uint8_t)orc_quantize_fast(buf[i], bits);
  return norm;
}

/* core/quantizer.cpp:131-137 */
float orc_quantize_into(const float *x, int dim, const int8_t *D, int bits,
                        uint8_t *packed) {
  uint8_t idx[ORC_MAX_PADDED];
  int padded = orc_next_pow2(dim);
  float s = orc_quantize_core(x, dim, padded, D, bits, idx);
  orc_pack_indices(idx, padded, bits, packed);
  return s;
}

/* core/quantizer.cpp:139-151 */
void orc_dequantize_raw(const uint8_t *packed, float scale, int dim,
                        const int8_t *D, int bits, float *out) {
  int padded = orc_next_pow2(dim);
  const float *cb = orc_codebook(bits);
  float inv_sq = 1.f / sqrtf((float)padded);
  uint8_t idx[ORC_MAX_PADDED];
  float buf[ORC_MAX_PADDED];
  orc_unpack_indices(packed, padded, bits, idx);
  for (int i = 0; i < padded; ++i) buf[i] = cb[idx[i]] * inv_sq;
  orc_fwht_inverse(buf, D, padded);
  for (int i = 0; i < dim; ++i) out[i] = buf[i] * scale;
}

/* ------------------------------------------------------------------ */
/* One attention head: cache/ring_buffer.cpp + attention/attention.cpp  */
/* ------------------------------------------------------------------ */

typedef struct orc_head {
  int dim, padded, k_bits, v_bits, capacity, hybrid_thresh;
  float v_mass;
  int8_t *D;
  /* KVFlatBuffer, include/ring_buffer.h:61-96 */
  uint8_t *k_data, *v_data;
  float *k_scale, *v_scale;
  int *positions;
  int k_pb, v_pb, head, size;
  /* hybrid FP32 mirror, include/attention.h:20 */
  float *raw_kv;
  size_t raw_len, raw_cap;
  /* Sparse-V walk: 4 = blocks of four rows, then single rows (attention/attention.cpp:456-472);
   * 1 = single rows from the start, the rule of upstream's second stack
   * (HARFixedStrategy::compute_full, strategies/har_fixed.cpp:258-264). */
  int sparse_block;
} orc_head;

static int packed_bytes(int padded, int bits) { /* cache/ring_buffer.cpp:52-53 */
  return bits == 16 ? padded * (int)sizeof(float) : (padded * bits + 7) / 8;
}

static int valid_bits(int b) { return b == 16 || (b >= 2 && b <= 4); }

void orc_head_destroy(orc_head *h) {
  if (!h) return;
  free(h->D); free(h->k_data); free(h->v_data);
  free(h->k_scale); free(h->v_scale); free(h->positions); free(h->raw_kv);
  free(h);
}

/* core/adaptq_c_api.cpp:63-74 (argument checks) + attention/attention.cpp:324-337
 * + core/quantizer.cpp:21-34 + cache/ring_buffer.cpp:47-84.  Returns NULL
 * where upstream returns NULL or throws. */
orc_head *orc_head_create(int dim, int k_bits, int v_bits, int capacity,
                          uint64_t seed, float v_mass, int hybrid_thresh) {
  if (dim <= 0 || !valid_bits(k_bits) || !valid_bits(v_bits) || capacity < 0 ||
      hybrid_thresh < 0)
    return NULL;
  int padded = orc_next_pow2(dim);
  if (padded > ORC_MAX_PADDED) return NULL;
  orc_head *h = (orc_head *)calloc(1, sizeof(orc_head));
  if (h) h->sparse_block = 4;
  if (!h) return NULL;
  h->dim = dim; h->padded = padded; h->k_bits = k_bits; h->v_bits = v_bits;
  h->capacity = capacity; h->hybrid_thresh = hybrid_thresh; h->v_mass = v_mass;
  h->k_pb = packed_bytes(padded, k_bits);
  h->v_pb = packed_bytes(padded, v_bits);
  h->D = (int8_t *)malloc((size_t)padded);
  orc_gen_rademacher(h->D, padded, seed);
  size_t kb = (size_t)capacity * h->k_pb, vb = (size_t)capacity * h->v_pb;
  h->k_data = (uint8_t *)calloc(kb + 64, 1);
  h->v_data = (uint8_t *)calloc(vb + 64, 1);
  h->k_scale = (float *)malloc(sizeof(float) * (size_t)(capacity + 1));
  h->v_scale = (float *)malloc(sizeof(float) * (size_t)(capacity + 1));
  h->positions = (int *)calloc((size_t)capacity + 1, sizeof(int));
  for (int i = 0; i < capacity; ++i) h->k_scale[i] = h->v_scale[i] = 1.f;
  return h;
}

static void raw_push(orc_head *h, const float *a, int n) {
  if (h->raw_len + (size_t)n > h->raw_cap) {
    size_t nc = h->raw_cap ? h->raw_cap * 2 : 1024;
    while (nc < h->raw_len + (size_t)n) nc *= 2;
    h->raw_kv = (float *)realloc(h->raw_kv, nc * sizeof(float));
    h->raw_cap = nc;
  }
  memcpy(h->raw_kv + h->raw_len, a, (size_t)n * sizeof(float));
  h->raw_len += (size_t)n;
}

/* attention/attention.cpp:338-366 + cache/ring_buffer.cpp:105-119 */
void orc_head_append(orc_head *h, const float *key, const float *val, int pos) {
  uint8_t tk[ORC_MAX_PADDED * 4], tv[ORC_MAX_PADDED * 4];
  float ks = 1.f, vs = 1.f;
  if (h->k_bits == 16) {
    memcpy(tk, key, (size_t)h->dim * 4);
    memset(tk + (size_t)h->dim * 4, 0, (size_t)(h->padded - h->dim) * 4);
  } else {
    ks = orc_quantize_into(key, h->dim, h->D, h->k_bits, tk);
  }
  if (h->v_bits == 16) {
    memcpy(tv, val, (size_t)h->dim * 4);
    memset(tv + (size_t)h->dim * 4, 0, (size_t)(h->padded - h->dim) * 4);
  } else {
    vs = orc_quantize_into(val, h->dim, h->D, h->v_bits, tv);
  }
  int will_evict = h->size >= h->capacity;
  if (h->capacity > 0) {
    int idx = h->head;
    memcpy(h->k_data + (size_t)idx * h->k_pb, tk, (size_t)h->k_pb);
    memcpy(h->v_data + (size_t)idx * h->v_pb, tv, (size_t)h->v_pb);
    h->k_scale[idx] = ks;
    h->v_scale[idx] = vs;
    h->positions[idx] = pos;
    h->head = (h->head + 1) % h->capacity;
    if (h->size < h->capacity) ++h->size;
  }
  if (h->hybrid_thresh > 0) {
    if (!will_evict &&
        h->raw_len < (size_t)h->hybrid_thresh * 2 * (size_t)h->dim) {
      raw_push(h, key, h->dim);
      raw_push(h, val, h->dim);
    } else if (will_evict && h->raw_len) {
      h->raw_len = 0;
    }
  }
}

/* core/adaptq_c_api.cpp:128-137 */
void orc_head_reset(orc_head *h) {
  h->size = 0; h->head = 0; h->raw_len = 0;
}

size_t orc_head_kv_bytes(const orc_head *h) { /* include/ring_buffer.h:93 */
  return (size_t)h->size * (size_t)(h->k_pb + h->v_pb);
}

/* Unpack one packed row into `padded` indices. */
static void row_indices(const uint8_t *row, int padded, int bits, uint8_t *idx) {
  orc_unpack_indices(row, padded, bits, idx);
}

/* attention/attention.cpp:85-91 -- (v0+v4 + v1+v5) + (v2+v6 + v3+v7) */
static float hsum8(const float *s) {
  float a0 = s[0] + s[4], a1 = s[1] + s[5], a2 = s[2] + s[6], a3 = s[3] + s[7];
  return (a0 + a1) + (a2 + a3);
}

/* attention/attention.cpp:93-136 -- eight FMA lanes over blocks of 8 */
static float kdot_lanes(const float *qr, const uint8_t *idx, const float *cb,
                        int padded) {
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int j = 0; j < padded; j += 8)
    for (int l = 0; l < 8; ++l) s[l] = fmaf(cb[idx[j + l]], qr[j + l], s[l]);
  return hsum8(s);
}

typedef struct { float w; int i; } wi_t;
static int cmp_desc(const void *a, const void *b) {
  const wi_t *x = (const wi_t *)a, *y = (const wi_t *)b;
  if (x->w > y->w) return -1;
  if (x->w < y->w) return 1;
  return (x->i > y->i) - (x->i < y->i); /* upstream std::sort leaves ties unspecified */
}

/* Hooks for the sparse-V parity tests (thread-unsafe on purpose: tests are
 * single-threaded).  force_count >= 0 replaces the stopping rule of
 * attention/attention.cpp:456-472 by "accumulate exactly this many rows of the
 * sorted order"; trace_* record the running mass and the row count after every
 * step (a block of four, or a single row) of the natural walk. */
static int sp_force_count = -1;
static float *sp_trace_mass = NULL;
static int *sp_trace_count = NULL;
static int sp_trace_cap = 0, sp_trace_len = 0;

/* attention/attention.cpp:480-660.  `variant`: 0 = the path upstream takes on
 * an AVX2+FMA x86 host (compute_avx2, :373-474), 1 = its scalar 2/3/4-bit
 * fallback (:635-659).  The hybrid and K16 branches are common to both. */
int orc_head_compute_variant(const orc_head *h, const float *q, float *out,
                             int variant) {
  const int n = h->size, cap = h->capacity, dim = h->dim, padded = h->padded;
  if (!n) {
    memset(out, 0, (size_t)dim * sizeof(float));
    return 0;
  }
  float *logits = (float *)malloc(sizeof(float) * (size_t)n);
  int *slots = (int *)malloc(sizeof(int) * (size_t)n);

  /* hybrid FP32 path, attention/attention.cpp:491-523 */
  if (h->hybrid_thresh > 0 && n <= h->hybrid_thresh &&
      h->raw_len == (size_t)n * 2 * (size_t)dim) {
    const float scale = 1.f / sqrtf((float)dim);
    float mx = -1e30f;
    for (int i = 0; i < n; ++i) {
      const float *k = h->raw_kv + (size_t)i * 2 * dim;
      float d = 0.f;
      for (int j = 0; j < dim; ++j) d += q[j] * k[j];
      logits[i] = d * scale;
      if (logits[i] > mx) mx = logits[i];
    }
    float sv = 0.f;
    for (int i = 0; i < n; ++i) {
      logits[i] = expf(logits[i] - mx);
      sv += logits[i];
    }
    float inv = (sv > 0.f && isfinite(sv)) ? (1.f / sv) : (1.f / (float)n);
    memset(out, 0, (size_t)dim * sizeof(float));
    for (int i = 0; i < n; ++i) {
      float w = logits[i] * inv;
      const float *v = h->raw_kv + (size_t)i * 2 * dim + dim;
      for (int j = 0; j < dim; ++j) out[j] += w * v[j];
    }
    free(logits); free(slots);
    return n;
  }

  float qr[ORC_MAX_PADDED], acc[ORC_MAX_PADDED];
  uint8_t idx[ORC_MAX_PADDED];
  memcpy(qr, q, (size_t)dim * sizeof(float));
  for (int i = dim; i < padded; ++i) qr[i] = 0.f;
  float attn_s = 1.f / sqrtf((float)dim);
  float isp = 1.f / sqrtf((float)padded);

  if (h->k_bits != 16) { /* attention/attention.cpp:537-550 */
    float qn = 0.f;
    for (int i = 0; i < dim; ++i) qn += q[i] * q[i];
    qn = sqrtf(qn + 1e-12f);
    float inv = 1.f / qn;
    for (int i = 0; i < padded; ++i) qr[i] *= inv;
    orc_fwht_forward(qr, h->D, padded);
    float sp = sqrtf((float)padded);
    float m = sp * qn;
    for (int i = 0; i < padded; ++i) qr[i] *= m;
    attn_s = 1.f / (sqrtf((float)dim) * (float)padded);
  }
  const float *k_cb = h->k_bits != 16 ? orc_codebook(h->k_bits) : NULL;
  const float *v_cb = h->v_bits != 16 ? orc_codebook(h->v_bits) : NULL;
  for (int i = 0; i < n; ++i) slots[i] = (h->head - n + cap + i) % cap;

  if (h->k_bits == 16) { /* attention/attention.cpp:565-600 */
    float mx = -1e30f;
    for (int i = 0; i < n; ++i) {
      const float *k = (const float *)(h->k_data + (size_t)slots[i] * h->k_pb);
      float d = 0.f;
      for (int j = 0; j < dim; ++j) d += qr[j] * k[j];
      logits[i] = d * attn_s;
      if (logits[i] > mx) mx = logits[i];
    }
    float sv = 0.f;
    for (int i = 0; i < n; ++i) {
      logits[i] = expf(logits[i] - mx);
      sv += logits[i];
    }
    float inv = 1.f / sv;
    for (int i = 0; i < n; ++i) logits[i] *= inv;
    memset(acc, 0, (size_t)padded * sizeof(float));
    for (int i = 0; i < n; ++i) {
      int s = slots[i];
      if (h->v_bits == 16) {
        const float *v = (const float *)(h->v_data + (size_t)s * h->v_pb);
        float w = logits[i];
        for (int j = 0; j < dim; ++j) acc[j] += w * v[j];
      } else {
        float ecb[16];
        float ew = logits[i] * h->v_scale[s] * isp;
        int cb_sz = 1 << h->v_bits;
        for (int k = 0; k < cb_sz; ++k) ecb[k] = ew * v_cb[k];
        row_indices(h->v_data + (size_t)s * h->v_pb, padded, h->v_bits, idx);
        for (int j = 0; j < padded; ++j) acc[j] += ecb[idx[j]];
      }
    }
    if (h->v_bits != 16) orc_fwht_inverse(acc, h->D, padded);
    memcpy(out, acc, (size_t)dim * sizeof(float));
    free(logits); free(slots);
    return n;
  }

  if (h->v_bits == 16) {
    /* Quantized K with FP32 V is not a working combination upstream (the
     * scalar fallback indexes a 16-entry table with 65536 entries,
     * attention/attention.cpp:648-655).  The oracle defines it the natural
     * way: softmax weights times the raw V rows, no inverse transform. */
    float mx = -1e30f;
    for (int i = 0; i < n; ++i) {
      int s = slots[i];
      row_indices(h->k_data + (size_t)s * h->k_pb, padded, h->k_bits, idx);
      logits[i] = kdot_lanes(qr, idx, k_cb, padded) * attn_s * h->k_scale[s];
      if (logits[i] > mx) mx = logits[i];
    }
    float sv = 0.f;
    for (int i = 0; i < n; ++i) { logits[i] = expf(logits[i] - mx); sv += logits[i]; }
    float inv = 1.f / sv;
    memset(acc, 0, (size_t)padded * sizeof(float));
    for (int i = 0; i < n; ++i) {
      const float *v = (const float *)(h->v_data + (size_t)slots[i] * h->v_pb);
      float w = logits[i] * inv;
      for (int j = 0; j < dim; ++j) acc[j] += w * v[j];
    }
    memcpy(out, acc, (size_t)dim * sizeof(float));
    free(logits); free(slots);
    return n;
  }

  if (variant == 1) { /* scalar fallback, attention/attention.cpp:635-659 */
    for (int i = 0; i < n; ++i) {
      int s = slots[i];
      row_indices(h->k_data + (size_t)s * h->k_pb, padded, h->k_bits, idx);
      /* kdot_scalar (:247-281) sums groups of 4 (2-bit) or 8 (3/4-bit)
       * products left to right, then adds the group to the running sum. */
      int g = h->k_bits == 2 ? 4 : 8;
      float sacc = 0.f;
      for (int j = 0; j < padded; j += g) {
        float t = qr[j] * k_cb[idx[j]];
        for (int l = 1; l < g; ++l) t = t + qr[j + l] * k_cb[idx[j + l]];
        sacc += t;
      }
      logits[i] = sacc * attn_s * h->k_scale[s];
    }
    /* softmax(), attention/attention.cpp:220-245 */
    if (n == 1) {
      logits[0] = 1.0f;
    } else {
      float mx = logits[0];
      for (int i = 1; i < n; ++i) if (logits[i] > mx) mx = logits[i];
      float sv = 0.f;
      for (int i = 0; i < n; ++i) { logits[i] = expf(logits[i] - mx); sv += logits[i]; }
      if (sv > 0.f && isfinite(sv)) {
        float inv = 1.f / sv;
        for (int i = 0; i < n; ++i) logits[i] *= inv;
      } else {
        float u = 1.f / (float)n;
        for (int i = 0; i < n; ++i) logits[i] = u;
      }
    }
    memset(acc, 0, (size_t)padded * sizeof(float));
    int cb_sz = 1 << h->v_bits;
    for (int i = 0; i < n; ++i) {
      int s = slots[i];
      float ecb[16];
      float ew = logits[i] * h->v_scale[s] * isp;
      for (int k = 0; k < cb_sz; ++k) ecb[k] = ew * v_cb[k];
      row_indices(h->v_data + (size_t)s * h->v_pb, padded, h->v_bits, idx);
      for (int j = 0; j < padded; ++j) acc[j] += ecb[idx[j]];
    }
    orc_fwht_inverse(acc, h->D, padded);
    memcpy(out, acc, (size_t)dim * sizeof(float));
    free(logits); free(slots);
    return n;
  }

  /* compute_avx2, attention/attention.cpp:373-474 */
  float mx = -1e30f;
  for (int i = 0; i < n; ++i) {
    int s = slots[i];
    row_indices(h->k_data + (size_t)s * h->k_pb, padded, h->k_bits, idx);
    logits[i] = kdot_lanes(qr, idx, k_cb, padded) * attn_s * h->k_scale[s];
    if (logits[i] > mx) mx = logits[i];
  }
  float sv = 0.f;
  for (int j = 0; j < n; ++j) {
    logits[j] = expf(logits[j] - mx);
    sv += logits[j];
  }
  float inv = 1.f / sv;
  for (int j = 0; j < n; ++j) logits[j] *= inv;
  memset(acc, 0, (size_t)padded * sizeof(float));

  if (h->v_mass <= 0.f) { /* dense V, :432-447: acc[j] = fma(cb, w', acc[j]) in token order */
    for (int i = 0; i < n; ++i) {
      int s = slots[i];
      float e = logits[i] * h->v_scale[s] * isp;
      row_indices(h->v_data + (size_t)s * h->v_pb, padded, h->v_bits, idx);
      for (int j = 0; j < padded; ++j) acc[j] = fmaf(v_cb[idx[j]], e, acc[j]);
    }
  } else { /* sparse V, :448-473 */
    wi_t *ord = (wi_t *)malloc(sizeof(wi_t) * (size_t)n);
    for (int i = 0; i < n; ++i) { ord[i].w = logits[i]; ord[i].i = i; }
    qsort(ord, (size_t)n, sizeof(wi_t), cmp_desc);
    float mass = 0.f;
    int ii = 0;
    sp_trace_len = 0;
    const int forced = sp_force_count;
    for (; h->sparse_block == 4 && ii + 3 < n && (forced >= 0 ? ii + 3 < forced : mass < h->v_mass); ii += 4) {
      for (int t = 0; t < 4; ++t) {
        int s = slots[ord[ii + t].i];
        float e = ord[ii + t].w * h->v_scale[s] * isp;
        row_indices(h->v_data + (size_t)s * h->v_pb, padded, h->v_bits, idx);
        for (int j = 0; j < padded; ++j) acc[j] = fmaf(v_cb[idx[j]], e, acc[j]);
      }
      mass += ord[ii].w + ord[ii + 1].w + ord[ii + 2].w + ord[ii + 3].w;
      if (sp_trace_mass && sp_trace_len < sp_trace_cap) {
        sp_trace_mass[sp_trace_len] = mass;
        sp_trace_count[sp_trace_len++] = ii + 4;
      }
    }
    for (; ii < n && (forced >= 0 ? ii < forced : mass < h->v_mass); ++ii) {
      int s = slots[ord[ii].i];
      float w = ord[ii].w;
      float e = w * h->v_scale[s] * isp;
      row_indices(h->v_data + (size_t)s * h->v_pb, padded, h->v_bits, idx);
      for (int j = 0; j < padded; ++j) acc[j] = fmaf(v_cb[idx[j]], e, acc[j]);
      mass += w;
      if (sp_trace_mass && sp_trace_len < sp_trace_cap) {
        sp_trace_mass[sp_trace_len] = mass;
        sp_trace_count[sp_trace_len++] = ii + 1;
      }
    }
    free(ord);
  }
  orc_fwht_inverse(acc, h->D, padded);
  memcpy(out, acc, (size_t)dim * sizeof(float));
  free(logits); free(slots);
  return n;
}

int orc_head_compute(const orc_head *h, const float *q, float *out) {
  return orc_head_compute_variant(h, q, out, 0);
}

void orc_head_set_sparse_block(orc_head *h, int rows) { h->sparse_block = rows == 1 ? 1 : 4; }

/* Sparse V with the cut moved: the first `count` rows of the weight-sorted order
 * are accumulated (in blocks of four while four remain below `count`, then
 * singles -- the same grouping the natural walk uses), whatever their mass.
 * For tests that must tell a borderline cut from a wrong result. */
int orc_head_compute_cut(const orc_head *h, const float *q, float *out, int count) {
  sp_force_count = count < 0 ? 0 : count;
  int n = orc_head_compute_variant(h, q, out, 0);
  sp_force_count = -1;
  return n;
}

/* The natural sparse-V walk of one query: running mass and accumulated row
 * count after every step.  Returns the number of steps recorded (<= cap). */
int orc_head_sparse_trace(const orc_head *h, const float *q, float *out, float *mass,
                          int *count, int cap) {
  sp_trace_mass = mass; sp_trace_count = count; sp_trace_cap = cap; sp_trace_len = 0;
  orc_head_compute_variant(h, q, out, 0);
  sp_trace_mass = NULL; sp_trace_count = NULL; sp_trace_cap = 0;
  return sp_trace_len;
}

/* attention/attention.cpp:662-677 -- every query is an independent compute */
int orc_head_compute_batch(const orc_head *h, const float *qs, int nq, float *outs) {
  if (h->size == 0) {
    memset(outs, 0, (size_t)nq * h->dim * sizeof(float));
    return 0;
  }
  for (int i = 0; i < nq; ++i)
    orc_head_compute(h, qs + (size_t)i * h->dim, outs + (size_t)i * h->dim);
  return h->size;
}

/* Field access for the tests (the upstream struct is public,
 * include/attention.h:9-20, include/ring_buffer.h:61-96). */
const uint8_t *orc_head_k_data(const orc_head *h) { return h->k_data; }
const uint8_t *orc_head_v_data(const orc_head *h) { return h->v_data; }
const float *orc_head_k_scale(const orc_head *h) { return h->k_scale; }
const float *orc_head_v_scale(const orc_head *h) { return h->v_scale; }
const int8_t *orc_head_signs(const orc_head *h) { return h->D; }
int orc_head_ring_head(const orc_head *h) { return h->head; }
int orc_head_size(const orc_head *h) { return h->size; }
int orc_head_padded(const orc_head *h) { return h->padded; }
int orc_head_k_row_bytes(const orc_head *h) { return h->k_pb; }
int orc_head_v_row_bytes(const orc_head *h) { return h->v_pb; }
int orc_head_mirror_tokens(const orc_head *h) {
  return (int)(h->raw_len / (2 * (size_t)h->dim));
}

/* Per-head seed of the multi-head handle, core/adaptq_c_api.cpp:160 */
uint64_t orc_mha_head_seed(uint64_t base_seed, int head_idx) {
  return base_seed ^ ((uint64_t)head_idx * 0xDEADBEEFCAFEULL);
}

/* Bulk helpers so Python tests do not loop per token. keys/vals are
 * [n_tokens][dim]; queries [nq][dim]. */
void orc_head_append_many(orc_head *h, const float *keys, const float *vals,
                          int n_tokens, int pos0) {
  for (int t = 0; t < n_tokens; ++t)
    orc_head_append(h, keys + (size_t)t * h->dim, vals + (size_t)t * h->dim, pos0 + t);
}
