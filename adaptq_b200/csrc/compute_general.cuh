// General-purpose decode-attention kernels: every bit width (2/3/4/16 for K
// and V), every padded dimension up to 1024, the hybrid FP32 window, split-KV
// partials and their merge, and the sparse-V selection.
//
// Replaces upstream AttentionHead::compute (attention/attention.cpp:480-660):
// hybrid branch :491-523, query rotation :526-550, K16 branch :565-600,
// quantised branch (compute_avx2) :373-474, inverse transform
// (core/fwht.cpp:106-134).  Scores come straight from the packed indices
// through a q[j]*centroid table in shared memory; nothing is dequantised.
//
// A softmax over a set is independent of the order of the set, so the dense
// paths walk the ring's physical slots 0..n-1 (every slot below `size` is
// live, wrapped or not) instead of upstream's oldest-to-newest order.
#pragma once
#include "common.cuh"

namespace aq {

constexpr int CG_THREADS = 256;
constexpr int CG_WARPS = CG_THREADS / 32;

struct ComputeLaunch {
  CacheView c;
  const float *q; // [heads_in_call][nq][dim]
  float *out;     // [heads_in_call][nq][dim]            (mode 0)
  float *partial; // [n_splits][heads_in_call*nq][2+P]  (mode 1)
  float *weights; // [heads_in_call][nq][w_stride]       (mode 2: normalised softmax weights)
  int w_stride;
  int head0, heads_in_call, nq;
  int n;        // live tokens (same for every head of the call)
  int rot;      // ring slot of the oldest live token: logical position i sits in slot (rot + i) % capacity
  int use_mirror;
  int n_splits, span; // tokens per split
  int chunk;          // tokens per shared-memory pass
  int mode;
  int *status;  // checked build: where a failed index check is recorded
  // mode 1 with fused merge: the block that completes an item's last partial merges them
  int *counters;      // [heads_in_call*nq] arrival counts, zero before and after every launch (nullptr: no fused merge)
  float *final_out;   // outputs (or combined partials when final_to_partial)
  int final_to_partial;
};

// Shared-memory carve-up (floats): qr[P] | vec[P] | red[64] | vcb[16] | lut[P*CBK or 0] | sc[chunk]
__host__ __device__ inline size_t cg_smem_floats(int P, int k_quant_levels, int chunk) {
  return (size_t)P * 2 + 64 + 16 + (size_t)P * k_quant_levels + chunk;
}

// ---- packed rows by words -------------------------------------------------------------------
// For padded dimensions that are multiples of 32 a packed row is a whole number of 32-bit
// words, and 32 consecutive coordinates fill exactly BITS words.  Read as big-endian words the
// MSB-first layouts of upstream's packers (core/quantizer.cpp:156-194) become one bit stream:
// coordinate k of a 32-coordinate group starts k*BITS bits below the top of its first word.
template <int WORDS> __device__ __forceinline__ void load_words_be(const uint8_t *p, uint32_t (&w)[WORDS]) {
  if constexpr (WORDS == 4) {
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else if constexpr (WORDS == 2) {
    const uint2 v = __ldg(reinterpret_cast<const uint2 *>(p));
    w[0] = v.x; w[1] = v.y;
  } else {
#pragma unroll
    for (int i = 0; i < WORDS; ++i) w[i] = __ldg(reinterpret_cast<const uint32_t *>(p) + i);
  }
#pragma unroll
  for (int i = 0; i < WORDS; ++i) w[i] = __byte_perm(w[i], 0, 0x0123);
}

// level of coordinate k (k*BITS bits from the top of w[0]); k is a constant after unrolling
template <int BITS, int WORDS> __device__ __forceinline__ uint32_t level_of(const uint32_t (&w)[WORDS], int k) {
  const int o = k * BITS, wi = o >> 5, sh = o & 31;
  if (sh + BITS <= 32) return (w[wi] >> (32 - BITS - sh)) & ((1u << BITS) - 1u);
  return __funnelshift_l(w[wi + 1 < WORDS ? wi + 1 : wi], w[wi], sh) >> (32 - BITS);
}

// One thread scores one packed K row against the table lut[j * 2^BITS + level]: the lanes of
// a warp read the same j with their own levels, i.e. words of one 2^BITS-word segment, which
// never collide in a bank.
template <int BITS> __device__ __forceinline__ float score_row_words(const uint8_t *kr, const float *lut, int P) {
  constexpr int L = 1 << BITS;
  float s0 = 0.f, s1 = 0.f;
  for (int g = 0; g < P / 32; ++g) {
    uint32_t w[BITS];
    load_words_be<BITS>(kr + g * 4 * BITS, w);
    const float *lt = lut + (size_t)g * 32 * L;
#pragma unroll
    for (int k = 0; k < 32; k += 2) {
      s0 += lt[k * L + level_of<BITS, BITS>(w, k)];
      s1 += lt[(k + 1) * L + level_of<BITS, BITS>(w, k + 1)];
    }
  }
  return s0 + s1;
}

// V rows by words: a thread owns one unit of a row (one word at 2 or 4 bits, three words = 32
// coordinates at 3 bits) for every token of its token group.
template <int BITS> struct VUnit {
  static constexpr int WORDS = BITS == 3 ? 3 : 1;
  static constexpr int NCO = WORDS * 32 / BITS; // coordinates per unit: 16 / 32 / 8
};

template <int BITS>
__device__ __forceinline__ void v_accumulate_words(float *acc, float rescale, const uint8_t *vunit, int v_row, const float *sc, int cn,
                                                   int tg, int TG, const float *s_cb) {
  using U = VUnit<BITS>;
#pragma unroll
  for (int k = 0; k < U::NCO; ++k) acc[k] *= rescale;
#pragma unroll 2
  for (int i = tg; i < cn; i += TG) {
    uint32_t w[U::WORDS];
    load_words_be<U::WORDS>(vunit + (size_t)i * v_row, w);
    const float wt = sc[i];
#pragma unroll
    for (int k = 0; k < U::NCO; ++k) acc[k] += wt * s_cb[level_of<BITS, U::WORDS>(w, k)];
  }
}

// Sum the token groups' accumulators into vec[P]: lanes that hold the same unit first (shuffles),
// then one row per warp (or per token group when a row has more than 32 units) through `buf`.
template <int BITS, int THREADS> __device__ __forceinline__ void v_fold_words(float *acc, int P, float *buf, float *vec) {
  using UU = VUnit<BITS>;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int U = P / UU::NCO; // units per row, a power of two
  if (U < 32) {
    for (int off = U; off < 32; off <<= 1) {
#pragma unroll
      for (int k = 0; k < UU::NCO; ++k) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], off);
    }
  }
  const int rows = U <= 32 ? THREADS / 32 : THREADS / U;
  const int row = U <= 32 ? warp : tid / U;
  const int u = tid % U;
  if (U >= 32 || lane < U) {
#pragma unroll
    for (int k = 0; k < UU::NCO; ++k) buf[(size_t)row * P + u * UU::NCO + k] = acc[k];
  }
  __syncthreads();
  for (int j = tid; j < P; j += THREADS) {
    float t = 0.f;
    for (int r = 0; r < rows; ++r) t += buf[(size_t)r * P + j];
    vec[j] = t;
  }
}

__device__ __forceinline__ float block_reduce(float v, float *red, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
  for (int i = 1; i < CG_WARPS; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
  return r;
}

// Merge n_parts split-KV partials per (head, query): rescale to the common
// max, sum, normalise, one inverse transform.  parts laid out
// [n_parts][items][2+P] with part stride `part_stride` floats.
// One block (CG_THREADS threads) merges the n_parts partials of `item`; vec: P floats of shared memory.
// Partials are read past L1 (__ldcg): other blocks of the same launch may have written them.
//
// Non-finite values travel as they do upstream (attention/attention.cpp:422-429 has no
// guard): a part whose sum is NaN makes the result NaN, a part whose weight underflows
// to zero still contributes 0 * acc.  Only a part marked empty -- max == -inf, which no
// span with tokens produces because the running maximum starts at -1e30f as upstream's
// does -- is skipped (its accumulator was never written).  guard_n > 0 selects the
// hybrid window's rule (attention.cpp:513): a sum that is zero or not finite is
// replaced by guard_n, i.e. the weights become exp(..)/n.
__device__ __forceinline__ void merge_partials_block(const float *parts, size_t part_stride, int n_parts, const CacheView &c,
                                                     int item, int h, float *out, int v_f32, int to_partial, float *vec,
                                                     int guard_n) {
  const int P = c.padded, dim = c.dim;
  const int tid = threadIdx.x;
  const float *base = parts + (size_t)item * (2 + P);
  // All loads of a step are independent of each other, so their latencies
  // overlap: the (max, sum) pairs are read one part per thread, the
  // accumulators with the parts dealt round-robin to thread groups.
  __shared__ float s_w[1024];        // weight exp(m_p - M) of the first 1024 parts; -1 marks an empty part
  __shared__ float s_red[CG_WARPS];
  __shared__ float s_grp[CG_THREADS];
  const int lane = tid & 31, warp = tid >> 5;
  float m_loc = -INFINITY;
  for (int p = tid; p < n_parts; p += CG_THREADS) m_loc = fmaxf(m_loc, __ldcg(base + (size_t)p * part_stride));
  m_loc = warp_max(m_loc);
  if (lane == 0) s_red[warp] = m_loc;
  __syncthreads();
  float M = s_red[0];
  for (int w = 1; w < CG_WARPS; ++w) M = fmaxf(M, s_red[w]);
  __syncthreads();
  float l_loc = 0.f;
  for (int p = tid; p < n_parts; p += CG_THREADS) {
    const float *pp = base + (size_t)p * part_stride;
    const float m = __ldcg(pp);
    const bool live = m != -INFINITY;
    const float w = live ? expf(m - M) : -1.f;
    if (p < 1024) s_w[p] = w;
    if (live) l_loc += __ldcg(pp + 1) * w;
  }
  l_loc = warp_sum(l_loc);
  if (lane == 0) s_red[warp] = l_loc;
  __syncthreads(); // also publishes s_w
  float L = 0.f;
  for (int w = 0; w < CG_WARPS; ++w) L += s_red[w];
  float invL = 1.f / L;
  if (guard_n > 0 && !(L > 0.f && L < INFINITY)) invL = 1.f / (float)guard_n;
  if (to_partial) invL = 1.f;
  if (M == -INFINITY) invL = 0.f; // every part is empty: zeros, as for an empty cache
  auto weight = [&](int p) -> float {
    if (p < 1024) return s_w[p];
    const float m = __ldcg(base + (size_t)p * part_stride);
    return m != -INFINITY ? expf(m - M) : -1.f;
  };
  if (P <= CG_THREADS) {
    const int groups = CG_THREADS / P, g = tid / P, j = tid % P;
    float s = 0.f;
    if (g < groups) {
#pragma unroll 8
      for (int p = g; p < n_parts; p += groups) {
        const float w = weight(p);
        if (w != -1.f) s += __ldcg(base + (size_t)p * part_stride + 2 + j) * w;
      }
    }
    s_grp[tid] = s;
    __syncthreads();
    if (tid < P) {
      float t = 0.f;
      for (int gg = 0; gg < groups; ++gg) t += s_grp[gg * P + tid];
      vec[tid] = t * invL;
    }
  } else {
    for (int j = tid; j < P; j += CG_THREADS) {
      float s = 0.f;
#pragma unroll 8
      for (int p = 0; p < n_parts; ++p) {
        const float w = weight(p);
        if (w != -1.f) s += __ldcg(base + (size_t)p * part_stride + 2 + j) * w;
      }
      vec[j] = s * invL;
    }
  }
  __syncthreads();
  if (to_partial) { // one combined, still un-normalised partial per (head, query)
    float *po = out + (size_t)item * (2 + P);
    if (tid == 0) { po[0] = M; po[1] = L; }
    for (int j = tid; j < P; j += CG_THREADS) po[2 + j] = vec[j];
    return;
  }
  float *o = out + (size_t)item * dim;
  if (v_f32) {
    for (int j = tid; j < dim; j += CG_THREADS) o[j] = vec[j];
    return;
  }
  block_butterflies(vec, P);
  const uint32_t *sg = c.signs + (size_t)h * c.sign_words;
  const float isp = 1.f / sqrtf((float)P);
  for (int j = tid; j < dim; j += CG_THREADS) o[j] = vec[j] * isp * sign_of(sg, j);
}

__global__ void __launch_bounds__(CG_THREADS) merge_partials_kernel(
    const float *parts, size_t part_stride, int n_parts, CacheView c, int head0, int nq, float *out,
    int v_f32, int to_partial, int guard_n) {
  extern __shared__ __align__(16) unsigned char smem_gen[];
  const int item = blockIdx.x; // hl*nq + qi
  merge_partials_block(parts, part_stride, n_parts, c, item, head0 + item / nq, out, v_f32, to_partial,
                       reinterpret_cast<float *>(smem_gen), guard_n);
}

// KW / VW: the packed keys / values are read by words (quantised, padded dimension a multiple
// of 32); otherwise by bytes or as floats.
template <bool KW, bool VW>
__global__ void __launch_bounds__(CG_THREADS) compute_general_kernel(const ComputeLaunch a) {
  extern __shared__ __align__(128) unsigned char smem_gen[];
  unsigned char *smem_raw = smem_gen;
  const CacheView &c = a.c;
  const int P = c.padded, dim = c.dim;
  const int split = blockIdx.x, hl = blockIdx.y, qi = blockIdx.z;
  const int h = a.head0 + hl;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  const bool mirror = a.use_mirror != 0;
  const bool k_f32 = mirror || c.k_bits == 16;
  const bool v_f32 = mirror || c.v_bits == 16;
  const int kcb = k_f32 ? 0 : (1 << c.k_bits);

  float *qr = reinterpret_cast<float *>(smem_raw);
  float *vec = qr + P;
  float *red = vec + P;
  float *s_vcb = red + 64;
  float *lut = s_vcb + 16;
  float *sc = lut + (size_t)P * kcb;

  const float *q = a.q + ((size_t)hl * a.nq + qi) * dim;
  const uint32_t *sg = c.signs + (size_t)h * c.sign_words;

  // ---- query: raw for FP32 keys, rotated for quantised keys ---------------
  for (int i = tid; i < P; i += CG_THREADS) qr[i] = i < dim ? q[i] : 0.f;
  __syncthreads();
  float attn_s = 1.f / sqrtf((float)dim);
  const float isp = 1.f / sqrtf((float)P);
  if (!k_f32) {
    float part = 0.f;
    for (int i = tid; i < dim; i += CG_THREADS) part += qr[i] * qr[i];
    float qn = sqrtf(block_reduce(part, red, false) + 1e-12f);
    float inv = 1.f / qn;
    for (int i = tid; i < P; i += CG_THREADS) qr[i] = qr[i] * inv * sign_of(sg, i);
    __syncthreads();
    block_butterflies(qr, P);
    const float m = sqrtf((float)P) * qn;
    for (int i = tid; i < P; i += CG_THREADS) qr[i] = qr[i] * isp * m;
    __syncthreads();
    attn_s = 1.f / (sqrtf((float)dim) * (float)P);
    const float *cb = c_cb[c.k_bits - 2];
    if constexpr (KW) { // table[j][level]: a warp's lanes (one token each) read one segment per j
      for (int i = tid; i < P * kcb; i += CG_THREADS) lut[i] = qr[i / kcb] * cb[i % kcb];
    } else { // table[level][j] = q_rot[j] * centroid[level]; column j sits in bank j%32
      for (int i = tid; i < P * kcb; i += CG_THREADS) lut[i] = qr[i % P] * cb[i / P];
    }
    __syncthreads();
  }
  if constexpr (VW) {
    if (tid < 16) s_vcb[tid] = tid < (1 << c.v_bits) ? c_cb[c.v_bits - 2][tid] : 0.f;
    // visible after the first barrier of the token loop
  }

  const uint8_t *kbase = c.k_slab + (size_t)h * c.k_stride;
  const uint8_t *vbase = c.v_slab + (size_t)h * c.v_stride;
  const float *ksc = c.k_scale + (size_t)h * c.s_stride;
  const float *vsc = c.v_scale + (size_t)h * c.s_stride;
  const float *mir = mirror ? c.mirror + (size_t)h * c.mirror_stride : nullptr;

  griddep_wait(); // the cache (rows, scales, FP32 window) is read from here on
  int t_begin = min(a.n, split * a.span), t_end = min(a.n, t_begin + a.span);
  if (!AQ_CHECK(a.status, t_end <= c.cap && h >= 0 && h < c.n_heads, 12)) t_begin = t_end = 0; // nothing is read

  // Each thread owns output columns j = jcol + r*CG_THREADS of token group tg.
  const int TG = P < CG_THREADS ? CG_THREADS / P : 1;
  const int jcol = P < CG_THREADS ? tid % P : tid;
  const int tg = P < CG_THREADS ? tid / P : 0;
  constexpr int MAXR = 4; // P <= 1024
  float acc[MAXR] = {0.f, 0.f, 0.f, 0.f};
  // by words: unit vu of token group vtg, up to 32 coordinates per thread
  float accw[VW ? 32 : 1];
#pragma unroll
  for (int k = 0; k < (VW ? 32 : 1); ++k) accw[k] = 0.f;
  const int v_nco = c.v_bits == 2 ? 16 : c.v_bits == 3 ? 32 : 8;
  const int VU = VW ? P / v_nco : 1, vu = tid % VU, vtg = tid / VU, VTG = CG_THREADS / VU;
  // the running maximum starts where upstream's does (attention.cpp:384, :498, :566): logits
  // below it (or NaN) never become the maximum, and their weights come out as upstream's do
  float run_m = -1e30f, run_l = 0.f;
  const float *vcb = v_f32 ? nullptr : c_cb[c.v_bits - 2];

  for (int t0 = t_begin; t0 < t_end; t0 += a.chunk) {
    const int cn = min(a.chunk, t_end - t0);
    // ---- scores ----------------------------------------------------------
    if constexpr (KW) {
      for (int i = tid; i < cn; i += CG_THREADS) {
        const int s = t0 + i;
        const uint8_t *kr = kbase + (size_t)s * c.k_row;
        const float sum = c.k_bits == 4 ? score_row_words<4>(kr, lut, P)
                          : c.k_bits == 3 ? score_row_words<3>(kr, lut, P) : score_row_words<2>(kr, lut, P);
        sc[i] = sum * attn_s * ksc[s];
      }
    } else if (k_f32 && !mirror && (dim & 3) == 0) {
      // FP32 key rows (16-byte aligned): one thread per token, the whole row in flight at once
      const float4 *q4 = reinterpret_cast<const float4 *>(qr);
      for (int i = tid; i < cn; i += CG_THREADS) {
        const float4 *kr = reinterpret_cast<const float4 *>(kbase + (size_t)(t0 + i) * c.k_row);
        float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
        for (int j = 0; j < dim / 4; ++j) {
          const float4 kv = __ldg(kr + j), qv = q4[j];
          s0 += qv.x * kv.x + qv.y * kv.y;
          s1 += qv.z * kv.z + qv.w * kv.w;
        }
        sc[i] = (s0 + s1) * attn_s;
      }
    } else {
#pragma unroll 4
      for (int i = warp; i < cn; i += CG_WARPS) {
        const int s = t0 + i;
        float sum = 0.f;
        if (k_f32) {
          const float *kr = mirror ? mir + (size_t)s * 2 * dim : reinterpret_cast<const float *>(kbase + (size_t)s * c.k_row);
          for (int j = lane; j < dim; j += 32) sum += qr[j] * kr[j];
        } else {
          const uint8_t *kr = kbase + (size_t)s * c.k_row;
          for (int j = lane; j < P; j += 32) sum += lut[unpack_at(kr, j, c.k_bits) * P + j];
        }
        sum = warp_sum(sum);
        if (lane == 0) sc[i] = k_f32 ? sum * attn_s : sum * attn_s * ksc[s];
      }
    }
    __syncthreads();
    if (a.mode == 2) { // raw logits out, stored by LOGICAL position (oldest token first, as upstream
      // walks them, attention.cpp:562-563) so that the later sort breaks ties the same way
      float *w = a.weights + ((size_t)hl * a.nq + qi) * a.w_stride;
      for (int i = tid; i < cn; i += CG_THREADS) {
        int pos = t0 + i - a.rot;
        if (pos < 0) pos += c.cap;
        w[pos] = sc[i];
      }
      __syncthreads();
      continue;
    }
    // ---- online softmax over this pass -------------------------------------
    float mx = -INFINITY;
    for (int i = tid; i < cn; i += CG_THREADS) mx = fmaxf(mx, sc[i]);
    mx = block_reduce(mx, red, true);
    const float new_m = fmaxf(run_m, mx);
    const float rescale = expf(run_m - new_m);
    float ls = 0.f;
    for (int i = tid; i < cn; i += CG_THREADS) {
      float e = expf(sc[i] - new_m);
      ls += e;
      // fold the per-token V factor in once: w * vscale * (1/sqrt p)
      sc[i] = v_f32 ? e : e * vsc[t0 + i] * isp;
    }
    ls = block_reduce(ls, red, false);
    run_l = run_l * rescale + ls;
    run_m = new_m;
    __syncthreads();
    // ---- V accumulation ------------------------------------------------------
    if constexpr (VW) {
      const uint8_t *vunit = vbase + (size_t)t0 * c.v_row + (size_t)vu * (c.v_bits == 3 ? 12 : 4);
      if (c.v_bits == 2) v_accumulate_words<2>(accw, rescale, vunit, c.v_row, sc, cn, vtg, VTG, s_vcb);
      else if (c.v_bits == 3) v_accumulate_words<3>(accw, rescale, vunit, c.v_row, sc, cn, vtg, VTG, s_vcb);
      else v_accumulate_words<4>(accw, rescale, vunit, c.v_row, sc, cn, vtg, VTG, s_vcb);
    } else {
#pragma unroll
      for (int r = 0; r < MAXR; ++r) {
        const int j = jcol + r * CG_THREADS;
        if (j >= P || (P < CG_THREADS && r > 0)) break;
        float av = acc[r] * rescale;
#pragma unroll 4
        for (int i = tg; i < cn; i += TG) {
          const int s = t0 + i;
          if (v_f32) {
            if (j < dim) {
              const float *vr = mirror ? mir + (size_t)s * 2 * dim + dim : reinterpret_cast<const float *>(vbase + (size_t)s * c.v_row);
              av += sc[i] * vr[j];
            }
          } else {
            av += sc[i] * vcb[unpack_at(vbase + (size_t)s * c.v_row, j, c.v_bits)];
          }
        }
        acc[r] = av;
      }
    }
    __syncthreads();
  }
  if (a.mode == 2) return;

  // ---- fold token groups ------------------------------------------------------
  // vec[j] = sum over token groups; TG groups of P columns fit CG_THREADS exactly
  if constexpr (VW) { // sc holds at least 8*P floats (the host sizes it)
    if (c.v_bits == 2) v_fold_words<2, CG_THREADS>(accw, P, sc, vec);
    else if (c.v_bits == 3) v_fold_words<3, CG_THREADS>(accw, P, sc, vec);
    else v_fold_words<4, CG_THREADS>(accw, P, sc, vec);
  } else if (P < CG_THREADS) {
    float *fold = sc; // chunk >= CG_THREADS floats is guaranteed by the host
    fold[tid] = acc[0];
    __syncthreads();
    if (tid < P) {
      float s = 0.f;
      for (int g = 0; g < TG; ++g) s += fold[g * P + tid];
      vec[tid] = s;
    }
  } else {
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
      const int j = jcol + r * CG_THREADS;
      if (j < P) vec[j] = acc[r];
    }
  }
  __syncthreads();

  if (a.mode == 1) {
    const int item = hl * a.nq + qi;
    const size_t part_stride = (size_t)a.heads_in_call * a.nq * (size_t)(2 + P);
    float *pp = a.partial + (size_t)split * part_stride + (size_t)item * (size_t)(2 + P);
    if (!AQ_CHECK(a.status, split < a.n_splits && item < a.heads_in_call * a.nq, 14)) return;
    if (tid == 0) { pp[0] = run_m; pp[1] = run_l; }
    for (int j = tid; j < P; j += CG_THREADS) pp[2 + j] = vec[j];
    if (a.counters == nullptr) return;
    // The block that brings an item's count to n_splits merges its partials (no block
    // ever waits for another one); it also puts the count back to zero for the next launch.
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&a.counters[item], 1) == a.n_splits - 1 ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    if (tid == 0) a.counters[item] = 0;
    __threadfence();
    merge_partials_block(a.partial, part_stride, a.n_splits, c, item, h, a.final_out, v_f32 ? 1 : 0, a.final_to_partial, vec,
                         mirror ? a.n : 0);
    return;
  }
  // ---- normalise, inverse transform, write ----------------------------------------
  // the hybrid window replaces a zero or non-finite sum by n (attention.cpp:513); the other
  // branches divide by whatever the sum is (:428, :582)
  const float invl = (mirror && !(run_l > 0.f && run_l < INFINITY)) ? 1.f / (float)a.n : 1.f / run_l;
  float *o = a.out + ((size_t)hl * a.nq + qi) * dim;
  if (v_f32) {
    for (int j = tid; j < dim; j += CG_THREADS) o[j] = vec[j] * invl;
    return;
  }
  for (int j = tid; j < P; j += CG_THREADS) vec[j] *= invl;
  __syncthreads();
  block_butterflies(vec, P);
  for (int j = tid; j < dim; j += CG_THREADS) o[j] = vec[j] * isp * sign_of(sg, j);
}

// Tail of merge_peers_kernel for P = 32*EPL: weighted sum of the ranks' accumulators,
// normalisation, inverse transform (core/fwht.cpp:106-134) and store, all in one warp.
template <int EPL>
__device__ __forceinline__ void peers_finish(const float *base, size_t part_stride, int world, float w_p, float invL, float isp,
                                             const uint32_t *sg, int dim, int lane, float *o) {
  float v[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) v[e] = 0.f;
  for (int r = 0; r < world; ++r) {
    const float w = __shfl_sync(0xffffffffu, w_p, r);
    if (w != -1.f) { // -1 marks a rank without tokens
#pragma unroll
      for (int e = 0; e < EPL; ++e) v[e] += w * __ldcg(base + (size_t)r * part_stride + 2 + EPL * lane + e);
    }
  }
#pragma unroll
  for (int e = 0; e < EPL; ++e) v[e] *= invL;
  warp_butterflies<EPL>(v, lane);
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int j = EPL * lane + e;
    if (j < dim) o[j] = v[e] * isp * sign_of(sg, j);
  }
}

// Merge of partials that PEER GPUs store into this GPU's gather buffer
// (parts laid out [world][items][2+P]).  Rank r's kernel adds 1 to flags[r] (system
// scope, with release semantics) for every item it has delivered; `expected` is the
// running total this step must reach.  The wait is bounded: if a peer's count does
// not arrive within AQ_WAIT_BUDGET_NS the warp records status 3, writes zeros and
// returns, so a lost peer costs an error code, never a hang.
__global__ void __launch_bounds__(128) merge_peers_kernel(
    const float *parts, size_t part_stride, int world, const unsigned int *flags, unsigned int expected, int *status,
    CacheView c, int head0, int nq, int items, float *out) {
  // one warp per (head, query): at most 8 partials of at most 1024 floats, no block barriers
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const int P = c.padded, dim = c.dim;
  int ok = 1;
  if (lane < world) {
    unsigned int seen = 0;
    unsigned long long t0 = 0;
    for (int spins = 0;; ++spins) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + lane) : "memory");
      if ((int)(seen - expected) >= 0) break;       // counts only grow; compare modulo 2^32
      if (spins == 0) t0 = global_ns();
      else if (global_ns() - t0 > AQ_WAIT_BUDGET_NS) { ok = 0; break; }
      __nanosleep(100);
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  float *o = out + (size_t)item * dim;
  if (!ok) {
    if (lane == 0) atomicExch(status, 3);
    for (int j = lane; j < dim; j += 32) o[j] = 0.f;
    return;
  }
  const float *base = parts + (size_t)item * (2 + P);
  // same rules as merge_partials_block: only a rank that delivered (-inf, 0) is skipped
  float m_p = -INFINITY, l_p = 0.f;
  if (lane < world) {
    m_p = __ldcg(base + (size_t)lane * part_stride);
    l_p = __ldcg(base + (size_t)lane * part_stride + 1);
  }
  const float M = warp_max(m_p);
  const bool live = m_p != -INFINITY;
  const float w_p = live ? expf(m_p - M) : -1.f;
  const float L = warp_sum(live ? l_p * w_p : 0.f);
  const float invL = M == -INFINITY ? 0.f : 1.f / L;
  const uint32_t *sg = c.signs + (size_t)(head0 + item / nq) * c.sign_words;
  const float isp = 1.f / sqrtf((float)P);
  // the usual sizes: in registers, butterflies with shuffles (lane l owns elements EPL*l .. EPL*l+EPL-1)
  if (P == 128) { peers_finish<4>(base, part_stride, world, w_p, invL, isp, sg, dim, lane, o); return; }
  if (P == 64) { peers_finish<2>(base, part_stride, world, w_p, invL, isp, sg, dim, lane, o); return; }
  // other padded sizes: through this warp's slice of shared memory
  extern __shared__ __align__(16) unsigned char smem_gen[];
  float *vec = reinterpret_cast<float *>(smem_gen) + (size_t)(threadIdx.x >> 5) * P;
  for (int j = lane; j < P; j += 32) {
    float sacc = 0.f;
    for (int r = 0; r < world; ++r) {
      const float w = __shfl_sync(0xffffffffu, w_p, r);
      if (w != -1.f) sacc += w * __ldcg(base + (size_t)r * part_stride + 2 + j);
    }
    vec[j] = sacc * invL;
  }
  __syncwarp();
  for (int len = 1; len < P; len <<= 1) {
    for (int t = lane; t < (P >> 1); t += 32) {
      const int i = ((t / len) * (len << 1)) + (t % len);
      const float x = vec[i], y = vec[i + len];
      vec[i] = x + y;
      vec[i + len] = x - y;
    }
    __syncwarp();
  }
  for (int j = lane; j < dim; j += 32) o[j] = vec[j] * isp * sign_of(sg, j);
}

// ---------------------------------------------------------------------------
// Sparse V (upstream attention/attention.cpp:448-473): the heaviest softmax
// weights are accumulated, four at a time, until their running mass reaches
// v_mass; the weights are not renormalised.
// Step 1 (this kernel): logits -> weights e*(1/sum) in place, plus the token
// index list for the sort.  One block per (head, query).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(CG_THREADS) softmax_weights_kernel(float *weights, int *order, int w_stride, int n,
                                                                     int rot, int cap) {
  __shared__ float red[64];
  float *w = weights + (size_t)blockIdx.x * w_stride;
  int *o = order + (size_t)blockIdx.x * w_stride;
  const int tid = threadIdx.x;
  float mx = -1e30f;
  for (int i = tid; i < n; i += CG_THREADS) mx = fmaxf(mx, w[i]);
  mx = block_reduce(mx, red, true);
  float s = 0.f;
  for (int i = tid; i < n; i += CG_THREADS) {
    float e = expf(w[i] - mx);
    w[i] = e;
    s += e;
  }
  s = block_reduce(s, red, false);
  const float inv = 1.f / s;
  for (int i = tid; i < n; i += CG_THREADS) {
    w[i] *= inv;
    o[i] = i + rot < cap ? i + rot : i + rot - cap; // logical position -> ring slot
  }
}

// Step 3 (after a stable descending sort of (weight, token) per block):
// find the cut exactly as upstream does -- blocks of four while four remain
// and the mass is short, then singles -- and accumulate those V rows.
__global__ void __launch_bounds__(CG_THREADS) sparse_accumulate_kernel(
    const float *sorted_w, const int *sorted_tok, int w_stride, int n, CacheView c, int head0, int nq, float *out) {
  extern __shared__ __align__(16) unsigned char smem_gen[];
  unsigned char *smem_raw = smem_gen;
  float *vec = reinterpret_cast<float *>(smem_raw);
  __shared__ int s_count;
  const int P = c.padded, dim = c.dim;
  const int item = blockIdx.x;
  const int h = head0 + item / nq;
  const int tid = threadIdx.x;
  const float *w = sorted_w + (size_t)item * w_stride;
  const int *tok = sorted_tok + (size_t)item * w_stride;
  if (tid == 0) {
    float mass = 0.f;
    int ii = 0;
    if (c.sparse_block == 4)
      for (; ii + 3 < n && mass < c.v_mass; ii += 4)
        mass = __fadd_rn(mass, __fadd_rn(__fadd_rn(__fadd_rn(w[ii], w[ii + 1]), w[ii + 2]), w[ii + 3]));
    for (; ii < n && mass < c.v_mass; ++ii) mass = __fadd_rn(mass, w[ii]);
    s_count = ii;
  }
  __syncthreads();
  const int count = s_count;
  const uint8_t *vbase = c.v_slab + (size_t)h * c.v_stride;
  const float *vsc = c.v_scale + (size_t)h * c.s_stride;
  const float *vcb = c_cb[c.v_bits - 2];
  const float isp = 1.f / sqrtf((float)P);
  for (int j = tid; j < P; j += CG_THREADS) {
    float av = 0.f;
    for (int i = 0; i < count; ++i) {
      const int s = tok[i];
      av += (w[i] * vsc[s] * isp) * vcb[unpack_at(vbase + (size_t)s * c.v_row, j, c.v_bits)];
    }
    vec[j] = av;
  }
  __syncthreads();
  block_butterflies(vec, P);
  const uint32_t *sg = c.signs + (size_t)h * c.sign_words;
  float *o = out + (size_t)item * dim;
  for (int j = tid; j < dim; j += CG_THREADS) o[j] = vec[j] * isp * sign_of(sg, j);
}

} // namespace aq
