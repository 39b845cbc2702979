// Append kernels: FP32 vector -> (sign flip, Walsh-Hadamard, Lloyd-Max
// quantisation, MSB-first bit packing) -> ring slot of the device cache.
//
// Replaces upstream AttentionHead::append_kv (attention/attention.cpp:338-366),
// Quantizer::quantize_into / _quantize_core (core/quantizer.cpp:53-137),
// fwht_forward (core/fwht.cpp:33-104), quantize_fast (core/codebook.cpp:119-144),
// pack_indices (core/quantizer.cpp:156-225) and KVFlatBuffer::insert
// (cache/ring_buffer.cpp:105-119).
//
// Bit-exactness: every floating-point step is issued as an individually
// rounded IEEE operation in upstream's order (no FMA contraction): the norm
// and the clip's sum of squares are strictly sequential chains over the
// index, the butterflies run in stage order len = 1, 2, ... p/2, and the two
// scalings by 1/sqrt(p) and sqrt(p) stay separate multiplies.
#pragma once
#include "common.cuh"

namespace aq {

struct AppendLaunch {
  CacheView c;
  const float *src; // token t, head head0+i at  src + t*src_token_stride + i*dim
  size_t src_token_stride; // floats between consecutive tokens
  int which;        // 0 = keys, 1 = values
  int head0, heads_in_call, n_tokens;
  int ring_head, ring_size, mirror_cnt; // state shared by the heads of this call
  int head_major;
  int contig;       // items are token-major and item g starts at src + g*dim (one contiguous block)
  int *status;
  // exact division of 32-bit values by the item divisor (n_tokens when head_major,
  // else heads_in_call) and by the ring capacity: q = umulhi(x, magic) >> shift
  // after adding `add` (round-up variant), filled in by the host
  uint32_t div_magic, div_shift, div_add;
  uint32_t cap_magic, cap_shift, cap_add;
  float sqrt_p, inv_sqrt_p; // sqrtf(padded) and 1/sqrtf(padded), IEEE-rounded on the host
};

struct ItemPlace {
  bool store;  // write the packed row + scale
  bool mirror; // write the FP32 mirror row
  int h, t, slot;
};

// Where does work item g go?  Tokens that a later token of the same call
// overwrites (n_tokens > capacity) are dropped, which keeps the parallel
// writes race-free and matches the FIFO end state.
__device__ __forceinline__ ItemPlace place_item(const AppendLaunch &a, long long g) {
  ItemPlace p;
  int hl;
  if (a.head_major) {
    hl = (int)(g / a.n_tokens);
    p.t = (int)(g % a.n_tokens);
  } else {
    p.t = (int)(g / a.heads_in_call);
    hl = (int)(g % a.heads_in_call);
  }
  p.h = a.head0 + hl;
  const int cap = a.c.cap, T = a.n_tokens;
  p.store = cap > 0 && p.t >= T - cap;
  p.slot = cap > 0 ? (int)(((long long)a.ring_head + p.t) % cap) : 0;
  // Mirror rule of upstream attention/attention.cpp:354-365: push while the
  // ring has not started evicting and the mirror is short of hybrid_thresh;
  // the first eviction clears it, so a call that ends past capacity writes none.
  bool call_evicts = (long long)a.ring_size + T > cap;
  p.mirror = a.c.hyb > 0 && !call_evicts && (a.mirror_cnt + p.t < a.c.hyb);
  return p;
}

// x / d for x < 2^31 with the host-computed (magic, shift, add) of d.
__device__ __forceinline__ uint32_t fast_div(uint32_t x, uint32_t magic, uint32_t shift, uint32_t add) {
  return __umulhi(x + add, magic) >> shift;
}

// Same as place_item with 32-bit arithmetic and multiply-shift divisions (the
// tile kernel is only used below 2^31 items).
__device__ __forceinline__ ItemPlace place_item32(const AppendLaunch &a, uint32_t g) {
  ItemPlace p;
  uint32_t hl;
  const uint32_t q = fast_div(g, a.div_magic, a.div_shift, a.div_add);
  if (a.head_major) {
    hl = q;
    p.t = (int)(g - q * (uint32_t)a.n_tokens);
  } else {
    p.t = (int)q;
    hl = g - q * (uint32_t)a.heads_in_call;
  }
  p.h = a.head0 + (int)hl;
  const int cap = a.c.cap, T = a.n_tokens;
  p.store = cap > 0 && p.t >= T - cap;
  const uint32_t pos = (uint32_t)a.ring_head + (uint32_t)p.t;
  p.slot = cap > 0 ? (int)(pos - fast_div(pos, a.cap_magic, a.cap_shift, a.cap_add) * (uint32_t)cap) : 0;
  const bool call_evicts = (long long)a.ring_size + T > cap;
  p.mirror = a.c.hyb > 0 && !call_evicts && (a.mirror_cnt + p.t < a.c.hyb);
  return p;
}

__device__ __forceinline__ const float *item_src(const AppendLaunch &a, const ItemPlace &p) {
  return a.src + (size_t)p.t * a.src_token_stride + (size_t)(p.h - a.head0) * a.c.dim;
}

// ---------------------------------------------------------------------------
// Building blocks of the tile kernel (register-resident path).
// ---------------------------------------------------------------------------

// Threshold search through a shared-memory table indexed by floor(4v) + 64: the
// 128 buckets [k/4, (k+1)/4), k = -64..63, cover |v| < 16 (transformed
// coordinates of a unit vector never exceed sqrt(p) <= 11.4 in magnitude).  No
// bucket holds more than one decision threshold of the 2-, 3- or 4-bit
// codebooks, so an entry is {that threshold, or +inf; number of thresholds
// below the bucket}, and
//   index = entry.count + (v >= entry.threshold)
// is upstream's binary search with its `v >= t` decisions
// (core/codebook.cpp:119-144) for every finite v in range, including -0.0
// (4*(-0.0) + C rounds to C, i.e. to the bucket that holds the exact 0).
constexpr int QT_ENTRIES = 128;

template <int BITS> __device__ __forceinline__ void build_quant_table(uint2 *qtab, int tid, int nthreads) {
  constexpr int NT = (1 << BITS) - 1; // thresholds, ascending
  for (int e = tid; e < QT_ENTRIES; e += nthreads) {
    const float lo = 0.25f * (float)(e - 64), hi = 0.25f * (float)(e - 63);
    uint32_t below = 0;
    float thr = INFINITY;
    for (int j = 0; j < NT; ++j) {
      const float t = c_thr[BITS - 2][j];
      if (t < lo) ++below;
      else if (t < hi) thr = t;
    }
    qtab[e] = make_uint2(__float_as_uint(thr), below);
  }
}

// The search for one coordinate, with the index added into `word` at bit position SHIFT:
// floor(4v) + 64 lands in the low mantissa bits of 2^23 + 64 + 4v rounded down, the count of
// thresholds below that bucket goes into the word with one multiply-add, and the last
// `v >= t` decision (upstream's comparison, core/codebook.cpp:128-131) with one predicated add.
template <int BITS, uint32_t SHIFT> __device__ __forceinline__ void quantize_into_word(uint32_t &word, float v, uint32_t qtab_addr) {
  const float t = __fmaf_rd(v, 4.0f, 8388608.0f + 64.0f);
  const uint32_t addr = (__float_as_uint(t) << 3) + (qtab_addr - 0x58000000u);
  asm("{\n\t.reg .b32 thr, cnt;\n\t.reg .pred p;\n\t"
      "ld.shared.v2.b32 {thr, cnt}, [%1];\n\t"
      "mad.lo.u32 %0, cnt, %3, %0;\n\t"
      "setp.ge.f32 p, %2, thr;\n\t"
      "@p add.u32 %0, %0, %3;\n\t}"
      : "+r"(word)
      : "r"(addr), "f"(v), "n"(1u << SHIFT));
}

// Bit position of coordinate k of a packed 32-bit word (MSB-first within bytes).
template <int BITS> __device__ __forceinline__ uint32_t index_shift(int k) {
  return BITS == 4 ? (uint32_t)(8 * (k >> 1) + ((k & 1) ? 0 : 4)) : (uint32_t)(8 * (k >> 2) + (6 - 2 * (k & 3)));
}

// Two IEEE round-to-nearest FP32 operations per instruction (sm_100 f32x2, through
// the float2 intrinsics so that the compiler keeps the pairs in aligned registers).
// Each half is rounded exactly like the scalar operation, so results are
// bit-identical to upstream's scalar code; only the issue slots are halved.
__device__ __forceinline__ float2 mulp(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 addp(float2 a, float2 b) { return __fadd2_rn(a, b); }
// a - b as b * (-1) + a: the product is exact, so this rounds once, like the subtraction
__device__ __forceinline__ float2 subp(float2 a, float2 b) { return __ffma2_rn(b, make_float2(-1.0f, -1.0f), a); }
__device__ __forceinline__ float2 fmap(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

// ---------------------------------------------------------------------------
// General routine: one warp per vector, the vector lives in shared memory
// (`buf`, padded floats).  Any dim with padded <= 1024, any alignment, every
// special value.  Same arithmetic as upstream, in upstream's order.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void append_item_general(const AppendLaunch &a, long long g, float *buf, int lane) {
  const CacheView &c = a.c;
  const int P = c.padded, dim = c.dim;
  const int bits = a.which ? c.v_bits : c.k_bits;
  const int rowb = a.which ? c.v_row : c.k_row;
  ItemPlace p = place_item(a, g);
  if (!p.store && !p.mirror) return;
  const float *src = item_src(a, p);
  for (int i = lane; i < P; i += 32) buf[i] = i < dim ? src[i] : 0.f;
  __syncwarp();
  if (p.mirror) {
    float *m = c.mirror + (size_t)p.h * c.mirror_stride + (size_t)p.slot * 2 * dim + (a.which ? dim : 0);
    for (int i = lane; i < dim; i += 32) m[i] = buf[i];
  }
  if (!p.store) { __syncwarp(); return; }
  if (!AQ_CHECK(a.status, p.slot >= 0 && p.slot < c.cap && p.h >= 0 && p.h < c.n_heads, 11)) { __syncwarp(); return; }
  uint8_t *row = (a.which ? c.v_slab : c.k_slab) + (size_t)p.h * (a.which ? c.v_stride : c.k_stride) + (size_t)p.slot * rowb;
  float *scale = (a.which ? c.v_scale : c.k_scale) + (size_t)p.h * c.s_stride + p.slot;
  if (bits == 16) {
    float *dst = reinterpret_cast<float *>(row);
    for (int i = lane; i < P; i += 32) dst[i] = buf[i];
    if (lane == 0) *scale = 1.0f;
    __syncwarp();
    return;
  }
  const uint32_t *sg = c.signs + (size_t)p.h * c.sign_words;
  float norm = 0.f;
  if (lane == 0) {
    for (int i = 0; i < dim; ++i) norm = __fadd_rn(norm, __fmul_rn(buf[i], buf[i]));
    norm = __fsqrt_rn(__fadd_rn(norm, 1e-12f));
  }
  norm = __shfl_sync(0xffffffffu, norm, 0);
  const float inv = __fdiv_rn(1.0f, norm);
  for (int i = lane; i < P; i += 32) buf[i] = __fmul_rn(__fmul_rn(buf[i], inv), sign_of(sg, i));
  __syncwarp();
  for (int len = 1; len < P; len <<= 1) {
    for (int t = lane; t < (P >> 1); t += 32) {
      int i = ((t / len) * (len << 1)) + (t % len);
      float x0 = buf[i], x1 = buf[i + len];
      buf[i] = __fadd_rn(x0, x1);
      buf[i + len] = __fsub_rn(x0, x1);
    }
    __syncwarp();
  }
  const float sq = __fsqrt_rn((float)P), isq = __fdiv_rn(1.0f, sq);
  for (int i = lane; i < P; i += 32) buf[i] = __fmul_rn(__fmul_rn(buf[i], isq), sq);
  __syncwarp();
  float clip = 0.f;
  if (lane == 0) { // +-3 sigma clip, core/quantizer.cpp:81-89
    float sum2 = 0.f;
    for (int i = 0; i < P; ++i) sum2 = __fadd_rn(sum2, __fmul_rn(buf[i], buf[i]));
    clip = __fmul_rn(3.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum2, (float)P), 1e-12f)));
  }
  clip = __shfl_sync(0xffffffffu, clip, 0);
  auto qat = [&](int i) -> uint32_t {
    float v = buf[i];
    if (v > clip) v = clip;
    if (v < -clip) v = -clip;
    return (uint32_t)quantize_value_rt(v, bits);
  };
  if (bits == 4) {
    for (int m = lane; m < P / 2; m += 32) row[m] = (uint8_t)((qat(2 * m) << 4) | qat(2 * m + 1));
  } else if (bits == 2) {
    for (int m = lane; m < P / 4; m += 32)
      row[m] = (uint8_t)((qat(4 * m) << 6) | (qat(4 * m + 1) << 4) | (qat(4 * m + 2) << 2) | qat(4 * m + 3));
  } else {
    for (int g3 = lane; g3 < P / 8; g3 += 32) {
      uint32_t v24 = 0;
      for (int k = 0; k < 8; ++k) v24 |= qat(g3 * 8 + k) << (21 - 3 * k);
      row[g3 * 3] = (uint8_t)(v24 >> 16);
      row[g3 * 3 + 1] = (uint8_t)(v24 >> 8);
      row[g3 * 3 + 2] = (uint8_t)v24;
    }
  }
  if (lane == 0) *scale = norm;
  __syncwarp();
}

constexpr int GEN_WARPS = 4;

__global__ void __launch_bounds__(GEN_WARPS * 32) append_general_kernel(const AppendLaunch a) {
  griddep_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_gen[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float *buf = reinterpret_cast<float *>(smem_gen) + (size_t)warp * a.c.padded;
  const long long n_items = (long long)a.heads_in_call * a.n_tokens;
  for (long long g = (long long)blockIdx.x * GEN_WARPS + warp; g < n_items; g += (long long)gridDim.x * GEN_WARPS)
    append_item_general(a, g, buf, lane);
}

// ---------------------------------------------------------------------------
// Tile kernel.  One block = 512 threads works on tiles of 128 vectors whose
// rows arrive in shared memory through per-row bulk (TMA) copies.
//
//  pass 1  one thread per vector walks its row and forms the L2 norm as the
//          strictly sequential chain upstream computes (the only part that
//          cannot be split across lanes without changing the rounding);
//  pass 2  four lanes share a vector, each holding a contiguous quarter
//          (32 floats at dim 128) in registers: normalise, sign, butterflies
//          -- the first stages inside a lane, the last two across lanes with
//          shuffles, in upstream's stage order --, scaling, table quantiser,
//          bit packing; every lane stores the contiguous 16/12/8 bytes of the
//          packed row that its quarter produces.
//
// 64 data registers per vector quarter instead of 128 per vector is what
// lets 32 warps live on an SM (the arithmetic is a long dependent sequence,
// so it is occupancy that hides its latency).  The next tile's copies are
// issued as soon as every lane has pulled its quarter into registers.  The
// few vectors the table quantiser may not handle (tiny, infinite or NaN
// norms) are listed in pass 1 and redone by the general routine.
// ---------------------------------------------------------------------------
#ifndef AQ_AT_TILE
#define AQ_AT_TILE 64
#endif
constexpr int AT_TILE = AQ_AT_TILE;          // vectors per tile
constexpr int AT_THREADS = 4 * AT_TILE;      // four lanes per vector
#ifndef AQ_AT_BPS
#define AQ_AT_BPS (1024 / (4 * AQ_AT_TILE))
#endif
constexpr int AT_BLOCKS_PER_SM = AQ_AT_BPS;

template <int NBYTES> __device__ __forceinline__ void store_packed(uint8_t *dst, const uint32_t *w) {
  if constexpr (NBYTES == 16) {
    *reinterpret_cast<uint4 *>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  } else if constexpr (NBYTES == 12) {
    uint32_t *d = reinterpret_cast<uint32_t *>(dst);
    d[0] = w[0]; d[1] = w[1]; d[2] = w[2];
  } else if constexpr (NBYTES == 8) {
    *reinterpret_cast<uint2 *>(dst) = make_uint2(w[0], w[1]);
  } else if constexpr (NBYTES == 6) {
    uint16_t *d = reinterpret_cast<uint16_t *>(dst);
    d[0] = (uint16_t)w[0]; d[1] = (uint16_t)(w[0] >> 16); d[2] = (uint16_t)w[1];
  } else {
    static_assert(NBYTES == 4, "unexpected packed slice size");
    *reinterpret_cast<uint32_t *>(dst) = w[0];
  }
}

// One packed 32-bit word from 32/BITS consecutive coordinates (shifts unrolled at compile time).
template <int BITS, int K> __device__ __forceinline__ void quantize_word(uint32_t &word, const float *x, uint32_t qtab_addr) {
  if constexpr (K < 32 / BITS) {
    constexpr uint32_t SH = BITS == 4 ? (uint32_t)(8 * (K >> 1) + ((K & 1) ? 0 : 4)) : (uint32_t)(8 * (K >> 2) + (6 - 2 * (K & 3)));
    quantize_into_word<BITS, SH>(word, x[K], qtab_addr);
    quantize_word<BITS, K + 1>(word, x, qtab_addr);
  }
}

// Quarter-vector transform + quantisation.  xp: this lane's EPL = P/4 contiguous
// coordinates as EPL/2 packed pairs (they stay packed throughout, so the f32x2
// instructions need no register shuffling), sgw = the sign bits of those
// coordinates in bits 0..EPL-1.  Produces EPL*BITS/8 packed bytes in w.
template <int P, int BITS>
__device__ __forceinline__ void quantize_quarter(float2 (&xp)[P / 8], float inv, float sq, float isq,
                                                 uint32_t sgw, int lane, uint32_t (&w)[(P / 4 * BITS + 31) / 32],
                                                 uint32_t qtab_addr) {
  constexpr int EPL = P / 4, NP = EPL / 2;
  const float2 inv2 = make_float2(inv, inv);
  // normalise, Rademacher sign (a sign-bit XOR equals the multiply by +-1), and the
  // len = 1 stage, which pairs the two halves of a register pair (core/fwht.cpp:36-42)
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const float2 n = mulp(xp[i], inv2);
    const float a = __uint_as_float(__float_as_uint(n.x) ^ ((sgw << (31 - 2 * i)) & 0x80000000u));
    const float b = __uint_as_float(__float_as_uint(n.y) ^ ((sgw << (30 - 2 * i)) & 0x80000000u));
    xp[i] = make_float2(__fadd_rn(a, b), __fsub_rn(a, b));
  }
  // stages len = 2 .. EPL/2 stay inside the lane: pairs at distance len/2
#pragma unroll
  for (int hl = 1; hl < NP; hl <<= 1) {
#pragma unroll
    for (int i = 0; i < NP; i += (hl << 1)) {
#pragma unroll
      for (int j = 0; j < hl; ++j) {
        const float2 lo = xp[i + j], hi = xp[i + j + hl];
        xp[i + j] = addp(lo, hi);
        xp[i + j + hl] = subp(lo, hi);
      }
    }
  }
  // stages len = EPL and 2*EPL pair this lane with the lanes 8 and 16 away: the
  // lower quarter keeps a+b, the upper one a-b.  Both are partner + (+-1)*mine in
  // one fused multiply-add, which rounds exactly like the plain add or subtract.
#pragma unroll
  for (int m = 8; m <= 16; m <<= 1) {
    const float sgn = (lane & m) ? -1.0f : 1.0f;
    const float2 sgn2 = make_float2(sgn, sgn);
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const float2 other = make_float2(__shfl_xor_sync(0xffffffffu, xp[i].x, m), __shfl_xor_sync(0xffffffffu, xp[i].y, m));
      xp[i] = fmap(xp[i], sgn2, other);
    }
  }
  // x * (1/sqrt p) [core/fwht.cpp:60-65]  then * sqrt p [core/quantizer.cpp:73-75]
  const float2 sq2 = make_float2(sq, sq), isq2 = make_float2(isq, isq);
  float x[EPL];
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const float2 v = mulp(mulp(xp[i], isq2), sq2);
    x[2 * i] = v.x;
    x[2 * i + 1] = v.y;
  }
  if constexpr (BITS == 3) { // 8 indices -> 3 bytes, big-endian bit order
    uint32_t r[EPL / 8];
#pragma unroll
    for (int g = 0; g < EPL / 8; ++g) {
      uint32_t v24 = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        switch (k) { // the shift must be a compile-time constant
        case 0: quantize_into_word<3, 21>(v24, x[g * 8 + 0], qtab_addr); break;
        case 1: quantize_into_word<3, 18>(v24, x[g * 8 + 1], qtab_addr); break;
        case 2: quantize_into_word<3, 15>(v24, x[g * 8 + 2], qtab_addr); break;
        case 3: quantize_into_word<3, 12>(v24, x[g * 8 + 3], qtab_addr); break;
        case 4: quantize_into_word<3, 9>(v24, x[g * 8 + 4], qtab_addr); break;
        case 5: quantize_into_word<3, 6>(v24, x[g * 8 + 5], qtab_addr); break;
        case 6: quantize_into_word<3, 3>(v24, x[g * 8 + 6], qtab_addr); break;
        default: quantize_into_word<3, 0>(v24, x[g * 8 + 7], qtab_addr); break;
        }
      }
      r[g] = __byte_perm(v24, 0, 0x3012); // memory image of the three bytes, first byte lowest
    }
    if constexpr (EPL == 32) {
      w[0] = r[0] | (r[1] << 24);
      w[1] = (r[1] >> 8) | (r[2] << 16);
      w[2] = (r[2] >> 16) | (r[3] << 8);
    } else {
      w[0] = r[0] | (r[1] << 24);
      w[1] = r[1] >> 8;
    }
  } else {
    constexpr int PER = 32 / BITS;
#pragma unroll
    for (int i = 0; i < EPL; i += PER) {
      uint32_t word = 0;
      quantize_word<BITS, 0>(word, x + i, qtab_addr);
      w[i / PER] = word;
    }
  }
}

// The work of one block: tiles block_rank, block_rank + n_blocks, ... of launch `a`,
// for side `which` (0 keys, 1 values) whose rows start at `src` (these two override
// a.which / a.src, so that one launch descriptor serves both sides).
template <int P, int BITS>
__device__ __forceinline__ void append_tile_body(const AppendLaunch &a, const float *src, const int which,
                                                 const int block_rank, const int n_blocks) {
  constexpr int EPL = P / 4;     // coordinates per lane
  constexpr int PITCH = P + 4;   // floats; +16 B keeps both passes' 128-bit reads conflict-free
  // Contiguous sources arrive eight rows per bulk copy (a copy costs its issuing
  // thread tens of cycles whatever its size): rows then sit back to back in groups
  // of eight, with the 16-byte skew between groups instead of between rows, and
  // both passes pick their rows across groups to keep 128-bit reads conflict-free.
  constexpr int GROUP = 8, GPITCH = GROUP * P + 4;
  static_assert(AT_TILE % GROUP == 0 && AT_TILE / GROUP == 8, "eight groups of eight rows");
  constexpr int QB = BITS == 16 ? 4 : BITS;
  extern __shared__ __align__(128) unsigned char smem_rows[];
  float *tile = reinterpret_cast<float *>(smem_rows);
  float *redo_buf = tile + (size_t)AT_TILE * PITCH; // (AT_THREADS/32) x P floats for the general routine
  __shared__ __align__(8) uint64_t bar;
  __shared__ __align__(16) uint2 qtab[QT_ENTRIES];
  __shared__ float2 s_norm[AT_TILE]; // (norm, 1/norm); norm < 0 marks a vector not handled here
  __shared__ int redo_count[2];          // alternates with the tile parity
  __shared__ int redo_list[2][AT_TILE];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool contig = a.contig != 0;
  // vector of the tile this lane works on in pass 2, the row thread `tid` sums in pass 1
  const int vt = contig ? ((lane & 7) * GROUP + warp) : (warp * 8 + (lane & 7));
  const int row1 = contig ? ((tid & 7) * GROUP + (tid >> 3)) : tid;
  const int part = lane >> 3;           // which quarter of the vector
  auto row_ptr = [&](int r) -> float * {
    return contig ? tile + (size_t)(r >> 3) * GPITCH + (size_t)(r & 7) * P : tile + (size_t)r * PITCH;
  };
  if constexpr (BITS != 16) build_quant_table<QB>(qtab, tid, AT_THREADS);
  const uint32_t qtab_addr = smem_u32(qtab);
  const CacheView &c = a.c;
  const long long n_items = (long long)a.heads_in_call * a.n_tokens;
  const long long n_tiles = (n_items + AT_TILE - 1) / AT_TILE;
  const int dim = c.dim;
  const uint32_t row_bytes_in = (uint32_t)dim * 4u;

  if (tid == 0) {
    mbar_init(&bar, AT_TILE);
    fence_barrier_init();
    redo_count[0] = redo_count[1] = 0;
  }
  if (tid < AT_TILE) // zero the padding columns once (dim < P); bulk copies never touch them
    for (int i = dim; i < P; ++i) tile[(size_t)tid * PITCH + i] = 0.f;
  __syncthreads();

  auto issue = [&](long long tile_idx) { // threads 0..AT_TILE-1: one row each, or eight rows for the first eight
    if (contig) {
      const long long g0 = tile_idx * AT_TILE + (long long)tid * GROUP;
      if (tid < AT_TILE / GROUP && g0 < n_items) {
        const uint32_t bytes = (uint32_t)min((long long)GROUP, n_items - g0) * row_bytes_in;
        mbar_expect_tx(&bar, bytes);
        bulk_g2s(tile + (size_t)tid * GPITCH, src + (size_t)g0 * P, bytes, &bar);
        return;
      }
      mbar_arrive(&bar);
      return;
    }
    const long long g = tile_idx * AT_TILE + tid;
    if (g < n_items) {
      const ItemPlace p = place_item32(a, (uint32_t)g);
      if (p.store || p.mirror) {
        mbar_expect_tx(&bar, row_bytes_in);
        bulk_g2s(tile + (size_t)tid * PITCH, (src + (size_t)p.t * a.src_token_stride + (size_t)(p.h - a.head0) * a.c.dim), row_bytes_in, &bar);
        return;
      }
    }
    mbar_arrive(&bar);
  };

  long long tile_idx = block_rank;
  if (tile_idx < n_tiles && tid < AT_TILE) issue(tile_idx);
  uint32_t parity = 0;
  for (; tile_idx < n_tiles; tile_idx += n_blocks) {
    // Only the pass-1 warps poll the copy barrier; everyone else learns of the data
    // through the block barrier after pass 1 (a failed wait is flagged, not fatal:
    // all threads must still reach the barriers).
    if (tid < AT_TILE) {
      if (!mbar_wait(&bar, parity) && tid == 0) atomicExch(a.status, 1);
    }
    const uint32_t par = parity; // this tile's slot in the redo bookkeeping
    parity ^= 1u;

    // ---- pass 1: sequential norms (core/quantizer.cpp:59-66), one thread per vector ----
    if (BITS != 16 && tid < AT_TILE) {
      const long long g = tile_idx * AT_TILE + row1;
      bool live = false;
      if (g < n_items) live = place_item32(a, (uint32_t)g).store;
      if (live) {
        const float4 *r4 = reinterpret_cast<const float4 *>(row_ptr(row1));
        float sum = 0.f;
#pragma unroll 8
        for (int i = 0; i < P / 4; ++i) {
          const float4 v = r4[i];
          const float2 s01 = mulp(make_float2(v.x, v.y), make_float2(v.x, v.y));
          const float2 s23 = mulp(make_float2(v.z, v.w), make_float2(v.z, v.w));
          sum = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(sum, s01.x), s01.y), s23.x), s23.y);
        }
        const bool all_zero = sum == 0.f;
        const float norm = __fsqrt_rn(__fadd_rn(sum, 1e-12f));
        // norm >= 1e-5 makes the +-3 sigma clip a no-op and rules out NaN (see
        // quantize_into_word); an all-zero vector quantises to the middle index either way
        const bool plain = (norm >= 1e-5f && norm < INFINITY) || all_zero;
        s_norm[row1] = plain ? make_float2(norm, __fdiv_rn(1.0f, norm)) : make_float2(-1.f, 1.f);
        if (!plain) redo_list[par][atomicAdd(&redo_count[par], 1)] = row1;
      } else {
        s_norm[row1] = make_float2(-1.f, 1.f);
      }
    }

    // ---- pass 2: four lanes per vector -------------------------------------------------
    const long long g = tile_idx * AT_TILE + vt;
    ItemPlace p;
    p.store = p.mirror = false;
    if (g < n_items) p = place_item32(a, (uint32_t)g);
    __syncthreads(); // the tile has landed (seen by the pass-1 warps) and the norms are published
    if constexpr (BITS != 16) {
      const int n_redo = redo_count[par];
      if (tid == 0) redo_count[par ^ 1u] = 0; // the other slot was last read before the previous tile's second barrier
      if (n_redo > 0) { // rare: tiny, infinite or NaN norms go through the general routine (it reads the source again)
        AppendLaunch side = a; // rare path: a private copy with this side's fields
        side.src = src;
        side.which = which;
        for (int e = warp; e < n_redo; e += AT_THREADS / 32)
          append_item_general(side, tile_idx * AT_TILE + redo_list[par][e], redo_buf + (size_t)warp * P, lane);
      }
    }
    // Vectors that pass 1 handed to the general routine (norm < 0) are skipped here
    // altogether: their lanes run the transform on zeros, because the table
    // quantiser's address arithmetic is only defined for the finite, normalised
    // values of the vectors pass 1 accepted.
    const float2 nrm = BITS == 16 ? make_float2(1.f, 1.f) : s_norm[vt];
    const float norm = nrm.x;
    const bool skip = BITS != 16 && norm < 0.f;
    if (skip) p.store = p.mirror = false;
    if ((p.store || p.mirror) && !AQ_CHECK(a.status, p.slot >= 0 && p.slot < c.cap && p.h >= 0 && p.h < c.n_heads, 11))
      p.store = p.mirror = false;
    float2 xp[EPL / 2]; // coordinates (2i, 2i+1) of this quarter, packed
    {
      const bool have = p.store || p.mirror;
      const float4 *r4 = reinterpret_cast<const float4 *>(row_ptr(vt) + part * EPL);
      if (have) {
#pragma unroll
        for (int i = 0; i < EPL / 4; ++i) {
          const float4 v = r4[i];
          xp[2 * i] = make_float2(v.x, v.y);
          xp[2 * i + 1] = make_float2(v.z, v.w);
        }
      } else {
#pragma unroll
        for (int i = 0; i < EPL / 2; ++i) xp[i] = make_float2(0.f, 0.f);
      }
    }
    __syncthreads(); // every quarter is in registers; the tile buffer is free
    const long long next = tile_idx + n_blocks;
    if (next < n_tiles && tid < AT_TILE) {
      fence_proxy_async();
      issue(next);
    }
    if (p.mirror) {
      float4 *m4 = reinterpret_cast<float4 *>(c.mirror + (size_t)p.h * c.mirror_stride +
                                              (size_t)p.slot * 2 * dim + (which ? dim : 0) + part * EPL);
#pragma unroll
      for (int i = 0; i < EPL / 4; ++i)
        if (part * EPL + 4 * i < dim) m4[i] = make_float4(xp[2 * i].x, xp[2 * i].y, xp[2 * i + 1].x, xp[2 * i + 1].y);
    }
    if constexpr (BITS == 16) {
      if (p.store) {
        uint8_t *slab = which ? c.v_slab : c.k_slab;
        const size_t stride = which ? c.v_stride : c.k_stride;
        float4 *dst = reinterpret_cast<float4 *>(slab + (size_t)p.h * stride + (size_t)p.slot * (P * 4)) + part * (EPL / 4);
#pragma unroll
        for (int i = 0; i < EPL / 4; ++i) dst[i] = make_float4(xp[2 * i].x, xp[2 * i].y, xp[2 * i + 1].x, xp[2 * i + 1].y);
        if (part == 0) ((which ? c.v_scale : c.k_scale) + (size_t)p.h * c.s_stride)[p.slot] = 1.0f;
      }
    } else {
      // Every lane runs the transform (its shuffles need the whole warp); lanes whose
      // vector is not stored here -- ragged tile end, or a vector left to the general
      // routine -- work on zeros and skip the store.
      constexpr int NBYTES = EPL * BITS / 8;
      const bool keep = p.store;
      uint32_t sgw = 0; // sign bits of this quarter in bits 0..EPL-1
      if (keep) {
        sgw = c.signs[(size_t)p.h * c.sign_words + ((part * EPL) >> 5)];
        if constexpr (EPL < 32) sgw >>= (part * EPL) & 31;
      }
      uint32_t w[(EPL * BITS + 31) / 32];
      quantize_quarter<P, BITS>(xp, keep ? nrm.y : 1.f, a.sqrt_p, a.inv_sqrt_p, sgw, lane, w, qtab_addr);
      if (keep) {
        uint8_t *slab = which ? c.v_slab : c.k_slab;
        const size_t stride = which ? c.v_stride : c.k_stride;
        store_packed<NBYTES>(slab + (size_t)p.h * stride + (size_t)p.slot * (P * BITS / 8) + part * NBYTES, w);
        if (part == 0) ((which ? c.v_scale : c.k_scale) + (size_t)p.h * c.s_stride)[p.slot] = norm;
      }
    }
  }
}

template <int P, int BITS>
__global__ void __launch_bounds__(AT_THREADS, AT_BLOCKS_PER_SM) append_tile_kernel(const AppendLaunch a) {
  griddep_launch_dependents();
  append_tile_body<P, BITS>(a, a.src, a.which, (int)blockIdx.x, (int)gridDim.x);
}

// Keys and values of one call in a single launch: blockIdx.y picks the side, so
// the two sides share the SMs from the first cycle to the last and the launch,
// ramp-up and tail costs are paid once.
template <int P, int KB, int VB>
__global__ void __launch_bounds__(AT_THREADS, AT_BLOCKS_PER_SM) append_pair_kernel(const AppendLaunch a, const float *src_v) {
  griddep_launch_dependents();
  // a describes the call and carries the key rows in a.src; the value rows start at src_v
  if constexpr (KB == VB) { // one copy of the code serves both sides
    const int which = (int)blockIdx.y;
    append_tile_body<P, KB>(a, which ? src_v : a.src, which, (int)blockIdx.x, (int)gridDim.x);
  } else {
    if (blockIdx.y == 0) append_tile_body<P, KB>(a, a.src, 0, (int)blockIdx.x, (int)gridDim.x);
    else append_tile_body<P, VB>(a, src_v, 1, (int)blockIdx.x, (int)gridDim.x);
  }
}

} // namespace aq
