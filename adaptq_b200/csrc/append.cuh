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
  int *status;
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

// Same, with 32-bit arithmetic (the tile kernel is only used below 2^31 items).
__device__ __forceinline__ ItemPlace place_item32(const AppendLaunch &a, uint32_t g) {
  ItemPlace p;
  uint32_t hl;
  if (a.head_major) {
    hl = g / (uint32_t)a.n_tokens;
    p.t = (int)(g - hl * (uint32_t)a.n_tokens);
  } else {
    p.t = (int)(g / (uint32_t)a.heads_in_call);
    hl = g - (uint32_t)p.t * (uint32_t)a.heads_in_call;
  }
  p.h = a.head0 + (int)hl;
  const int cap = a.c.cap, T = a.n_tokens;
  p.store = cap > 0 && p.t >= T - cap;
  p.slot = cap > 0 ? (int)(((uint32_t)a.ring_head + (uint32_t)p.t) % (uint32_t)cap) : 0;
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

// Threshold search through a 32-entry shared-memory table: 16 buckets of width
// 0.25 over |v| (the last takes everything from 3.75 up) for v >= +0 and 16 for
// the sign bit set.  No bucket holds more than one decision threshold of the
// 2-, 3- or 4-bit codebooks (the exact 0 in the middle belongs to bucket 0 of
// both halves), so an entry is {that threshold as a signed float, or +inf;
// number of thresholds below the bucket}, and
//   index = entry.count + (v >= entry.threshold)
// is upstream's binary search with its `v >= t` decisions
// (core/codebook.cpp:119-144) for every finite v, including -0.0.  32 entries
// of 8 bytes; the two halves of the table are used by disjoint sets of lanes
// only by chance, so a lookup can see a 2-way bank conflict at worst.
constexpr int QT_ENTRIES = 32;

template <int BITS> __device__ __forceinline__ void build_quant_table(uint2 *qtab, int tid) {
  constexpr int NT = (1 << BITS) - 1; // thresholds, ascending
  if (tid < QT_ENTRIES) {
    const int k = tid & 15;
    const bool negative = tid >= 16;
    // bucket as an interval of v:  [k/4, (k+1)/4)  or  (-(k+1)/4, -k/4]
    const float lo = 0.25f * (float)k, hi = k == 15 ? INFINITY : 0.25f * (float)(k + 1);
    uint32_t below = 0;
    float thr = INFINITY;
    for (int j = 0; j < NT; ++j) {
      const float t = c_thr[BITS - 2][j];
      const bool inside = negative ? (t > -hi && t <= -lo) : (t >= lo && t < hi);
      const bool under = negative ? (t <= -hi) : (t < lo);
      if (under) ++below;
      if (inside) thr = t;
    }
    qtab[tid] = make_uint2(__float_as_uint(thr), below);
  }
}

template <int BITS> __device__ __forceinline__ uint32_t quantize_lookup(float v, uint32_t qtab_addr) {
  // floor(4*min(|v|, 3.99)) lands in the low mantissa bits of 2^23 + 4|v| rounded down;
  // the sign bit selects the upper half of the table
  const float t = __fmaf_rd(fminf(fabsf(v), 3.99f), 4.0f, 8388608.0f);
  const uint32_t key = ((__float_as_uint(v) >> 27) & 16u) | __float_as_uint(t); // 0x4B000000 + bucket
  const uint32_t addr = (key << 3) + (qtab_addr - 0x58000000u);                 // (key - 0x4B000000) * 8
  uint2 e;
  asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(e.x), "=r"(e.y) : "r"(addr));
  return e.y + (v >= __uint_as_float(e.x) ? 1u : 0u);
}

// Bit position of coordinate k of a packed 32-bit word (MSB-first within bytes).
template <int BITS> __device__ __forceinline__ uint32_t index_shift(int k) {
  return BITS == 4 ? (uint32_t)(8 * (k >> 1) + ((k & 1) ? 0 : 4)) : (uint32_t)(8 * (k >> 2) + (6 - 2 * (k & 3)));
}

// Two IEEE round-to-nearest FP32 operations per instruction (sm_100 f32x2).
// Each half is rounded exactly like the scalar operation, so results are
// bit-identical to upstream's scalar code; only the issue slots are halved.
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &a, float &b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ void butterfly2(float &l0, float &l1, float &h0, float &h1) {
  const unsigned long long L = pack2(l0, l1), H = pack2(h0, h1);
  unsigned long long S, D;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(S) : "l"(L), "l"(H));
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(D) : "l"(L), "l"(H));
  unpack2(S, l0, l1);
  unpack2(D, h0, h1);
}
__device__ __forceinline__ void mul2(float &a, float &b, unsigned long long m) {
  unsigned long long r;
  const unsigned long long v = pack2(a, b);
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(v), "l"(m));
  unpack2(r, a, b);
}

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
constexpr int AT_TILE = 128;
constexpr int AT_THREADS = 512;

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

// Quarter-vector transform + quantisation.  x: this lane's EPL = P/4 contiguous
// coordinates (already loaded), `part` = which quarter, sgw = the sign bits of
// those coordinates in bits 0..EPL-1.  Produces EPL*BITS/8 packed bytes in w.
template <int P, int BITS>
__device__ __forceinline__ void quantize_quarter(float (&x)[P / 4], float norm, uint32_t sgw, int lane,
                                                 uint32_t (&w)[(P / 4 * BITS + 31) / 32], uint32_t qtab_addr) {
  constexpr int EPL = P / 4;
  const float inv = __fdiv_rn(1.0f, norm);
  const unsigned long long inv2 = pack2(inv, inv);
#pragma unroll
  for (int i = 0; i < EPL; i += 2) {
    mul2(x[i], x[i + 1], inv2);
    x[i] = __uint_as_float(__float_as_uint(x[i]) ^ ((sgw << (31 - i)) & 0x80000000u));
    x[i + 1] = __uint_as_float(__float_as_uint(x[i + 1]) ^ ((sgw << (30 - i)) & 0x80000000u));
  }
  // stages len = 1 .. EPL/2 stay inside the lane (core/fwht.cpp:36-57)
#pragma unroll
  for (int i = 0; i < EPL; i += 2) {
    const float a = x[i], b = x[i + 1];
    x[i] = __fadd_rn(a, b);
    x[i + 1] = __fsub_rn(a, b);
  }
#pragma unroll
  for (int len = 2; len < EPL; len <<= 1) {
#pragma unroll
    for (int i = 0; i < EPL; i += (len << 1)) {
#pragma unroll
      for (int j = 0; j < len; j += 2) butterfly2(x[i + j], x[i + j + 1], x[i + j + len], x[i + j + len + 1]);
    }
  }
  // stages len = EPL and 2*EPL pair this lane with the lanes 8 and 16 away: the
  // lower quarter keeps a+b, the upper one a-b.  Both are partner + (+-1)*mine in
  // one fused multiply-add, which rounds exactly like the plain add or subtract.
#pragma unroll
  for (int m = 8; m <= 16; m <<= 1) {
    const float sgn = (lane & m) ? -1.0f : 1.0f;
    const unsigned long long sgn2 = pack2(sgn, sgn);
#pragma unroll
    for (int i = 0; i < EPL; i += 2) {
      const float o0 = __shfl_xor_sync(0xffffffffu, x[i], m), o1 = __shfl_xor_sync(0xffffffffu, x[i + 1], m);
      unsigned long long r;
      asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(pack2(x[i], x[i + 1])), "l"(sgn2), "l"(pack2(o0, o1)));
      unpack2(r, x[i], x[i + 1]);
    }
  }
  // x * (1/sqrt p) [core/fwht.cpp:60-65]  then * sqrt p [core/quantizer.cpp:73-75]
  const float sq = __fsqrt_rn((float)P);
  const float isq = __fdiv_rn(1.0f, sq);
  const unsigned long long sq2 = pack2(sq, sq), isq2 = pack2(isq, isq);
#pragma unroll
  for (int i = 0; i < EPL; i += 2) {
    mul2(x[i], x[i + 1], isq2);
    mul2(x[i], x[i + 1], sq2);
  }
  if constexpr (BITS == 3) { // 8 indices -> 3 bytes, big-endian bit order
    uint32_t r[EPL / 8];
#pragma unroll
    for (int g = 0; g < EPL / 8; ++g) {
      uint32_t v24 = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) v24 += quantize_lookup<3>(x[g * 8 + k], qtab_addr) << (21 - 3 * k);
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
#pragma unroll
      for (int k = 0; k < PER; ++k) word += quantize_lookup<BITS>(x[i + k], qtab_addr) << index_shift<BITS>(k);
      w[i / PER] = word;
    }
  }
}

template <int P, int BITS>
__global__ void __launch_bounds__(AT_THREADS, 2) append_tile_kernel(const AppendLaunch a) {
  constexpr int EPL = P / 4;     // coordinates per lane
  constexpr int PITCH = P + 4;   // floats; +16 B keeps both passes' 128-bit reads conflict-free
  constexpr int QB = BITS == 16 ? 4 : BITS;
  extern __shared__ __align__(128) unsigned char smem_rows[];
  float *tile = reinterpret_cast<float *>(smem_rows);
  float *redo_buf = tile + (size_t)AT_TILE * PITCH; // (AT_THREADS/32) x P floats for the general routine
  __shared__ __align__(8) uint64_t bar;
  __shared__ __align__(16) uint2 qtab[QT_ENTRIES];
  __shared__ float s_norm[AT_TILE];
  __shared__ int redo_count;
  __shared__ int redo_list[AT_TILE];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vt = warp * 8 + (lane & 7); // vector of the tile this lane works on in pass 2
  const int part = lane >> 3;           // which quarter of it
  if constexpr (BITS != 16) build_quant_table<QB>(qtab, tid);
  const uint32_t qtab_addr = smem_u32(qtab);
  const CacheView &c = a.c;
  const long long n_items = (long long)a.heads_in_call * a.n_tokens;
  const long long n_tiles = (n_items + AT_TILE - 1) / AT_TILE;
  const int dim = c.dim;
  const uint32_t row_bytes_in = (uint32_t)dim * 4u;

  if (tid == 0) {
    mbar_init(&bar, AT_TILE);
    fence_barrier_init();
    redo_count = 0;
  }
  if (tid < AT_TILE) // zero the padding columns once (dim < P); bulk copies never touch them
    for (int i = dim; i < P; ++i) tile[(size_t)tid * PITCH + i] = 0.f;
  __syncthreads();

  auto issue = [&](long long tile_idx) { // threads 0..127: one row each
    const long long g = tile_idx * AT_TILE + tid;
    if (g < n_items) {
      const ItemPlace p = place_item32(a, (uint32_t)g);
      if (p.store || p.mirror) {
        mbar_expect_tx(&bar, row_bytes_in);
        bulk_g2s(tile + (size_t)tid * PITCH, item_src(a, p), row_bytes_in, &bar);
        return;
      }
    }
    mbar_arrive(&bar);
  };

  long long tile_idx = blockIdx.x;
  if (tile_idx < n_tiles && tid < AT_TILE) issue(tile_idx);
  uint32_t parity = 0;
  for (; tile_idx < n_tiles; tile_idx += gridDim.x) {
    if (!mbar_wait(&bar, parity)) {
      if (tid == 0) atomicExch(a.status, 1);
      return;
    }
    parity ^= 1u;

    // ---- pass 1: sequential norms (core/quantizer.cpp:59-66), one thread per vector ----
    if (BITS != 16 && tid < AT_TILE) {
      const long long g = tile_idx * AT_TILE + tid;
      bool live = false;
      if (g < n_items) live = place_item32(a, (uint32_t)g).store;
      if (live) {
        const float4 *r4 = reinterpret_cast<const float4 *>(tile + (size_t)tid * PITCH);
        float sum = 0.f;
#pragma unroll 8
        for (int i = 0; i < P / 4; ++i) {
          const float4 v = r4[i];
          float s0 = v.x, s1 = v.y, s2 = v.z, s3 = v.w;
          mul2(s0, s1, pack2(v.x, v.y));
          mul2(s2, s3, pack2(v.z, v.w));
          sum = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(sum, s0), s1), s2), s3);
        }
        const bool all_zero = sum == 0.f;
        const float norm = __fsqrt_rn(__fadd_rn(sum, 1e-12f));
        // norm >= 1e-5 makes the +-3 sigma clip a no-op and rules out NaN (see
        // quantize_lookup); an all-zero vector quantises to the middle index either way
        const bool plain = (norm >= 1e-5f && norm < INFINITY) || all_zero;
        s_norm[tid] = plain ? norm : -1.f;
        if (!plain) redo_list[atomicAdd(&redo_count, 1)] = tid;
      } else {
        s_norm[tid] = -1.f;
      }
    }

    // ---- pass 2: four lanes per vector -------------------------------------------------
    const long long g = tile_idx * AT_TILE + vt;
    ItemPlace p;
    p.store = p.mirror = false;
    if (g < n_items) p = place_item32(a, (uint32_t)g);
    float x[EPL];
    {
      const bool have = p.store || p.mirror;
      const float4 *r4 = reinterpret_cast<const float4 *>(tile + (size_t)vt * PITCH + part * EPL);
#pragma unroll
      for (int i = 0; i < EPL / 4; ++i) {
        const float4 v = have ? r4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
      }
    }
    __syncthreads(); // rows are in registers, norms are published; the tile buffer is free
    const float norm = BITS == 16 ? 1.f : s_norm[vt];
    const long long next = tile_idx + gridDim.x;
    if (next < n_tiles && tid < AT_TILE) {
      fence_proxy_async();
      issue(next);
    }
    if (p.mirror) {
      float4 *m4 = reinterpret_cast<float4 *>(c.mirror + (size_t)p.h * c.mirror_stride + (size_t)p.slot * 2 * dim +
                                              (a.which ? dim : 0) + part * EPL);
#pragma unroll
      for (int i = 0; i < EPL / 4; ++i)
        if (part * EPL + 4 * i < dim) m4[i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
    }
    if constexpr (BITS == 16) {
      if (p.store) {
        uint8_t *slab = a.which ? c.v_slab : c.k_slab;
        const size_t stride = a.which ? c.v_stride : c.k_stride;
        float4 *dst = reinterpret_cast<float4 *>(slab + (size_t)p.h * stride + (size_t)p.slot * (P * 4)) + part * (EPL / 4);
#pragma unroll
        for (int i = 0; i < EPL / 4; ++i) dst[i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
        if (part == 0) ((a.which ? c.v_scale : c.k_scale) + (size_t)p.h * c.s_stride)[p.slot] = 1.0f;
      }
    } else {
      // Every lane runs the transform (its shuffles need the whole warp); lanes whose
      // vector is not stored here -- ragged tile end, or a vector left to the general
      // routine -- work on zeros and skip the store.
      constexpr int NBYTES = EPL * BITS / 8;
      const bool keep = p.store && norm >= 0.f;
      uint32_t sgw = 0; // sign bits of this quarter in bits 0..EPL-1
      if (keep) {
        sgw = c.signs[(size_t)p.h * c.sign_words + ((part * EPL) >> 5)];
        if constexpr (EPL < 32) sgw >>= (part * EPL) & 31;
      }
      uint32_t w[(EPL * BITS + 31) / 32];
      quantize_quarter<P, BITS>(x, keep ? norm : 1.f, sgw, lane, w, qtab_addr);
      if (keep) {
        uint8_t *slab = a.which ? c.v_slab : c.k_slab;
        const size_t stride = a.which ? c.v_stride : c.k_stride;
        store_packed<NBYTES>(slab + (size_t)p.h * stride + (size_t)p.slot * (P * BITS / 8) + part * NBYTES, w);
        if (part == 0) ((a.which ? c.v_scale : c.k_scale) + (size_t)p.h * c.s_stride)[p.slot] = norm;
      }
    }
    if constexpr (BITS != 16) {
      __syncthreads();
      const int n_redo = redo_count;
      if (n_redo > 0) { // rare: tiny, infinite or NaN norms
        for (int e = warp; e < n_redo; e += AT_THREADS / 32)
          append_item_general(a, tile_idx * AT_TILE + redo_list[e], redo_buf + (size_t)warp * P, lane);
        __syncthreads();
        if (tid == 0) redo_count = 0;
      }
    }
  }
}

} // namespace aq
