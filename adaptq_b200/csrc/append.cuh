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

__device__ __forceinline__ const float *item_src(const AppendLaunch &a, const ItemPlace &p) {
  return a.src + (size_t)p.t * a.src_token_stride + (size_t)(p.h - a.head0) * a.c.dim;
}

// ---------------------------------------------------------------------------
// Register-resident path: one thread owns one vector (P floats in registers).
// ---------------------------------------------------------------------------

// Threshold search through a 16-entry shared-memory table over |v| in steps of
// 0.25 (the last entry takes everything from 3.75 up): every such bucket holds
// at most one of the positive midpoints of the 2-, 3- and 4-bit codebooks, so
// an entry is {bits of that midpoint or 0xFFFFFFFF, number of midpoints below
// the bucket}.  16 entries of 8 bytes span the 32 banks exactly once: lookups
// never conflict.  With a = |v| as an integer (one less for negative v, which
// turns the comparison into the strict one the mirrored negative midpoints
// need),
//   m = entry.count + (a >= entry.midpoint),  index = m ^ (v < 0 ? half-1 : half)
// equals upstream's binary search (core/codebook.cpp:119-144) for every
// non-NaN v.  Used only on vectors where NaN cannot occur.
constexpr int QT_ENTRIES = 16;

template <int BITS> __device__ __forceinline__ void build_quant_table(uint2 *qtab, int tid) {
  constexpr int HALF = 1 << (BITS - 1);
  if (tid < QT_ENTRIES) {
    const float lo = 0.25f * (float)tid, hi = tid == QT_ENTRIES - 1 ? INFINITY : 0.25f * (float)(tid + 1);
    uint32_t m = 0, thr = 0xFFFFFFFFu;
    for (int k = 0; k < HALF - 1; ++k) {
      const float pk = c_thr[BITS - 2][HALF + k];
      if (pk < lo) ++m;
      else if (pk < hi) thr = __float_as_uint(pk);
    }
    qtab[tid] = make_uint2(thr, m);
  }
}

template <int BITS> __device__ __forceinline__ uint32_t quantize_lookup(float v, uint32_t qtab_addr) {
  constexpr uint32_t HALF = 1u << (BITS - 1);
  const bool neg = v < 0.0f;
  uint32_t a = __float_as_uint(v) & 0x7FFFFFFFu;
  a -= neg ? 1u : 0u;
  // floor(4*min(|v|, 3.99)) lands in the low mantissa bits of 2^23 + 4|v| rounded down
  const float t = __fmaf_rd(fminf(__uint_as_float(a), 3.99f), 4.0f, 8388608.0f);
  const uint32_t addr = (__float_as_uint(t) << 3) + (qtab_addr - 0x58000000u); // (bits - 0x4B000000) * 8
  uint2 e;
  asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(e.x), "=r"(e.y) : "r"(addr));
  const uint32_t m = e.y + (a >= e.x ? 1u : 0u);
  return m ^ (neg ? HALF - 1u : HALF);
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

// Returns false (and leaves `w` untouched) for the rare vectors that need the
// literal clip path; the caller re-does those with the general routine.
template <int P, int BITS>
__device__ __forceinline__ bool quantize_row_regs(float (&x)[P], const uint32_t (&sg)[(P + 31) / 32],
                                                  uint32_t (&w)[(P * BITS + 31) / 32], uint32_t qtab_addr,
                                                  float &norm_out) {
  // L2 norm: a strictly sequential chain, multiply and add rounded separately
  // (core/quantizer.cpp:59-66).  The squares are independent and go two at a time.
  float norm = 0.f;
#pragma unroll
  for (int i = 0; i < P; i += 2) {
    float s0 = x[i], s1 = x[i + 1];
    mul2(s0, s1, pack2(x[i], x[i + 1]));
    norm = __fadd_rn(norm, s0);
    norm = __fadd_rn(norm, s1);
  }
  const bool all_zero = norm == 0.f;
  norm = __fsqrt_rn(__fadd_rn(norm, 1e-12f));
  norm_out = norm;
  // The +-3 sigma clip (core/quantizer.cpp:81-89) can only change an index when
  // 3*sigma falls below the largest midpoint (2.1476).  sigma^2 equals
  // (norm^2 - 1e-12)/norm^2 up to rounding, so for norm >= 1e-5 it is >= 0.98 and
  // the clip is a no-op; a finite norm also rules out NaN.  An all-zero vector
  // quantises to the middle index with or without the clip.  Everything else
  // (tiny, infinite or NaN norms) is left to the general routine.
  if (!((norm >= 1e-5f && norm < INFINITY) || all_zero)) return false;

  const float inv = __fdiv_rn(1.0f, norm);
  const unsigned long long inv2 = pack2(inv, inv);
  // normalise, then the Rademacher sign (a sign-bit XOR equals the multiply by +-1)
#pragma unroll
  for (int i = 0; i < P; i += 2) {
    mul2(x[i], x[i + 1], inv2);
    x[i] = __uint_as_float(__float_as_uint(x[i]) ^ ((sg[i >> 5] << (31 - (i & 31))) & 0x80000000u));
    x[i + 1] = __uint_as_float(__float_as_uint(x[i + 1]) ^ ((sg[i >> 5] << (30 - (i & 31))) & 0x80000000u));
  }
  // butterflies in upstream's stage order (core/fwht.cpp:36-57): len = 1 pairs
  // neighbours, every later stage moves two neighbouring butterflies at once
#pragma unroll
  for (int i = 0; i < P; i += 2) {
    const float a = x[i], b = x[i + 1];
    x[i] = __fadd_rn(a, b);
    x[i + 1] = __fsub_rn(a, b);
  }
#pragma unroll
  for (int len = 2; len < P; len <<= 1) {
#pragma unroll
    for (int i = 0; i < P; i += (len << 1)) {
#pragma unroll
      for (int j = 0; j < len; j += 2) butterfly2(x[i + j], x[i + j + 1], x[i + j + len], x[i + j + len + 1]);
    }
  }
  // x * (1/sqrt p) [core/fwht.cpp:60-65]  then * sqrt p [core/quantizer.cpp:73-75]
  const float sq = __fsqrt_rn((float)P);
  const float isq = __fdiv_rn(1.0f, sq);
  const unsigned long long sq2 = pack2(sq, sq), isq2 = pack2(isq, isq);
#pragma unroll
  for (int i = 0; i < P; i += 2) {
    mul2(x[i], x[i + 1], isq2);
    mul2(x[i], x[i + 1], sq2);
  }
  if (BITS == 3) { // 8 indices -> 3 bytes, big-endian bit order
#pragma unroll
    for (int i = 0; i < P; i += 32) {
      uint32_t r[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t v24 = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) v24 |= quantize_lookup<3>(x[i + g * 8 + k], qtab_addr) << (21 - 3 * k);
        r[g] = __byte_perm(v24, 0, 0x3012); // memory image of the three bytes, first byte lowest
      }
      w[(i >> 5) * 3 + 0] = r[0] | (r[1] << 24);
      w[(i >> 5) * 3 + 1] = (r[1] >> 8) | (r[2] << 16);
      w[(i >> 5) * 3 + 2] = (r[2] >> 16) | (r[3] << 8);
    }
  } else {
    constexpr int PER = 32 / BITS;
#pragma unroll
    for (int i = 0; i < P; i += PER) {
      uint32_t word = 0;
#pragma unroll
      for (int k = 0; k < PER; ++k) word |= quantize_lookup<BITS>(x[i + k], qtab_addr) << index_shift<BITS>(k);
      w[i / PER] = word;
    }
  }
  return true;
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
// One block = THREADS vectors per tile; rows arrive in shared memory through
// per-row bulk (TMA) copies, each thread then pulls its row into registers,
// and the next tile's copies are issued before the arithmetic starts.  The
// few vectors the register path declines are listed and redone by the general
// routine before the block moves on.
// ---------------------------------------------------------------------------
template <int P, int BITS, int THREADS>
__global__ void __launch_bounds__(THREADS, (P == 128 ? 3 : 4))
append_rows_kernel(const AppendLaunch a) {
  constexpr int PITCH = P + 4; // floats; +16 B keeps 128-bit row reads conflict-free
  extern __shared__ __align__(128) unsigned char smem_rows[];
  float *tile = reinterpret_cast<float *>(smem_rows);
  float *redo_buf = tile + (size_t)THREADS * PITCH; // (THREADS/32) x P floats
  __shared__ __align__(8) uint64_t bar;
  __shared__ __align__(16) uint2 qtab[QT_ENTRIES];
  __shared__ int redo_count;
  __shared__ int redo_list[THREADS];

  const int tid = threadIdx.x;
  if constexpr (BITS != 16) build_quant_table<BITS>(qtab, tid);
  const uint32_t qtab_addr = smem_u32(qtab);
  const long long n_items = (long long)a.heads_in_call * a.n_tokens;
  const long long n_tiles = (n_items + THREADS - 1) / THREADS;
  const int dim = a.c.dim;
  const uint32_t row_bytes_in = (uint32_t)dim * 4u;
  float *my_row = tile + (size_t)tid * PITCH;

  if (tid == 0) {
    mbar_init(&bar, THREADS);
    fence_barrier_init();
    redo_count = 0;
  }
  // zero the padding columns once (dim < P); bulk copies never touch them
  for (int i = dim; i < P; ++i) my_row[i] = 0.f;
  __syncthreads();

  auto issue = [&](long long tile_idx) {
    long long g = tile_idx * THREADS + tid;
    if (g < n_items) {
      ItemPlace p = place_item(a, g);
      if (p.store || p.mirror) {
        mbar_expect_tx(&bar, row_bytes_in);
        bulk_g2s(my_row, item_src(a, p), row_bytes_in, &bar);
        return;
      }
    }
    mbar_arrive(&bar);
  };

  long long tile_idx = blockIdx.x;
  if (tile_idx < n_tiles) issue(tile_idx);
  uint32_t parity = 0;
  for (; tile_idx < n_tiles; tile_idx += gridDim.x) {
    if (!mbar_wait(&bar, parity)) {
      if (tid == 0) atomicExch(a.status, 1);
      return;
    }
    parity ^= 1u;
    const long long g = tile_idx * THREADS + tid;
    ItemPlace p;
    p.store = p.mirror = false;
    if (g < n_items) p = place_item(a, g);
    float x[P];
    if (p.store || p.mirror) {
      const float4 *r4 = reinterpret_cast<const float4 *>(my_row);
#pragma unroll
      for (int i = 0; i < P / 4; ++i) {
        float4 v = r4[i];
        x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
      }
    }
    __syncthreads(); // every row has been read; the tile buffer is free
    const long long next = tile_idx + gridDim.x;
    if (next < n_tiles) {
      fence_proxy_async();
      issue(next);
    }
    if (p.mirror) {
      float4 *m4 = reinterpret_cast<float4 *>(a.c.mirror + (size_t)p.h * a.c.mirror_stride +
                                              (size_t)p.slot * 2 * dim + (a.which ? dim : 0));
#pragma unroll
      for (int i = 0; i < P / 4; ++i)
        if (4 * i < dim) m4[i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
    }
    if (p.store) {
      const CacheView &c = a.c;
      uint8_t *slab = a.which ? c.v_slab : c.k_slab;
      const size_t stride = a.which ? c.v_stride : c.k_stride;
      float *scale = (a.which ? c.v_scale : c.k_scale) + (size_t)p.h * c.s_stride + p.slot;
      if constexpr (BITS == 16) {
        float4 *dst = reinterpret_cast<float4 *>(slab + (size_t)p.h * stride + (size_t)p.slot * (P * 4));
#pragma unroll
        for (int i = 0; i < P / 4; ++i) dst[i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
        *scale = 1.0f;
      } else {
        constexpr int NW = (P * BITS + 31) / 32;
        uint32_t sg[(P + 31) / 32];
#pragma unroll
        for (int i = 0; i < (P + 31) / 32; ++i) sg[i] = c.signs[(size_t)p.h * c.sign_words + i];
        uint32_t w[NW];
        float norm;
        if (quantize_row_regs<P, BITS>(x, sg, w, qtab_addr, norm)) {
          uint8_t *row = slab + (size_t)p.h * stride + (size_t)p.slot * (NW * 4);
          if ((NW * 4) % 16 == 0) {
            uint4 *d4 = reinterpret_cast<uint4 *>(row);
#pragma unroll
            for (int i = 0; i < NW / 4; ++i) d4[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
          } else {
            uint2 *d2 = reinterpret_cast<uint2 *>(row);
#pragma unroll
            for (int i = 0; i < NW / 2; ++i) d2[i] = make_uint2(w[2 * i], w[2 * i + 1]);
          }
          *scale = norm;
        } else {
          redo_list[atomicAdd(&redo_count, 1)] = tid;
        }
      }
    }
    if constexpr (BITS != 16) {
      __syncthreads();
      const int n_redo = redo_count;
      if (n_redo > 0) { // rare: tiny, infinite or NaN norms
        const int warp = tid >> 5, lane = tid & 31;
        for (int e = warp; e < n_redo; e += THREADS / 32)
          append_item_general(a, tile_idx * THREADS + redo_list[e], redo_buf + (size_t)warp * P, lane);
        __syncthreads();
        if (tid == 0) redo_count = 0;
      }
    }
  }
}

} // namespace aq
