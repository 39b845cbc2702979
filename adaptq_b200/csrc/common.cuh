// Shared device-side definitions for the AdapTQ sm_100a kernels.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace aq {

// ---------------------------------------------------------------------------
// Checked build (-DADAPTQ_CHECKED): device-side index checks that never trap.  A
// failed check records its code in the launch's status word (the host reports it
// through adaptq_mha_synchronize) and the guarded access is skipped, so the context
// stays usable.  In the normal build the macro is the constant `true`.
//   11 append: slot or head outside the cache      12 compute: token row outside the cache
//   13 streaming kernel: a stage copy would read past the head's slab
//   14 partial / output slot outside its buffer    15 sparse V: token index outside the cache
// ---------------------------------------------------------------------------
#ifdef ADAPTQ_CHECKED
#define AQ_CHECK(status_ptr, cond, code) ((cond) ? true : (atomicExch((status_ptr), (code)), false))
#else
#define AQ_CHECK(status_ptr, cond, code) (true)
#endif

// ---------------------------------------------------------------------------
// Lloyd-Max N(0,1) centroids and their midpoint decision thresholds.
// Same numbers as upstream core/codebook.cpp:32-62 (centroids) and :67-100
// (thresholds).  The thresholds are written as the expression (a+b)*0.5f so
// that the compiler rounds them exactly as upstream's compiler does; the
// middle one is an exact zero.
// Row b-2 holds the table for b bits.
// ---------------------------------------------------------------------------
#define AQ_CB2 -1.5104f, -0.4528f, 0.4528f, 1.5104f
#define AQ_CB3 -2.1529f, -1.3439f, -0.7560f, -0.2451f, 0.2451f, 0.7560f, 1.3439f, 2.1529f
#define AQ_CB4 -2.4008f, -1.8944f, -1.5105f, -1.2016f, -0.9138f, -0.6402f, -0.3795f, -0.1258f, \
                0.1258f,  0.3795f,  0.6402f,  0.9138f,  1.2016f,  1.5105f,  1.8944f,  2.4008f

__device__ __constant__ float c_cb[3][16] = {
    {AQ_CB2, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0},
    {AQ_CB3, 0, 0, 0, 0, 0, 0, 0, 0},
    {AQ_CB4}};

#define AQ_MID(a, b) (((a) + (b)) * 0.5f)
__device__ __constant__ float c_thr[3][16] = {
    {AQ_MID(-1.5104f, -0.4528f), 0.0f, AQ_MID(0.4528f, 1.5104f), 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0},
    {AQ_MID(-2.1529f, -1.3439f), AQ_MID(-1.3439f, -0.7560f), AQ_MID(-0.7560f, -0.2451f), 0.0f,
     AQ_MID(0.2451f, 0.7560f), AQ_MID(0.7560f, 1.3439f), AQ_MID(1.3439f, 2.1529f), 0, 0, 0, 0, 0, 0, 0, 0, 0},
    {AQ_MID(-2.4008f, -1.8944f), AQ_MID(-1.8944f, -1.5105f), AQ_MID(-1.5105f, -1.2016f),
     AQ_MID(-1.2016f, -0.9138f), AQ_MID(-0.9138f, -0.6402f), AQ_MID(-0.6402f, -0.3795f),
     AQ_MID(-0.3795f, -0.1258f), 0.0f, AQ_MID(0.1258f, 0.3795f), AQ_MID(0.3795f, 0.6402f),
     AQ_MID(0.6402f, 0.9138f), AQ_MID(0.9138f, 1.2016f), AQ_MID(1.2016f, 1.5105f),
     AQ_MID(1.5105f, 1.8944f), AQ_MID(1.8944f, 2.4008f), 0}};

// Host copies (same initialisers) for code that needs them on the CPU side.
static const float h_cb[3][16] = {
    {AQ_CB2, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}, {AQ_CB3, 0, 0, 0, 0, 0, 0, 0, 0}, {AQ_CB4}};

// ---------------------------------------------------------------------------
// Geometry of one handle's cache in HBM.
//
//   k_slab : [n_heads] x k_stride bytes; head h, slot s at  h*k_stride + s*k_row
//   v_slab : likewise.  Rows are byte-for-byte upstream's rows
//            (MSB-first packed indices, or FP32 when bits == 16).
//   k_scale, v_scale : [n_heads] x s_stride floats.
//   signs  : [n_heads] x sign_words uint32; bit i set  <=>  D[i] = -1.
//   mirror : [n_heads] x hyb x 2*dim floats (FP32 copy of the first tokens).
//
// The ring state (write position, live count, mirror length) lives on the host
// and reaches the kernels as launch arguments.
//
// Per-head strides are multiples of 128 bytes so that any tile that starts
// at a multiple of 16 tokens is 16-byte aligned for bulk (TMA) copies.
// ---------------------------------------------------------------------------
struct CacheView {
  uint8_t *k_slab, *v_slab;
  float *k_scale, *v_scale;
  const uint32_t *signs;
  float *mirror;
  size_t k_stride, v_stride, mirror_stride;
  int s_stride, sign_words;
  int n_heads, dim, padded, log2p, k_bits, v_bits, k_row, v_row, cap, hyb;
  float v_mass;
  // Sparse V walks the sorted weights in blocks of this many rows while a whole block
  // remains (4: AttentionHead, attention.cpp:456-465), then row by row; 1 = row by row
  // from the start (HARFixedStrategy::compute_full, strategies/har_fixed.cpp:258-264).
  int sparse_block;
};

__host__ __device__ inline int row_bytes(int padded, int bits) {
  return bits == 16 ? padded * 4 : (padded * bits + 7) / 8;
}

// Programmatic dependent launch.  A decode step launches the append kernel and then the
// attention kernel with the stream-serialisation attribute: the append kernel lets the
// dependent grid start at once (every one of its blocks calls this on entry, so all of them
// are resident by then), and the attention kernel runs its set-up (barrier initialisation,
// query rotation, score table) beside the append and waits here, for the whole append grid
// and its memory, before it first touches the cache.  Without the attribute both are no-ops.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Index j of a packed row (upstream core/quantizer.cpp:156-194 layouts).
__device__ __forceinline__ int unpack_at(const uint8_t *row, int j, int bits) {
  if (bits == 4) {
    int b = row[j >> 1];
    return (j & 1) ? (b & 15) : (b >> 4);
  } else if (bits == 2) {
    int b = row[j >> 2];
    return (b >> (6 - 2 * (j & 3))) & 3;
  } else {
    const uint8_t *p = row + (j >> 3) * 3;
    int v = (p[0] << 16) | (p[1] << 8) | p[2];
    return (v >> (21 - 3 * (j & 7))) & 7;
  }
}

// Binary search over the midpoint table with `v >= t` decisions; NaN maps to
// the centroid just below zero (upstream core/codebook.cpp:119-144).
template <int BITS> __device__ __forceinline__ int quantize_value(float v) {
  const float *T = c_thr[BITS - 2];
  if (v != v) return (1 << (BITS - 1)) - 1;
  if (BITS == 4) {
    int i = (v >= T[7]) ? 8 : 0;
    float t = i ? T[11] : T[3];
    i += (v >= t) ? 4 : 0;
    t = (i & 8) ? ((i & 4) ? T[13] : T[9]) : ((i & 4) ? T[5] : T[1]);
    i += (v >= t) ? 2 : 0;
    float ta = (i & 2) ? T[2] : T[0], tb = (i & 2) ? T[6] : T[4];
    float tc = (i & 2) ? T[10] : T[8], td = (i & 2) ? T[14] : T[12];
    t = (i & 8) ? ((i & 4) ? td : tc) : ((i & 4) ? tb : ta);
    i += (v >= t) ? 1 : 0;
    return i;
  } else if (BITS == 3) {
    int i = (v >= T[3]) ? 4 : 0;
    float t = i ? T[5] : T[1];
    i += (v >= t) ? 2 : 0;
    t = (i & 4) ? ((i & 2) ? T[6] : T[4]) : ((i & 2) ? T[2] : T[0]);
    i += (v >= t) ? 1 : 0;
    return i;
  } else {
    int i = (v >= T[1]) ? 2 : 0;
    float t = i ? T[2] : T[0];
    i += (v >= t) ? 1 : 0;
    return i;
  }
}

__device__ __forceinline__ int quantize_value_rt(float v, int bits) {
  return bits == 4 ? quantize_value<4>(v) : bits == 3 ? quantize_value<3>(v) : quantize_value<2>(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// In-place butterflies over a shared-memory vector of length p by the whole
// block (lower index a+b, upper a-b, stage order len = 1, 2, ... p/2 as
// upstream core/fwht.cpp:36-57).  Caller syncs before and after.
__device__ __forceinline__ void block_butterflies(float *x, int p) {
  for (int len = 1; len < p; len <<= 1) {
    for (int t = threadIdx.x; t < (p >> 1); t += blockDim.x) {
      int i = ((t / len) * (len << 1)) + (t % len);
      float a = x[i], b = x[i + len];
      x[i] = a + b;
      x[i + len] = a - b;
    }
    __syncthreads();
  }
}

// Walsh-Hadamard butterflies over P = 32*EPL values held EPL per lane (lane l
// owns elements EPL*l .. EPL*l+EPL-1), stage order len = 1, 2, ... P/2, lower
// index a+b, upper a-b (core/fwht.cpp:36-57).  One warp, no shared memory.
template <int EPL> __device__ __forceinline__ void warp_butterflies(float (&v)[EPL], int lane) {
#pragma unroll
  for (int len = 1; len < EPL; len <<= 1) {
#pragma unroll
    for (int i = 0; i < EPL; i += (len << 1)) {
#pragma unroll
      for (int j = 0; j < len; ++j) {
        const float a = v[i + j], b = v[i + j + len];
        v[i + j] = a + b;
        v[i + j + len] = a - b;
      }
    }
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const bool upper = (lane & m) != 0;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float other = __shfl_xor_sync(0xffffffffu, v[e], m);
      v[e] = upper ? other - v[e] : v[e] + other;
    }
  }
}

__device__ __forceinline__ float sign_of(const uint32_t *signs, int i) {
  return ((signs[i >> 5] >> (i & 31)) & 1u) ? -1.0f : 1.0f;
}

// mbarrier / bulk-copy (TMA) wrappers.  Every wait is bounded.
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Longest time any device-side wait (ring stage, peer arrival count) may take
// before it gives up and reports through the status word: half a second.
constexpr unsigned long long AQ_WAIT_BUDGET_NS = 500ull * 1000ull * 1000ull;
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_try(uint32_t addr, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(addr), "r"(parity), "r"(20000u) /* suspend-time hint, ns: fewer polling rounds */
      : "memory");
  return done != 0;
}
// Returns false if the phase did not complete within AQ_WAIT_BUDGET_NS.  The
// clock is only read once a first attempt has failed, so a wait that succeeds
// at once costs what a bare try_wait costs.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  if (mbar_try(addr, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    if (mbar_try(addr, parity)) return true;
    if (global_ns() - t0 > AQ_WAIT_BUDGET_NS) return false;
  }
}
// Non-blocking: has the phase with this parity completed?
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// 1-D bulk copy global -> shared; dst/src 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

} // namespace aq
