// Streaming split-KV decode-attention kernel for the bandwidth-bound shapes
// (2-, 3- or 4-bit K and V at padded dimension 128; 3- or 4-bit K with 2-, 3- or 4-bit V at
// 64; dense V).
//
// Replaces the same upstream code as compute_general.cuh -- the quantised
// branch of AttentionHead::compute (attention/attention.cpp:526-563, :606-633)
// with compute_avx2 (:373-474) and fwht_inverse (core/fwht.cpp:106-134) -- but
// organised for HBM streaming on sm_100a:
//
//  * persistent blocks, one per SM; a work item is (head, query, KV span);
//  * a producer warp feeds a ring of 16 KB shared-memory stages with bulk
//    (TMA) copies: the span's K rows (each stage with its tokens' K scales),
//    then its V scales, then its V rows -- K and V are separate slabs and are
//    read as separate streams; the producer runs ahead across phase and item
//    boundaries so HBM never waits for arithmetic, and no consumer loop holds
//    a global load;
//  * K scoring never unpacks an index: a table T[byte][column] =
//    sum over the 2 (4-bit) or 4 (2-bit) coordinates packed in that byte of
//    q_rot[coord]*centroid is built once per item; a score is the sum of one
//    table entry per packed byte.  Lanes own byte columns so every table read
//    is bank-conflict free, and the table sits on a 64 KB boundary so a
//    single byte-permute forms the address.  3-bit keys use 6-bit fields (two
//    coordinates) in place of bytes: T[field value][field column], in four
//    column-rotated copies so that the lanes of a warp step still read 32 banks;
//  * the softmax is exact two-pass over the span (max, then exp), like
//    upstream, with the scores held in shared memory;
//  * V accumulation is the dual trick: instead of decoding V, the weight of a
//    token is added into bucket[byte][column]; after the span, each output
//    coordinate is the centroid-weighted sum of its column's 256 buckets.
//    That costs one shared-memory reduction per packed byte (4 coordinates at
//    2 bits) instead of one multiply-add per coordinate.  The buckets are
//    32-bit fixed point (the span's weights are scaled so that they sum to
//    2^30): integer shared-memory reductions are native and order-independent,
//    so the result is deterministic; floating-point ones are not native.
//    3-bit values use the 6-bit fields of the key side: bucket[field value][field column];
//  * one inverse Walsh-Hadamard transform at the end (or in the merge kernel
//    when the sequence is split);
//  * a helper warp works one item ahead and one item behind the consumers: it
//    rotates the next item's query while the current item streams, and it
//    finishes an item (normalise, inverse transform, store) after the consumers
//    have moved on, so neither step sits between two items' streams.  A block
//    walks a contiguous run of items; consecutive spans of one (head, query)
//    reuse the K table.
//
// No tensor cores: the path is ~5 FLOP/byte of irregular table work.
#pragma once
#include "common.cuh"

namespace aq {

constexpr int CS_CONSUMERS = 512;           // 16 consumer warps
constexpr int CS_WARPS = CS_CONSUMERS / 32;
constexpr int CS_HELPER_TID = CS_CONSUMERS + 32;
constexpr int CS_THREADS = CS_CONSUMERS + 64; // + producer warp + helper warp
constexpr int CS_MISC_BYTES = 3072;
constexpr int CS_STAGE_BYTES = 16384;
constexpr int CS_MAX_STAGES = 6;             // ring stages: as many as fit beside the tables (3..5)
constexpr int CS_SPAN_MAX = 8192;           // tokens per work item (scores kept in shared memory)
constexpr int CS_TABLE_BYTES = 65536;       // [256][64] floats
constexpr size_t CS_SMEM_BYTES = 65536 /* alignment slack, holds the ring */ + CS_TABLE_BYTES /* K table */ +
                                 CS_TABLE_BYTES /* V buckets */ + CS_SPAN_MAX * 4 /* scores */ + CS_MISC_BYTES;

struct StreamLaunch {
  CacheView c;
  const float *q; // [heads_in_call][nq][dim]
  float *out;     // [heads_in_call][nq][dim]                 (n_splits == 1)
  float *partial; // [n_splits][heads_in_call*nq][2+P]        (n_splits  > 1)
  int head0, heads_in_call, nq;
  int n, n_splits, span; // span: tokens per split, multiple of 64
  int force_partial;     // write the partial even when there is a single span
  int *status;
  // n_splits > 1 with fused merge: the helper warp that completes a (head, query)'s last
  // span merges all of them inside the launch
  int *counters;         // [heads_in_call*nq] arrival counts, zero before and after every launch (nullptr: no fused merge)
  float *final_out;      // outputs, or combined partials when final_to_partial
  int final_to_partial;
  // Peer exchange (sequence sharded over GPUs): instead of final_out, the combined partial of
  // item i goes to peer_out[r] + (my_rank*items + i)*(2+P) for every rank r (plain stores over
  // NVLink; r == my_rank is this GPU's own buffer), followed by a system-scope add of 1 to
  // peer_flag[r][my_rank], which the receiving rank's merge kernel waits for.
  int n_peers, my_rank;
  float *peer_out[8];
  unsigned int *peer_flag[8];
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CS_CONSUMERS) : "memory"); }
// Not volatile: the address always derives from data loaded after the
// barrier that published it, so the compiler is free to schedule these.
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void red_shared_add(uint32_t addr, uint32_t v) {
  asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// exp(x) for x <= 0 from the hardware 2^t unit, with the rounding error of
// t = x*log2(e) (and the part of log2(e) a float cannot hold) put back through
// exp(x) = 2^t * (1 + r*ln 2): relative error ~2^-22, a third of the instructions of expf.
// Arguments below -200 (the result underflows long before) are clamped so that
// -inf gives 0 instead of inf - inf; NaN stays NaN.
__device__ __forceinline__ float exp_nonpos(float x) {
  const float L2E_HI = 1.4426950216293335f, L2E_LO = 1.9259629911266175e-8f;
  x = x < -200.f ? -200.f : x;
  const float t = x * L2E_HI;
  const float r = fmaf(x, L2E_HI, -t) + x * L2E_LO;
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t));
  return fmaf(e, r * 0.6931471805599453f, e);
}

// Block-wide reductions over the consumer threads with ONE barrier each.  The
// max and the sums use different arrays and alternate within an item, so an
// array is rewritten only after a later barrier has passed every reader.
__device__ __forceinline__ float consumer_max(float v, float *red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  if (lane == 0) red[warp] = v;
  consumer_sync();
  static_assert(CS_WARPS == 16, "four 128-bit reads cover the per-warp values");
  const float4 *r4 = reinterpret_cast<const float4 *>(red);
  const float4 a = r4[0], b = r4[1], c = r4[2], d = r4[3];
  return fmaxf(fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w))),
               fmaxf(fmaxf(fmaxf(c.x, c.y), fmaxf(c.z, c.w)), fmaxf(fmaxf(d.x, d.y), fmaxf(d.z, d.w))));
}
__device__ __forceinline__ void consumer_sum2(float &a, float &b, float *red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  if (lane == 0) { red[warp] = a; red[32 + warp] = b; }
  consumer_sync();
  // the same left-to-right order in every thread, so all threads hold identical sums
  const float4 *r4 = reinterpret_cast<const float4 *>(red);
  a = 0.f;
  b = 0.f;
#pragma unroll
  for (int i = 0; i < CS_WARPS / 4; ++i) {
    const float4 x = r4[i], y = r4[8 + i];
    a = (((a + x.x) + x.y) + x.z) + x.w;
    b = (((b + y.x) + y.y) + y.z) + y.w;
  }
}

// Sum STEPS per-lane partials across the 8 lanes of a token group so that
// each lane ends with complete sums; returns the value this lane owns and the
// step it belongs to (8 steps: lane wl owns step wl; 4 steps: lanes wl, wl^1
// own step wl>>1).
template <int STEPS>
__device__ __forceinline__ float group_transpose_sum(float (&v)[STEPS], int wl) {
  static_assert(STEPS == 4 || STEPS == 8, "4 or 8 steps");
  int cnt = STEPS;
#pragma unroll
  for (int off = 4; off >= 1; off >>= 1) {
    if (cnt > 1) {
      const int half = cnt >> 1;
      const bool up = (wl & off) != 0;
#pragma unroll
      for (int i = 0; i < STEPS / 2; ++i) {
        if (i < half) {
          float keep = up ? v[i + half] : v[i];
          float send = up ? v[i] : v[i + half];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
      }
      cnt = half;
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
    }
  }
  return v[0];
}

// The same over the 4 lanes of a token group: 4 steps -> lane wl owns step wl;
// 2 steps -> lanes 2*s and 2*s+1 both end with step s.
template <int STEPS>
__device__ __forceinline__ float quad_transpose_sum(float (&v)[STEPS], int wl) {
  static_assert(STEPS == 2 || STEPS == 4, "2 or 4 steps");
  const bool up2 = (wl & 2) != 0, up1 = (wl & 1) != 0;
  if constexpr (STEPS == 4) {
    const float k0 = up2 ? v[2] : v[0], s0 = up2 ? v[0] : v[2];
    const float k1 = up2 ? v[3] : v[1], s1 = up2 ? v[1] : v[3];
    const float x0 = k0 + __shfl_xor_sync(0xffffffffu, s0, 2);
    const float x1 = k1 + __shfl_xor_sync(0xffffffffu, s1, 2);
    const float k = up1 ? x1 : x0, s = up1 ? x0 : x1;
    return k + __shfl_xor_sync(0xffffffffu, s, 1);
  } else {
    const float k = up2 ? v[1] : v[0], s = up2 ? v[0] : v[1];
    const float x = k + __shfl_xor_sync(0xffffffffu, s, 2);
    return x + __shfl_xor_sync(0xffffffffu, x, 1);
  }
}

// KB/VB: bits; KW/VW: 32-bit words per packed row (8 or 16; 6 or 12 for 3-bit keys).
template <int KB, int KW, int VB, int VW>
__device__ __forceinline__ void compute_stream_body(const StreamLaunch &a) {
  constexpr int P = KW * 32 / KB;
  static_assert(P == VW * 32 / VB, "K and V rows must describe the same padded dimension");
  constexpr bool K3 = KB == 3;
  static_assert(!K3 || KW == 6 || KW == 12, "3-bit keys: padded dimension 64 or 128");
  constexpr int KROW = KW * 4, VROW = VW * 4;
  // tokens per stage; 3-bit rows (24 or 48 bytes) fill 12 KB of a stage with a power of two of tokens
  constexpr bool V3 = VB == 3;
  static_assert(!V3 || VW == 6 || VW == 12, "3-bit values: padded dimension 64 or 128");
  constexpr int TKN = K3 ? 12288 / KROW : CS_STAGE_BYTES / KROW, TVN = V3 ? 12288 / VROW : CS_STAGE_BYTES / VROW;
  // Lanes that share a token in the K stream: 4 with 32-byte rows, 8 with 64-byte rows
  // (measured: fewer shuffles pay with the short rows, not with the long ones); with 3-bit keys
  // every lane takes three words (four 3-byte groups = 32 coordinates) of the row.
  constexpr int KLPT = K3 ? KW / 3 : (KW == 16 ? 8 : 4);
  constexpr int KTPS = 32 / KLPT;                                           // tokens per warp step (K)
  // V stream: 8 lanes per token (4 tokens per warp step); 4 lanes and 8 tokens with 16-byte rows
  constexpr int VLPT = V3 ? VW / 3 : (VW >= 8 ? 8 : 4);
  constexpr int VTPS = 32 / VLPT;
  constexpr int KSTEPS = TKN / CS_WARPS / KTPS, VSTEPS = TVN / CS_WARPS / VTPS;
  constexpr int KWPL = KW / KLPT, VWPL = VW / VLPT;                         // words per lane
  constexpr int KC = KW * 4, VC = VW * 4;                                   // byte columns
  constexpr int KE = 8 / KB, VE = 8 / VB;                                   // coordinates per byte
  // 32 byte columns (2-bit V at dim 128, 4-bit at dim 64): bucket rows of 32 columns (128 bytes),
  // which leaves room for two more ring stages; the address is formed doubled and shifted back
  // 16 byte columns (2-bit V at dim 64): the same 128-byte rows hold TWO copies of the 16 columns
  // side by side -- tokens 0..3 of a warp step add into the first, tokens 4..7 into the second --
  // so the 32 lanes of a reduction still fall on 32 different banks; the fold adds the copies.
  // 3-bit values: buckets by 6-bit field, bucket[copy][field value][field column], four
  // column-rotated copies of 64 x 64 like the 3-bit key table (64 KB).
  constexpr bool TWOCOPY = !V3 && VC == 16;
  constexpr bool COMPACT = !V3 && (VC == 32 || TWOCOPY);
  constexpr int VCOLS = TWOCOPY ? 32 : VC;                                 // bucket columns, copies included
  constexpr int BUCKET_BYTES = COMPACT ? 32768 : CS_TABLE_BYTES;           // [256][32 or 64] 32-bit buckets

  extern __shared__ __align__(1024) unsigned char smem_stream[];
  unsigned char *smem = smem_stream;
  const uint32_t base = smem_u32(smem);
  const uint32_t table_addr = (base + 65535u) & ~65535u; // 64 KB aligned: low 16 address bits are free
  const uint32_t front = table_addr - base;
  unsigned char *table_p = smem + front;
  const uint32_t bucket_addr = table_addr + CS_TABLE_BYTES;
  uint32_t *bucket = reinterpret_cast<uint32_t *>(table_p + CS_TABLE_BYTES);
  float *sc = reinterpret_cast<float *>(table_p + CS_TABLE_BYTES + BUCKET_BYTES);
  unsigned char *misc = reinterpret_cast<unsigned char *>(sc + CS_SPAN_MAX);
  constexpr int ACC_PITCH = 132;                         // P accumulators + running max + sum
  float *qrot = reinterpret_cast<float *>(misc);         // 2 x 128: rotated queries, double-buffered
  float *accb = qrot + 256;                              // 2 x ACC_PITCH: finished items for the helper warp
  float *red_max = accb + 2 * ACC_PITCH;                 // 32 floats
  float *red_sum = red_max + 32;                         // 64 floats
  float *s_cb = red_sum + 64;                            // 16 floats: V centroids
  uint64_t *full = reinterpret_cast<uint64_t *>(s_cb + 16);
  uint64_t *empty = full + CS_MAX_STAGES;
  uint64_t *qfull = empty + CS_MAX_STAGES;               // [2] rotated query written / table built from it
  uint64_t *qempty = qfull + 2;
  uint64_t *afull = qempty + 2;                          // [2] accumulator handed over / stored
  uint64_t *aempty = afull + 2;
  int *s_fail = reinterpret_cast<int *>(aempty + 2);
  // The ring lives in whatever is left: the slack in front of the 64 KB-aligned
  // table and the tail behind the misc block.
  unsigned char *back = misc + CS_MISC_BYTES;
  const int back_bytes = (int)(CS_SMEM_BYTES - front - CS_TABLE_BYTES - BUCKET_BYTES - CS_SPAN_MAX * 4 - CS_MISC_BYTES);
  int n_front = min((int)(front / CS_STAGE_BYTES), CS_MAX_STAGES);
  int n_back = min(back_bytes / CS_STAGE_BYTES, CS_MAX_STAGES - n_front);
  // Each K stage comes with its tokens' K scales (a second bulk copy on the same
  // barrier).  They go into what the stages leave over, or take a stage's place.
  constexpr int KS_STAGE_BYTES = TKN * 4;
  constexpr int KS_AREA_BYTES = CS_MAX_STAGES * KS_STAGE_BYTES;
  unsigned char *ks_area;
  if ((int)front - n_front * CS_STAGE_BYTES >= KS_AREA_BYTES) {
    ks_area = smem + (size_t)n_front * CS_STAGE_BYTES;
  } else if (back_bytes - n_back * CS_STAGE_BYTES >= KS_AREA_BYTES) {
    ks_area = back + (size_t)n_back * CS_STAGE_BYTES;
  } else if (n_back > 0) {
    --n_back;
    ks_area = back + (size_t)n_back * CS_STAGE_BYTES;
  } else {
    n_front = max(n_front - 1, 0);
    ks_area = smem + (size_t)n_front * CS_STAGE_BYTES;
  }
  const int n_stages = n_front + n_back;
  const bool layout_ok = n_stages >= 2;
  auto stage_ptr = [&](int s) -> unsigned char * {
    return s < n_front ? smem + (size_t)s * CS_STAGE_BYTES : back + (size_t)(s - n_front) * CS_STAGE_BYTES;
  };

  const int tid = threadIdx.x;
  const CacheView &c = a.c;
  const int dim = c.dim;
  const int items_base = a.heads_in_call * a.nq;
  const int n_items = items_base * a.n_splits;
  // A block owns a contiguous run of items, so the spans of one (head, query)
  // follow each other and share the query rotation and the K table.
  const int item_begin = (int)((long long)blockIdx.x * n_items / gridDim.x);
  const int item_end = (int)((long long)(blockIdx.x + 1) * n_items / gridDim.x);

  if (tid == 0) {
    for (int s = 0; s < CS_MAX_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CS_WARPS);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qfull[s], 1);
      mbar_init(&qempty[s], 1);
      mbar_init(&afull[s], P / 32);
      mbar_init(&aempty[s], 1);
    }
    *s_fail = layout_ok ? 0 : 2;
    for (int i = 0; i < 16; ++i) s_cb[i] = c_cb[VB - 2][i];
    fence_barrier_init();
  }
  __syncthreads();
  if (!layout_ok) {
    if (tid == 0) atomicExch(a.status, 2);
    return;
  }

  // Every wait in this kernel is bounded; a wait that gives up raises the
  // block's failure flag, after which all later waits are skipped and the
  // block drains (the host reads the status word and reports the call as failed).
  auto guarded_wait = [&](uint64_t *bar, uint32_t parity) {
    if (*reinterpret_cast<volatile int *>(s_fail) == 0 && !mbar_wait(bar, parity)) {
      *reinterpret_cast<volatile int *>(s_fail) = 1;
      atomicExch(a.status, 1);
    }
  };
  constexpr int EPL = P / 32; // query / accumulator elements per lane of the helper warp
  const float isp = 1.f / sqrtf((float)P);

  // ======================= producer warp ====================================
  if (tid >= CS_CONSUMERS && tid < CS_HELPER_TID) {
    if (tid != CS_CONSUMERS) return;
    griddep_wait(); // everything the cache holds is read through this thread's copies
    int stage = 0;
    uint32_t phase = 0;
    for (int item = item_begin; item < item_end; ++item) {
      const int split = item % a.n_splits, hq = item / a.n_splits;
      const int h = a.head0 + hq / a.nq;
      const int t0 = min(a.n, split * a.span), t1 = min(a.n, t0 + a.span);
      const uint8_t *kb = c.k_slab + (size_t)h * c.k_stride;
      const uint8_t *vb = c.v_slab + (size_t)h * c.v_stride;
      const float *ksb = c.k_scale + (size_t)h * c.s_stride;
      const uint8_t *vsb = reinterpret_cast<const uint8_t *>(c.v_scale + (size_t)h * c.s_stride);
      // three passes over the span: K rows (with their scales), the V scales as
      // plain 16 KB tiles for the softmax phase, then the V rows
      for (int pass = 0; pass < 3; ++pass) {
        const int rowb = pass == 0 ? KROW : pass == 1 ? 4 : VROW;
        const int tn = pass == 0 ? TKN : pass == 1 ? CS_STAGE_BYTES / 4 : TVN;
        const uint8_t *src = pass == 0 ? kb : pass == 1 ? vsb : vb;
        for (int t = t0; t < t1; t += tn) {
          if (*reinterpret_cast<volatile int *>(s_fail) == 0 && !mbar_wait(&empty[stage], phase ^ 1u)) {
            *reinterpret_cast<volatile int *>(s_fail) = 1;
            atomicExch(a.status, 1);
          }
          const int cnt = min(tn, t1 - t);
          const uint32_t bytes = ((uint32_t)(cnt * rowb) + 15u) & ~15u;
          // scales: rounded up to 16 bytes; the per-head scale rows carry 128 bytes of padding
          const uint32_t sbytes = pass ? 0u : (((uint32_t)cnt * 4u + 15u) & ~15u);
          // a copy may run into the 128-byte slack behind a head's rows, never past it
          if (!AQ_CHECK(a.status, (size_t)t * rowb + bytes <= (pass == 0 ? c.k_stride : pass == 1 ? (size_t)c.s_stride * 4 : c.v_stride) &&
                                      h >= 0 && h < c.n_heads, 13)) {
            *reinterpret_cast<volatile int *>(s_fail) = 1; // consumers stop waiting; the block drains
            return;
          }
          mbar_expect_tx(&full[stage], bytes + sbytes);
          bulk_g2s(stage_ptr(stage), src + (size_t)t * rowb, bytes, &full[stage]);
          if (sbytes) bulk_g2s(ks_area + (size_t)stage * KS_STAGE_BYTES, ksb + t, sbytes, &full[stage]);
          if (++stage == n_stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    return;
  }

  // ======================= helper warp ======================================
  // prologue(i): rotate the query of item i (attention.cpp:537-550) into
  // qrot[buffer] unless item i continues the previous item's (head, query).
  // epilogue(i): take the finished accumulator of item i, then either store the
  // split-KV partial or normalise, apply the inverse transform
  // (core/fwht.cpp:106-134) and store the output.
  // Order: prologue(first), then for every item prologue(i+1) before epilogue(i).
  if (tid >= CS_HELPER_TID) {
    const int lane = tid & 31;
    int prev_hq = -1, qcount = 0;
    uint32_t sg_latest = 0;
    auto prologue = [&](int item) {
      const int hq = item / a.n_splits;
      if (hq == prev_hq) return;
      prev_hq = hq;
      const float *qp = a.q + (size_t)hq * dim;
      float v[EPL];
      float part = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        v[e] = (EPL * lane + e) < dim ? __ldg(qp + EPL * lane + e) : 0.f;
        part += v[e] * v[e];
      }
      const uint32_t sg = __ldg(c.signs + (size_t)(a.head0 + hq / a.nq) * c.sign_words + ((EPL * lane) >> 5));
      const float qn = sqrtf(warp_sum(part) + 1e-12f);
      const float inv = 1.f / qn;
#pragma unroll
      for (int e = 0; e < EPL; ++e) v[e] = v[e] * inv * (((sg >> ((EPL * lane + e) & 31)) & 1u) ? -1.f : 1.f);
      warp_butterflies<EPL>(v, lane);
      const float back = sqrtf((float)P) * qn;
      const int b = qcount & 1;
      guarded_wait(&qempty[b], (((uint32_t)qcount >> 1) & 1u) ^ 1u); // the table of two queries ago is built
#pragma unroll
      for (int e = 0; e < EPL; ++e) qrot[b * 128 + EPL * lane + e] = v[e] * isp * back;
      sg_latest = sg;
      ++qcount;
      __syncwarp();
      if (lane == 0) mbar_arrive(&qfull[b]);
    };
    // Combined partial of item hq -> every rank's gather buffer, then one count per rank.
    auto deliver_to_peers = [&](int hq, float M, float L, const float (&acc)[EPL]) {
      for (int r = 0; r < a.n_peers; ++r) {
        float *po = a.peer_out[r] + ((size_t)a.my_rank * items_base + hq) * (size_t)(2 + P);
        if (lane == 0) { po[0] = M; po[1] = L; }
#pragma unroll
        for (int e = 0; e < EPL; ++e) po[2 + EPL * lane + e] = acc[e];
      }
      // The counts move with release semantics at system scope: the warp barrier orders every
      // lane's stores before the releasing lanes, and a release is cumulative, so whoever
      // acquires the new count also sees the partial.
      __syncwarp();
      if (lane < a.n_peers)
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(a.peer_flag[lane] + a.my_rank) : "memory");
    };
    if (item_begin < item_end) prologue(item_begin);
    for (int item = item_begin, idx = 0; item < item_end; ++item, ++idx) {
      const uint32_t sg = sg_latest;
      if (item + 1 < item_end) prologue(item + 1);
      const int b = idx & 1;
      guarded_wait(&afull[b], ((uint32_t)idx >> 1) & 1u);
      const float *ab = accb + b * ACC_PITCH;
      const int split = item % a.n_splits, hq = item / a.n_splits;
      float v[EPL];
#pragma unroll
      for (int e = 0; e < EPL; ++e) v[e] = ab[EPL * lane + e];
      const float mx = ab[P], ls = ab[P + 1];
      __syncwarp();
      if (lane == 0) mbar_arrive(&aempty[b]); // values are in registers: the slot may be refilled
      if (a.n_peers > 0 && a.n_splits == 1) { // a single span already is the combined partial
        deliver_to_peers(hq, mx, ls, v);
      } else if (a.n_splits > 1 || a.force_partial) {
        float *pp = a.partial + ((size_t)split * items_base + hq) * (size_t)(2 + P);
        if (!AQ_CHECK(a.status, split < a.n_splits && hq < items_base, 14)) continue;
        if (lane == 0) { pp[0] = mx; pp[1] = ls; }
#pragma unroll
        for (int e = 0; e < EPL; ++e) pp[2 + EPL * lane + e] = v[e];
        if (a.counters != nullptr && a.n_splits > 1) {
          // Whoever brings the count to n_splits merges (nobody waits for anybody) and
          // puts the count back to zero for the next launch.
          __threadfence();
          __syncwarp();
          int ticket = 0;
          if (lane == 0) ticket = atomicAdd(&a.counters[hq], 1);
          ticket = __shfl_sync(0xffffffffu, ticket, 0);
          if (ticket == a.n_splits - 1) {
            if (lane == 0) a.counters[hq] = 0;
            __threadfence();
            const size_t pstride = (size_t)items_base * (size_t)(2 + P);
            const float *base = a.partial + (size_t)hq * (size_t)(2 + P);
            // same rules as merge_partials_block: NaN sums and zero weights travel as
            // they do upstream; every span of this launch holds tokens, so none is skipped
            float M = -INFINITY;
            for (int p = lane; p < a.n_splits; p += 32) M = fmaxf(M, __ldcg(base + (size_t)p * pstride));
            M = warp_max(M);
            float L = 0.f, am[EPL];
#pragma unroll
            for (int e = 0; e < EPL; ++e) am[e] = 0.f;
            for (int p0 = 0; p0 < a.n_splits; p0 += 32) {
              const int p = p0 + lane;
              float w = 0.f;
              if (p < a.n_splits) {
                const float *q2 = base + (size_t)p * pstride;
                w = expf(__ldcg(q2) - M);
                L += __ldcg(q2 + 1) * w;
              }
              const int cnt = min(32, a.n_splits - p0);
#pragma unroll 8
              for (int j = 0; j < cnt; ++j) {
                const float wj = __shfl_sync(0xffffffffu, w, j);
                const float2 *row = reinterpret_cast<const float2 *>(base + (size_t)(p0 + j) * pstride + 2 + EPL * lane);
#pragma unroll
                for (int e = 0; e < EPL / 2; ++e) {
                  const float2 x = __ldcg(row + e);
                  am[2 * e] += wj * x.x;
                  am[2 * e + 1] += wj * x.y;
                }
              }
            }
            L = warp_sum(L);
            if (a.n_peers > 0) {
              deliver_to_peers(hq, M, L, am);
            } else if (a.final_to_partial) {
              float *po = a.final_out + (size_t)hq * (size_t)(2 + P);
              if (lane == 0) { po[0] = M; po[1] = L; }
#pragma unroll
              for (int e = 0; e < EPL; ++e) po[2 + EPL * lane + e] = am[e];
            } else {
              const float invl = 1.f / L;
#pragma unroll
              for (int e = 0; e < EPL; ++e) am[e] *= invl;
              warp_butterflies<EPL>(am, lane);
#pragma unroll
              for (int e = 0; e < EPL; ++e) {
                const int j = EPL * lane + e;
                if (j < dim) a.final_out[(size_t)hq * dim + j] = am[e] * isp * (((sg >> (j & 31)) & 1u) ? -1.f : 1.f);
              }
            }
          }
        }
      } else {
        const float invl = 1.f / ls;
#pragma unroll
        for (int e = 0; e < EPL; ++e) v[e] *= invl;
        warp_butterflies<EPL>(v, lane);
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          const int j = EPL * lane + e;
          if (j < dim) a.out[(size_t)hq * dim + j] = v[e] * isp * (((sg >> (j & 31)) & 1u) ? -1.f : 1.f);
        }
      }
    }
    return;
  }

  // ======================= consumer warps ===================================
  const int lane = tid & 31, warp = tid >> 5;
  const int tq = lane >> 3, wl = lane & 7;
  // Per-lane constants.  The lane reads word kword[m] of its token's row and
  // visits that word's four bytes in the rotated order (k + tq) & 3, which puts
  // the 32 lanes of a warp on 32 different banks of the table / bucket arrays.
  // K stream with four lanes per token (lane = 4*kg + kwl, kg = token within the
  // step): the lane takes words kwl + 4*j of the row, in an order rotated by the
  // token, so that the 32 data-word reads of a step and the 32 table reads of a
  // byte position each fall on 32 different banks.
  const int kg = K3 ? (int)((unsigned)lane / KLPT) : (KLPT == 4 ? lane >> 2 : tq), kwl = K3 ? (int)((unsigned)lane % KLPT) : (KLPT == 4 ? lane & 3 : wl);
  int kword[KWPL], vword[VWPL];
  uint32_t ksel[4], kselk[4], kconst[KWPL][4], vconst[VWPL][4];
#pragma unroll
  for (int m = 0; m < KWPL; ++m) {
    if (K3) kword[m] = 3 * kwl + m;
    else if (KLPT == 4) kword[m] = KW == 16 ? kwl + 4 * ((m + (kg >> 1)) & 3) : kwl + 4 * ((m + (kg >> 2)) & 1);
    else kword[m] = KWPL == 1 ? wl : ((wl + 8 * (tq >> 1) + 8 * m) & 15);
  }
  // 3-bit keys.  A row is a string of 6-bit fields (two coordinates each); the table is
  // T[field value][field column], 64 x 64 floats, kept in FOUR copies whose columns are rotated
  // by 4*copy positions.  A lane walks its four 3-byte groups in the stored order and the four
  // fields of a group in an order rotated by k3rf; with the copy chosen by the token the 32
  // lanes of a warp step read 32 different banks:
  //   bank = (16*(kwl & 1) + 4*((group + copy) & 3) + ((field + k3rf) & 3)) mod 32,
  // and (kwl & 1, copy, k3rf) runs over all 32 combinations across the lanes.
  const int k3copy = kg & 3;
  const int k3rf = KLPT == 4 ? 2 * (kwl >> 1) + (kg >> 2) : (kg >> 2);
  uint32_t k3shr[4], k3const[4][4];
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int ff = (b + k3rf) & 3;
    k3shr[b] = 18 - 6 * ff; // group value in bits 8..31: field ff sits at bit 26 - 6*ff, wanted at bit 8
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int pos = (16 * kwl + 4 * g + ff + 4 * k3copy) & (P / 2 - 1);
      k3const[g][b] = table_addr | (uint32_t)(k3copy << 14) | (uint32_t)(pos << 2);
    }
  }
  const int krot = KLPT == 4 ? (KW == 16 ? (kg & 1) + 2 * (kg >> 2) : (kg & 3)) : tq;
  // V stream lane roles: token vg of the warp step, word slot vwl of its row
  const int vg = V3 ? (int)((unsigned)lane / VLPT) : (VLPT == 4 ? lane >> 2 : tq), vwl = V3 ? (int)((unsigned)lane % VLPT) : (VLPT == 4 ? lane & 3 : wl);
#pragma unroll
  for (int m = 0; m < VWPL; ++m) vword[m] = V3 ? 3 * vwl + m : (VWPL == 1 ? vwl : ((wl + 8 * (tq >> 1) + 8 * m) & 15));
  // 3-bit values: the same lane roles and bank argument as for 3-bit keys, on the buckets
  const int v3copy = vg & 3;
  const int v3rf = VLPT == 4 ? 2 * (vwl >> 1) + (vg >> 2) : (vg >> 2);
  uint32_t v3shr[4], v3const[4][4];
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int ff = (b + v3rf) & 3;
    v3shr[b] = 18 - 6 * ff;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int pos = (16 * vwl + 4 * g + ff + 4 * v3copy) & (P / 2 - 1);
      v3const[g][b] = bucket_addr | (uint32_t)(v3copy << 14) | (uint32_t)(pos << 2);
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int kk = (k + vg) & 3;
    ksel[k] = 0x7604u | ((uint32_t)kk << 4); // result = {const.b0, data.byte[kk], const.b2, const.b3}
    const int kkk = (k + krot) & 3;
    kselk[k] = 0x7604u | ((uint32_t)kkk << 4);
#pragma unroll
    for (int m = 0; m < KWPL; ++m) kconst[m][k] = table_addr | (uint32_t)((4 * kword[m] + kkk) << 2);
#pragma unroll
    // bucket rows are 64 columns (256 bytes), so the packed byte lands in address
    // bits 8..15 with one byte-permute
    for (int m = 0; m < VWPL; ++m) {
      const int column = (TWOCOPY ? 16 * (vg >> 2) : 0) + 4 * vword[m] + kk;
      vconst[m][k] = COMPACT ? ((bucket_addr << 1) | (uint32_t)(column << 3)) : (bucket_addr | (uint32_t)(column << 2));
    }
  }
  float *table = reinterpret_cast<float *>(table_p);
  const float *kcb = c_cb[KB - 2];
  const float attn_s = 1.f / (sqrtf((float)dim) * (float)P);

  int stage = 0;
  uint32_t phase = 0;
  bool next_ready = false;
  // Poll the barrier of the stage after the current one without blocking; the
  // answer is used by the next wait_full(), so the poll's latency (it queues
  // behind the table reads) overlaps this tile's arithmetic.
  auto peek_next = [&]() {
    const int ns = stage + 1 == n_stages ? 0 : stage + 1;
    const uint32_t np = stage + 1 == n_stages ? phase ^ 1u : phase;
    next_ready = mbar_test(&full[ns], np);
  };
  auto wait_full = [&]() {
    // The stage was already tested (peek_next) while the previous tile was being
    // processed; only a stage that had not landed by then is waited for here.
    if (!next_ready && *reinterpret_cast<volatile int *>(s_fail) == 0 && !mbar_wait(&full[stage], phase)) {
      *reinterpret_cast<volatile int *>(s_fail) = 1;
      atomicExch(a.status, 1);
    }
  };
  auto release = [&]() {
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);
    if (++stage == n_stages) { stage = 0; phase ^= 1u; }
  };

  // The buckets start at zero; afterwards the fold that reads a bucket clears it.
  for (int i = tid; i < BUCKET_BYTES / 4; i += CS_CONSUMERS) bucket[i] = 0u;
  int prev_hq = -1, quse = 0;
  for (int item = item_begin, idx = 0; item < item_end; ++item, ++idx) {
    const int split = item % a.n_splits, hq = item / a.n_splits;
    const int t0 = min(a.n, split * a.span), t1 = min(a.n, t0 + a.span);
    const int len = t1 - t0;

    if (hq == prev_hq) {
      // same (head, query) as the previous item: the table stands.  The barrier keeps
      // this item's score writes behind the last fold reads of the previous item.
      consumer_sync();
    } else {
    prev_hq = hq;
    const int qb = quse & 1;
    guarded_wait(&qfull[qb], ((uint32_t)quse >> 1) & 1u);
    ++quse;
    const float *qr = qrot + qb * 128;
    // ---- build the K byte table ----------------------------------------------------
    {
      // thread -> column (consecutive lanes, consecutive banks), a slice of the byte values;
      // with 32 byte columns (2-bit keys at dim 128, 4-bit at dim 64) the threads split the byte
      // values 16 ways instead of 8 so that none is idle
      constexpr int TCOLS = (!K3 && KC == 32) ? 32 : 64;
      constexpr int HPT = 16 / (CS_CONSUMERS / TCOLS); // high-nibble values per thread
      const int col = tid & (TCOLS - 1), bq = TCOLS == 32 ? tid >> 5 : tid >> 6;
      if constexpr (K3) {
        // thread -> field column and the first coordinate's level (bq = 0..7); all four copies
        if (col < P / 2) {
          const float q0 = qr[2 * col], q1 = qr[2 * col + 1];
          const float av = q0 * kcb[bq];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float val = av + q1 * kcb[i];
#pragma unroll
            for (int cp = 0; cp < 4; ++cp)
              table[cp * 4096 + (bq * 8 + i) * 64 + ((col + 4 * cp) & (P / 2 - 1))] = val;
          }
        }
      } else if (col < KC) {
        if (KE == 2) {
          float lo[16];
          const float q0 = qr[2 * col], q1 = qr[2 * col + 1];
#pragma unroll
          for (int i = 0; i < 16; ++i) lo[i] = q1 * kcb[i];
#pragma unroll
          for (int hi = 0; hi < HPT; ++hi) {
            const int hv = bq * HPT + hi;
            const float av = q0 * kcb[hv];
#pragma unroll
            for (int i = 0; i < 16; ++i) table[(hv * 16 + i) * 64 + col] = av + lo[i];
          }
        } else { // 4 two-bit coordinates per byte, first coordinate in the top bits
          float t23[16];
          const float q0 = qr[4 * col], q1 = qr[4 * col + 1], q2 = qr[4 * col + 2], q3 = qr[4 * col + 3];
#pragma unroll
          for (int i = 0; i < 16; ++i) t23[i] = q2 * kcb[i >> 2] + q3 * kcb[i & 3];
#pragma unroll
          for (int hi = 0; hi < HPT; ++hi) {
            const int hv = bq * HPT + hi;
            const float t01 = q0 * kcb[hv >> 2] + q1 * kcb[hv & 3];
#pragma unroll
            for (int i = 0; i < 16; ++i) table[(hv * 16 + i) * 64 + col] = t01 + t23[i];
          }
        }
      }
    }
    consumer_sync();
    if (tid == 0) mbar_arrive(&qempty[qb]); // every thread has read the rotated query
    }
    // ---- K stream: logits into sc[] ----------------------------------------------------
    // After the group reduction one lane per token owns its dot product; that lane
    // also reads the token's K scale (it arrived with the stage) and keeps a running
    // maximum, so no separate scaling pass is needed.
    // which token of the warp's slice this lane owns after the group reduction
    const int own_step = KLPT == 2 ? kwl : KLPT == 4 ? (KSTEPS == 4 ? kwl : (kwl >> 1)) : (KSTEPS == 8 ? wl : (wl >> 1));
    const bool owner = KLPT == 2 ? true : KLPT == 4 ? (KSTEPS == 4 || (kwl & 1) == 0) : (KSTEPS == 8 || (wl & 1) == 0);
    const int own_tok = warp * (TKN / CS_WARPS) + KTPS * own_step + kg;
    float lane_max = -1e30f; // where upstream's running maximum starts (attention.cpp:384)
    for (int t = t0; t < t1; t += TKN) {
      wait_full();
      const uint32_t *stw = reinterpret_cast<const uint32_t *>(stage_ptr(stage));
      const bool own_valid = owner && t + own_tok < t1;
      const float ksv = own_valid ? reinterpret_cast<const float *>(ks_area + (size_t)stage * KS_STAGE_BYTES)[own_tok] : 0.f;
      uint32_t dk[KSTEPS][KWPL];
#pragma unroll
      for (int s = 0; s < KSTEPS; ++s) {
        const int tok = warp * (TKN / CS_WARPS) + KTPS * s + kg; // token within the stage
#pragma unroll
        for (int m = 0; m < KWPL; ++m) dk[s][m] = stw[tok * KW + kword[m]];
      }
      peek_next();
      float pv[KSTEPS];
#pragma unroll
      for (int s = 0; s < KSTEPS; ++s) {
        float a0 = 0.f, a1 = 0.f;
        if constexpr (K3) {
          // the lane's four 3-byte groups, big-endian, in bits 8..31 (the low byte is never used)
          uint32_t g3[4];
          g3[0] = __byte_perm(dk[s][0], 0u, 0x0124);
          g3[1] = __byte_perm(dk[s][0], dk[s][1], 0x3450);
          g3[2] = __byte_perm(dk[s][1], dk[s][2], 0x2340);
          g3[3] = __byte_perm(dk[s][2], 0u, 0x1230);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            a0 += lds_f32(((g3[g] >> k3shr[0]) & 0x3F00u) | k3const[g][0]);
            a1 += lds_f32(((g3[g] >> k3shr[1]) & 0x3F00u) | k3const[g][1]);
            a0 += lds_f32(((g3[g] >> k3shr[2]) & 0x3F00u) | k3const[g][2]);
            a1 += lds_f32(((g3[g] >> k3shr[3]) & 0x3F00u) | k3const[g][3]);
          }
        } else {
#pragma unroll
          for (int m = 0; m < KWPL; ++m) {
            const uint32_t d = dk[s][m];
            a0 += lds_f32(__byte_perm(d, kconst[m][0], kselk[0]));
            a1 += lds_f32(__byte_perm(d, kconst[m][1], kselk[1]));
            a0 += lds_f32(__byte_perm(d, kconst[m][2], kselk[2]));
            a1 += lds_f32(__byte_perm(d, kconst[m][3], kselk[3]));
          }
        }
        pv[s] = a0 + a1;
      }
      float total;
      if constexpr (KLPT == 2) { // lane kwl keeps step kwl
        const float keep = kwl ? pv[1] : pv[0], send = kwl ? pv[0] : pv[1];
        total = keep + __shfl_xor_sync(0xffffffffu, send, 1);
      } else if constexpr (KLPT == 4) total = quad_transpose_sum<KSTEPS>(pv, kwl);
      else total = group_transpose_sum<KSTEPS>(pv, wl);
      if (own_valid) {
        const float logit = total * attn_s * ksv;
        sc[t - t0 + own_tok] = logit;
        lane_max = fmaxf(lane_max, logit);
      }
      release();
    }
    // ---- exact two-pass softmax over the span ------------------------------------------
    // Each thread owns tokens tid, tid+512, ...; their V scales come through the
    // ring (4096 per stage) and every intermediate stays in registers.
    constexpr int NPT = CS_SPAN_MAX / CS_CONSUMERS;
    constexpr int SCT = CS_STAGE_BYTES / 4;       // scales per stage
    constexpr int RPS = SCT / CS_CONSUMERS;       // ... = this many of a thread's tokens
    float sv[NPT], vv[NPT];
#pragma unroll
    for (int cchunk = 0; cchunk < NPT / RPS; ++cchunk) {
      if (cchunk * SCT < len) {
        wait_full();
        const float *vs = reinterpret_cast<const float *>(stage_ptr(stage));
        peek_next();
#pragma unroll
        for (int rr = 0; rr < RPS; ++rr) {
          const int r = cchunk * RPS + rr;
          vv[r] = tid + r * CS_CONSUMERS < len ? vs[tid + rr * CS_CONSUMERS] : 0.f;
        }
        release();
      } else {
#pragma unroll
        for (int rr = 0; rr < RPS; ++rr) vv[cchunk * RPS + rr] = 0.f;
      }
    }
    const float mx = consumer_max(lane_max, red_max); // its barrier also publishes sc[]
#pragma unroll
    for (int r = 0; r < NPT; ++r) {
      const int i = tid + r * CS_CONSUMERS;
      sv[r] = i < len ? sc[i] : -INFINITY;
    }
    float ls = 0.f, wsum = 0.f;
#pragma unroll
    for (int r = 0; r < NPT; ++r) {
      const float e = tid + r * CS_CONSUMERS < len ? exp_nonpos(sv[r] - mx) : 0.f; // padding weighs nothing
      ls += e;
      sv[r] = e * vv[r] * isp;
      wsum += sv[r];
    }
    consumer_sum2(ls, wsum, red_sum);
    // weights -> 32-bit fixed point with the span's total mapped to 2^30, so no
    // bucket can overflow and the rounding error is below 2^-31 of the total per token
    // A total that is NaN or infinite (a NaN logit, an infinite V scale) makes the
    // accumulator NaN, as upstream's floating-point sums would be.
    const float fx = (wsum > 0.f && wsum < INFINITY) ? 1073741824.0f / wsum : 0.f;
    const float inv_fx = fx > 0.f ? wsum * (1.0f / 1073741824.0f) : (wsum == 0.f ? 0.f : __int_as_float(0x7fc00000));
    uint32_t *scu = reinterpret_cast<uint32_t *>(sc);
    const int len_pad = min(CS_SPAN_MAX, (len + TVN - 1) / TVN * TVN);
    // Stored in the order the V stream reads them: the VSTEPS weights that one lane
    // needs from a tile (tokens VTPS*s + vg of its warp's slice) sit side by side, so the
    // lane fetches them with 128-bit loads.
    constexpr int TPWV = TVN / CS_WARPS;
    static_assert(CS_CONSUMERS % TPWV == 0, "a thread's tokens share their place in the warp slice");
    const int rem = tid % TPWV;
    const int shift = (rem % VTPS) * VSTEPS + (rem / VTPS) - rem; // the same for all of this thread's tokens
#pragma unroll
    for (int r = 0; r < NPT; ++r) {
      const int i = tid + r * CS_CONSUMERS;
      if (i < len_pad) scu[i + shift] = __float2uint_rn(sv[r] * fx);
    }
    consumer_sync();
    // ---- V stream: add each token's weight into bucket[byte][column] ---------------------
    for (int t = t0; t < t1; t += TVN) {
      wait_full();
      const uint32_t *stw = reinterpret_cast<const uint32_t *>(stage_ptr(stage));
      uint32_t dv[VSTEPS][VWPL], wv[VSTEPS];
      const uint4 *wp = reinterpret_cast<const uint4 *>(scu + (t - t0) + warp * TPWV + vg * VSTEPS);
      if constexpr (VSTEPS == 2) {
        const uint2 w2 = *reinterpret_cast<const uint2 *>(wp);
        wv[0] = w2.x; wv[1] = w2.y;
      } else {
#pragma unroll
        for (int s4 = 0; s4 < VSTEPS / 4; ++s4) {
          const uint4 w4 = wp[s4];
          wv[4 * s4] = w4.x; wv[4 * s4 + 1] = w4.y; wv[4 * s4 + 2] = w4.z; wv[4 * s4 + 3] = w4.w;
        }
      }
#pragma unroll
      for (int s = 0; s < VSTEPS; ++s) {
        const int tok = warp * TPWV + VTPS * s + vg;
#pragma unroll
        for (int m = 0; m < VWPL; ++m) dv[s][m] = stw[tok * VW + vword[m]];
      }
      peek_next();
#pragma unroll
      for (int s = 0; s < VSTEPS; ++s) {
        if constexpr (V3) {
          uint32_t g3[4];
          g3[0] = __byte_perm(dv[s][0], 0u, 0x0124);
          g3[1] = __byte_perm(dv[s][0], dv[s][1], 0x3450);
          g3[2] = __byte_perm(dv[s][1], dv[s][2], 0x2340);
          g3[3] = __byte_perm(dv[s][2], 0u, 0x1230);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
#pragma unroll
            for (int b = 0; b < 4; ++b) red_shared_add(((g3[g] >> v3shr[b]) & 0x3F00u) | v3const[g][b], wv[s]);
          }
        } else {
#pragma unroll
          for (int m = 0; m < VWPL; ++m) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t ad = __byte_perm(dv[s][m], vconst[m][k], ksel[k]);
              red_shared_add(COMPACT ? (ad >> 1) : ad, wv[s]);
            }
          }
        }
      }
      release();
    }
    consumer_sync();
    // ---- buckets -> rotated-domain accumulator -------------------------------------------
    // acc[j] = sum over byte values of bucket[byte][column(j)] * centroid[digit_j(byte)].
    // A thread owns one byte column and a slice of the 256 byte values, reads each
    // bucket once, clears it for the next item and feeds the VE coordinates packed
    // in that byte.
    if constexpr (V3) {
      // A thread owns one field column (two coordinates) and a slice of the 64 field values,
      // reads its buckets in all four copies, clears them, and weighs by the two digits.
      constexpr int FC = P / 2, NPARTS = CS_CONSUMERS / FC, VPP = 64 / NPARTS; // 8 parts x 8 values, or 16 x 4
      const int col = tid % FC, part = tid / FC;
      const float *vcb = c_cb[1];
      float hi_sum = 0.f, lo_acc = 0.f;
#pragma unroll
      for (int i = 0; i < VPP; ++i) {
        const int v = part * VPP + i;
        uint32_t bi = 0;
#pragma unroll
        for (int cp = 0; cp < 4; ++cp) {
          const int idx = cp * 4096 + v * 64 + ((col + 4 * cp) & (FC - 1));
          bi += bucket[idx]; // the copies together hold at most the span's total (2^30)
          bucket[idx] = 0u;
        }
        const float bv = (float)bi;
        hi_sum += bv; // the first digit, (part * VPP) >> 3, is the same for all of this thread's values
        lo_acc += bv * vcb[v & 7];
      }
      const float hi_acc = hi_sum * vcb[(part * VPP) >> 3];
      sc[part * P + col * 2] = hi_acc * inv_fx;
      sc[part * P + col * 2 + 1] = lo_acc * inv_fx;
      consumer_sync();
      if (tid < P) {
        float t = 0.f;
#pragma unroll
        for (int g = 0; g < NPARTS; ++g) t += sc[g * P + tid];
        const int ab = idx & 1;
        guarded_wait(&aempty[ab], (((uint32_t)idx >> 1) & 1u) ^ 1u);
        float *dst = accb + ab * ACC_PITCH;
        dst[tid] = t;
        if (tid == 0) { dst[P] = mx; dst[P + 1] = ls; }
        __syncwarp();
        if (lane == 0) mbar_arrive(&afull[ab]);
      }
    } else {
      constexpr int NPARTS = CS_CONSUMERS / VCOLS, BPP = 256 / NPARTS;
      constexpr int LOGB = BPP == 16 ? 4 : 5; // byte value = (part << LOGB) | i
      static_assert(BPP == 16 || BPP == 32, "16 or 32 byte values per thread");
      const int col = tid % VCOLS, part = tid / VCOLS; // a warp shares `part`
      const float *vcb = c_cb[VB - 2];
      // The digit of coordinate e is bits [sh, sh+VB) of the byte value, sh = 8 - VB*(e+1).
      // With the loop over i unrolled it is a compile-time constant where those bits lie
      // inside i, fixed per thread where they lie inside `part` (then the buckets are
      // summed first and multiplied once), and one of two per-thread values in between.
      float av[VE], psum[VE], cmix[VE][2];
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        constexpr int MASK = (1 << VB) - 1;
        const int sh = 8 - VB * (e + 1);
        av[e] = 0.f;
        psum[e] = 0.f;
        cmix[e][0] = vcb[((part << LOGB) >> sh) & MASK];
        cmix[e][1] = vcb[(((part << LOGB) | (1 << (LOGB - 1))) >> sh) & MASK];
      }
#pragma unroll
      for (int i = 0; i < BPP; ++i) {
        const int b = part * BPP + i;
        uint32_t bi;
        if (COMPACT) {
          bi = bucket[b * 32 + col];
          bucket[b * 32 + col] = 0u;
        } else {
          bi = bucket[b * 64 + col];
          bucket[b * 64 + col] = 0u;
        }
        const float bv = (float)bi;
#pragma unroll
        for (int e = 0; e < VE; ++e) {
          constexpr int MASK = (1 << VB) - 1;
          const int sh = 8 - VB * (e + 1);
          if (sh >= LOGB) psum[e] += bv;                                        // digit set by `part`
          else if (sh + VB <= LOGB) av[e] += bv * vcb[(i >> sh) & MASK];         // digit set by i
          else av[e] += bv * cmix[e][(i >> (LOGB - 1)) & 1];                     // top bit of i, rest from `part`
        }
      }
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        const int sh = 8 - VB * (e + 1);
        if (sh >= LOGB) av[e] = psum[e] * cmix[e][0];
      }
      // sc[] is free (the V stream has finished with the weights): use it as fold space
      constexpr int NG = TWOCOPY ? 2 * NPARTS : NPARTS; // partial accumulators per coordinate
      const int grp = TWOCOPY ? 2 * part + (col >> 4) : part, ccol = TWOCOPY ? (col & 15) : col;
#pragma unroll
      for (int e = 0; e < VE; ++e) sc[grp * P + ccol * VE + e] = av[e] * inv_fx;
      consumer_sync();
      if (tid < P) { // hand the finished item to the helper warp and move on
        float t = 0.f;
#pragma unroll
        for (int g = 0; g < NG; ++g) t += sc[g * P + tid];
        const int ab = idx & 1;
        guarded_wait(&aempty[ab], (((uint32_t)idx >> 1) & 1u) ^ 1u);
        float *dst = accb + ab * ACC_PITCH;
        dst[tid] = t;
        if (tid == 0) { dst[P] = mx; dst[P + 1] = ls; }
        __syncwarp();
        if (lane == 0) mbar_arrive(&afull[ab]);
      }
    }
  }
}

// Two entry points that differ only in how the register budget is stated.  The byte-table
// instantiations are scheduled better under a plain register cap than under launch bounds
// (measured: K4/V2 4.69 -> 4.86 TB/s with the same 96 registers), the ones with 6-bit fields
// the other way round (K3/V2 3.60 vs 3.46 TB/s); a block of 576 threads can hold 96.
template <int KB, int KW, int VB, int VW>
__global__ void __maxnreg__(104) compute_stream_kernel(const StreamLaunch a) {
  compute_stream_body<KB, KW, VB, VW>(a);
}
template <int KB, int KW, int VB, int VW>
__global__ void __launch_bounds__(CS_THREADS, 1) compute_stream_kernel_fields(const StreamLaunch a) {
  compute_stream_body<KB, KW, VB, VW>(a);
}

} // namespace aq
