// Sparse-V decode attention in one block per (head, query), for caches of up to
// SP_THREADS * 16 tokens.
//
// Replaces the sparse tail of upstream's compute_avx2
// (attention/attention.cpp:448-473): softmax weights, order by weight
// (descending), accumulate V rows in blocks of four while four remain and the
// running mass is below v_mass, then singles; weights are not renormalised.
//
// The logits come from compute_general_kernel (mode 2), ordered oldest token
// first like upstream's slot list (attention.cpp:562-563), so equal weights keep
// that order through the stable sort -- the order a stable sort of upstream's
// list would give (upstream's std::sort leaves ties unspecified).  Here: softmax in
// registers, a stable block-wide radix sort of (weight, token) pairs (written here:
// block_sort_pairs), the
// block sums ((w0+w1)+w2)+w3 in parallel and the running mass sequentially in
// upstream's association (so the cut is the one a sequential walk finds), then
// the V rows of the chosen tokens with token groups in parallel, one inverse
// transform.  Longer caches use the device-wide segmented sort instead.
#pragma once
#include "common.cuh"
#include "compute_general.cuh"

namespace aq {

constexpr int SP_THREADS = 512;
constexpr int SP_WARPS = SP_THREADS / 32;
// Sort counters: 256 digit values x 16 warps, one padding word per digit so that the 32 lanes
// of a warp, which update different digits of their own warp's column, fall on different banks.
constexpr int SP_CNT_PITCH = SP_WARPS + 1;
constexpr int SP_CNT_WORDS = 256 * SP_CNT_PITCH;                      // 4352
constexpr int SP_CNT_PER_THREAD = (SP_CNT_WORDS + SP_THREADS - 1) / SP_THREADS; // 9

template <int ITEMS> struct SparseSmem {
  static constexpr int CAP = SP_THREADS * ITEMS;
  // scratch (sort counters, later the block sums and the byte-path fold) | weights | tokens | vec[1024] | red[64]
  static constexpr size_t sort_bytes = (size_t)SP_CNT_PER_THREAD * SP_THREADS * 4;
  static constexpr size_t scratch_bytes = sort_bytes > (size_t)CAP ? sort_bytes : (size_t)CAP; // >= CAP/4 floats and >= SP_THREADS floats
  static constexpr size_t bytes = scratch_bytes + (size_t)CAP * 8 + 1024 * 4 + 64 * 4; // a multiple of 16
};

// Position of item k of thread tid: a warp holds 32*ITEMS consecutive positions, item k of its
// lanes 32 consecutive ones.  (The sort ranks a warp's items k = 0, 1, ... in turn.)
template <int ITEMS> __device__ __forceinline__ int sp_pos(int tid, int k) { return (tid >> 5) * (32 * ITEMS) + k * 32 + (tid & 31); }

// Stable block-wide sort of (weight, token) pairs, largest weight first, equal weights in the
// order of their positions; the result goes to s_w[0..CAP) / s_tok[0..CAP).
// Weights lie in [0, 1], so their IEEE bit patterns occupy 30 bits and order like integers; the
// sort runs on the complemented pattern (ascending) with four least-significant-digit passes of
// 8 bits.  A pass: every warp counts its digits (lanes with equal digits find each other with
// match.any; the items of a warp are ranked k = 0, 1, ... in turn so that a running per-warp
// count gives the rank among the warp's earlier items), the counts [digit][warp] are scanned in
// that order over the block, and the pairs move to their ranks through s_w / s_tok.
// Padding (weight 0 at positions >= n) ties with real zero weights and stays behind them.
template <int ITEMS>
__device__ __forceinline__ void block_sort_pairs(float (&key)[ITEMS], int (&val)[ITEMS], float *s_w, int *s_tok, uint32_t *cnt,
                                                 uint32_t *warp_tot) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t *s_u = reinterpret_cast<uint32_t *>(s_w);
  uint32_t u[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) u[k] = ~__float_as_uint(key[k]) & 0x3FFFFFFFu;
  const uint32_t lt = (1u << lane) - 1u;
#pragma unroll 1
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 8 * pass;
    for (int e = tid; e < SP_CNT_PER_THREAD * SP_THREADS; e += SP_THREADS) cnt[e] = 0u;
    __syncthreads();
    uint32_t rank[ITEMS];
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t d = (u[k] >> shift) & 255u;
      const uint32_t same = __match_any_sync(0xffffffffu, d);
      uint32_t *slot = cnt + d * SP_CNT_PITCH + warp;
      const uint32_t before = *slot;
      __syncwarp();
      if (lane == __ffs(same) - 1) *slot = before + __popc(same);
      __syncwarp();
      rank[k] = before + __popc(same & lt);
    }
    __syncthreads();
    // exclusive scan of the counts in the order [digit][warp]
    {
      uint32_t loc[SP_CNT_PER_THREAD], tsum = 0u;
      const int e0 = tid * SP_CNT_PER_THREAD;
#pragma unroll
      for (int j = 0; j < SP_CNT_PER_THREAD; ++j) { loc[j] = cnt[e0 + j]; tsum += loc[j]; }
      uint32_t inc = tsum;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += t;
      }
      if (lane == 31) warp_tot[warp] = inc;
      __syncthreads();
      uint32_t base = inc - tsum;
      for (int w = 0; w < warp; ++w) base += warp_tot[w];
#pragma unroll
      for (int j = 0; j < SP_CNT_PER_THREAD; ++j) { cnt[e0 + j] = base; base += loc[j]; }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t d = (u[k] >> shift) & 255u;
      const uint32_t r = cnt[d * SP_CNT_PITCH + warp] + rank[k];
      s_u[r] = u[k];
      s_tok[r] = val[k];
    }
    __syncthreads();
    if (pass < 3) {
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const int p = sp_pos<ITEMS>(tid, k);
        u[k] = s_u[p];
        val[k] = s_tok[p];
      }
    }
  }
  // complemented patterns back to weights, in place
  for (int p = tid; p < SP_THREADS * ITEMS; p += SP_THREADS) s_u[p] = ~s_u[p] & 0x3FFFFFFFu;
  __syncthreads();
}

// The block computes its own logits (no separate logits launch) for packed rows of whole words
// up to padded dimension 128: the [coordinate][level] table then fits the fold space.
inline bool sparse_logits_in_block(int P) { return P % 32 == 0 && P <= 128; }

inline size_t sparse_fold_bytes(int P, int v_bits) {
  if (P % 32 != 0) return 0;
  const int units = P / (v_bits == 2 ? 16 : v_bits == 3 ? 32 : 8);
  const int rows = units <= 32 ? SP_THREADS / 32 : SP_THREADS / units;
  return (size_t)rows * P * sizeof(float);
}

__device__ __forceinline__ float sp_block_reduce(float v, float *red, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
  for (int i = 1; i < SP_THREADS / 32; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
  return r;
}

// Upstream's sequential walk (attention.cpp:455-473): add arr[0], arr[1], ... while the running
// mass is below `limit`; returns how many were added.  The sums are strictly sequential (that
// fixes the cut); the values are fetched eight at a time ahead of the sum so that the chain is
// one addition and one comparison per element, not a shared-memory round trip.
__device__ __forceinline__ int walk_mass(const float *arr, int len, float limit, float &mass) {
  int i = 0, cnt = 0;
  bool open = true;
  while (open && i < len) {
    float x[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = arr[min(i + k, len - 1)];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (open && i + k < len && mass < limit) {
        mass = __fadd_rn(mass, x[k]);
        ++cnt;
      } else {
        open = false;
      }
    }
    i += 8;
  }
  return cnt;
}

// V rows of the first `count` sorted tokens, by words (padded dimension a multiple of 32).
// A token's factor is w * vscale * (1/sqrt p); its V scale is fetched together with its row.
// `buf` takes sparse_fold_bytes() for the fold.
template <int BITS>
__device__ __forceinline__ void sparse_v_words(const float *s_w, const int *s_tok, int count, const uint8_t *vbase, const float *vsc,
                                               float isp, const CacheView &c, const float *s_cb, float *buf, float *vec,
                                               int *status) {
  using UU = VUnit<BITS>;
  const int tid = threadIdx.x, P = c.padded;
  const int U = P / UU::NCO, u = tid % U, tg = tid / U, TG = SP_THREADS / U;
  float acc[UU::NCO];
#pragma unroll
  for (int k = 0; k < UU::NCO; ++k) acc[k] = 0.f;
  const uint8_t *vunit = vbase + (size_t)u * (UU::WORDS * 4);
#pragma unroll 2
  for (int i = tg; i < count; i += TG) {
    const int tok = s_tok[i];
    if (!AQ_CHECK(status, tok >= 0 && tok < c.cap, 15)) continue;
    uint32_t w[UU::WORDS];
    load_words_be<UU::WORDS>(vunit + (size_t)tok * c.v_row, w);
    const float wt = s_w[i] * __ldg(vsc + tok) * isp;
#pragma unroll
    for (int k = 0; k < UU::NCO; ++k) acc[k] += wt * s_cb[level_of<BITS, UU::WORDS>(w, k)];
  }
  v_fold_words<BITS, SP_THREADS>(acc, P, buf, vec);
}

// Inverse transform of vec[32*EPL] and the store of the output, by one warp in registers
// (core/fwht.cpp:106-134: butterflies, * 1/sqrt p, * sign).
template <int EPL>
__device__ __forceinline__ void sparse_finish_warp(const float *vec, float isp, const uint32_t *sg, float *o, int dim, int lane) {
  float v[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) v[e] = vec[EPL * lane + e];
  warp_butterflies<EPL>(v, lane);
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int j = EPL * lane + e;
    if (j < dim) o[j] = v[e] * isp * sign_of(sg, j);
  }
}

// Query rotation (attention.cpp:537-550) by one warp in registers: qr[32*EPL] in shared memory.
template <int EPL>
__device__ __forceinline__ void sparse_rotate_warp(const float *qp, const uint32_t *sg, int dim, float *qr, int lane) {
  constexpr int P = 32 * EPL;
  float v[EPL];
  float part = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int j = EPL * lane + e;
    v[e] = j < dim ? __ldg(qp + j) : 0.f;
    part += v[e] * v[e];
  }
  const float qn = sqrtf(warp_sum(part) + 1e-12f);
  const float qinv = 1.f / qn;
#pragma unroll
  for (int e = 0; e < EPL; ++e) v[e] = v[e] * qinv * sign_of(sg, EPL * lane + e);
  warp_butterflies<EPL>(v, lane);
  const float back = sqrtf((float)P) * qn, isq = 1.f / sqrtf((float)P);
#pragma unroll
  for (int e = 0; e < EPL; ++e) qr[EPL * lane + e] = v[e] * isq * back;
}

template <int ITEMS>
__global__ void __launch_bounds__(SP_THREADS) sparse_fused_kernel(const float *logits, int w_stride, int n, int rot, CacheView c,
                                                                  int head0, int nq, float *out, int *status, const float *q) {
  using S = SparseSmem<ITEMS>;
  extern __shared__ __align__(16) unsigned char smem_sp[];
  float *scratch = reinterpret_cast<float *>(smem_sp);
  float *s_w = reinterpret_cast<float *>(smem_sp + S::scratch_bytes);
  int *s_tok = reinterpret_cast<int *>(s_w + S::CAP);
  float *vec = reinterpret_cast<float *>(s_tok + S::CAP);
  float *red = vec + 1024;
  __shared__ int s_count;

  const int P = c.padded, dim = c.dim;
  const int item = blockIdx.x;
  const int h = head0 + item / nq;
  const int tid = threadIdx.x;
  float key[ITEMS];
  int val[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) { // logical order (oldest token first); the rows are read by slot
    const int i = sp_pos<ITEMS>(tid, k);
    val[k] = i + rot < c.cap ? i + rot : i + rot - c.cap;
  }
  if (q != nullptr) {
    // ---- logits in this block (sparse_logits_in_block() holds): the query rotation of
    // compute_general_kernel (attention.cpp:537-550), then one thread per K row against the
    // [coordinate][level] table, which borrows the fold space behind the fixed part
    float *qr = vec, *lut = reinterpret_cast<float *>(smem_sp + S::bytes);
    const float *qp = q + (size_t)item * dim;
    const uint32_t *sg = c.signs + (size_t)h * c.sign_words;
    if (tid < 32) { // sparse_logits_in_block(): the padded dimension is 32, 64 or 128
      if (P == 128) sparse_rotate_warp<4>(qp, sg, dim, qr, tid);
      else if (P == 64) sparse_rotate_warp<2>(qp, sg, dim, qr, tid);
      else sparse_rotate_warp<1>(qp, sg, dim, qr, tid);
    }
    __syncthreads();
    const int L = 1 << c.k_bits;
    const float *kcb = c_cb[c.k_bits - 2];
    for (int i = tid; i < P * L; i += SP_THREADS) lut[i] = qr[i / L] * kcb[i % L];
    __syncthreads();
    const float attn_s = 1.f / (sqrtf((float)dim) * (float)P);
    const uint8_t *kbase = c.k_slab + (size_t)h * c.k_stride;
    const float *ksc = c.k_scale + (size_t)h * c.s_stride;
    griddep_wait(); // the cache is read from here on
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const int i = sp_pos<ITEMS>(tid, k);
      key[k] = -INFINITY;
      if (i < n && AQ_CHECK(status, val[k] >= 0 && val[k] < c.cap, 15)) {
        const uint8_t *kr = kbase + (size_t)val[k] * c.k_row;
        const float sum = c.k_bits == 4 ? score_row_words<4>(kr, lut, P)
                          : c.k_bits == 3 ? score_row_words<3>(kr, lut, P) : score_row_words<2>(kr, lut, P);
        key[k] = sum * attn_s * ksc[val[k]];
      }
    }
    __syncthreads(); // vec and the table are free again
  } else {
    const float *lg = logits + (size_t)item * w_stride;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const int i = sp_pos<ITEMS>(tid, k);
      key[k] = i < n ? lg[i] : -INFINITY;
    }
  }
  // ---- softmax weights, exactly as the unfused path: e = exp(l - max), w = e * (1/sum) ----
  float mx = -1e30f;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) mx = fmaxf(mx, key[k]);
  mx = sp_block_reduce(mx, red, true);
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = sp_pos<ITEMS>(tid, k);
    key[k] = i < n ? expf(key[k] - mx) : 0.f;
    s += key[k];
  }
  s = sp_block_reduce(s, red, false);
  const float inv = 1.f / s;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = sp_pos<ITEMS>(tid, k);
    key[k] = i < n ? key[k] * inv : 0.f; // padding: weight 0, behind the real tokens (stable sort)
  }
  // ---- stable descending sort of (weight, token) into s_w / s_tok ---------------------------
  __syncthreads();
  block_sort_pairs<ITEMS>(key, val, s_w, s_tok, reinterpret_cast<uint32_t *>(scratch), reinterpret_cast<uint32_t *>(red) + 48);
  // ---- the cut: blocks of four while four remain and the mass is short, then singles -------
  float *bsum = scratch; // the sort scratch is free now
  const int n4 = n / 4;
  for (int b = tid; b < n4; b += SP_THREADS)
    bsum[b] = __fadd_rn(__fadd_rn(__fadd_rn(s_w[4 * b], s_w[4 * b + 1]), s_w[4 * b + 2]), s_w[4 * b + 3]);
  if (tid < 16) red[32 + tid] = tid < (1 << c.v_bits) ? c_cb[c.v_bits - 2][tid] : 0.f; // V centroids for the by-words path
  __syncthreads();
  if (tid == 0) {
    float mass = 0.f;
    int ii = 0;
    if (c.sparse_block == 4) ii = 4 * walk_mass(bsum, n4, c.v_mass, mass);
    ii += walk_mass(s_w + ii, n - ii, c.v_mass, mass);
    s_count = ii;
  }
  __syncthreads();
  const int count = s_count;
  // ---- per-token factor w * vscale * (1/sqrt p), in place ------------------------------------
  const uint8_t *vbase = c.v_slab + (size_t)h * c.v_stride;
  const float *vsc = c.v_scale + (size_t)h * c.s_stride;
  const float *vcb = c_cb[c.v_bits - 2];
  const float isp = 1.f / sqrtf((float)P);
  // ---- V rows of the chosen tokens -------------------------------------------------------------
  if (P % 32 == 0) {
    // by words: thread = (unit of a row, token group); the units of a row are read side by side.
    // (the centroid copy in red[32..47] was written before the walk's barrier)
    float *s_cb = red + 32;
    float *fold = reinterpret_cast<float *>(smem_sp + S::bytes); // sparse_fold_bytes() behind the fixed part
    if (c.v_bits == 2) sparse_v_words<2>(s_w, s_tok, count, vbase, vsc, isp, c, s_cb, fold, vec, status);
    else if (c.v_bits == 3) sparse_v_words<3>(s_w, s_tok, count, vbase, vsc, isp, c, s_cb, fold, vec, status);
    else sparse_v_words<4>(s_w, s_tok, count, vbase, vsc, isp, c, s_cb, fold, vec, status);
  } else {
    // per-token factor w * vscale * (1/sqrt p), in place
    for (int i = tid; i < count; i += SP_THREADS)
      if (AQ_CHECK(status, s_tok[i] >= 0 && s_tok[i] < c.cap, 15)) s_w[i] = s_w[i] * vsc[s_tok[i]] * isp;
    __syncthreads();
    // by bytes: thread = (column, token group)
    const int TG = P < SP_THREADS ? SP_THREADS / P : 1;
    const int jcol = P < SP_THREADS ? tid % P : tid;
    const int tg = P < SP_THREADS ? tid / P : 0;
    float av = 0.f;
    if (jcol < P) {
#pragma unroll 4
      for (int i = tg; i < count; i += TG) {
        if (!AQ_CHECK(status, s_tok[i] >= 0 && s_tok[i] < c.cap, 15)) continue;
        av += s_w[i] * vcb[unpack_at(vbase + (size_t)s_tok[i] * c.v_row, jcol, c.v_bits)];
      }
    }
    __syncthreads(); // bsum is dead; reuse the scratch for the fold
    scratch[tid] = av;
    __syncthreads();
    if (tid < P) {
      float t = 0.f;
      for (int g = 0; g < TG; ++g) t += scratch[g * P + tid];
      vec[tid] = t;
    }
  }
  __syncthreads();
  const uint32_t *sg = c.signs + (size_t)h * c.sign_words;
  float *o = out + (size_t)item * dim;
  if (P == 32 || P == 64 || P == 128) { // one warp, in registers: no block barriers
    if (tid < 32) {
      if (P == 128) sparse_finish_warp<4>(vec, isp, sg, o, dim, tid);
      else if (P == 64) sparse_finish_warp<2>(vec, isp, sg, o, dim, tid);
      else sparse_finish_warp<1>(vec, isp, sg, o, dim, tid);
    }
    return;
  }
  block_butterflies(vec, P);
  for (int j = tid; j < dim; j += SP_THREADS) o[j] = vec[j] * isp * sign_of(sg, j);
}

} // namespace aq
