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
// registers, a stable block-wide radix sort of (weight, token) pairs, the
// block sums ((w0+w1)+w2)+w3 in parallel and the running mass sequentially in
// upstream's association (so the cut is the one a sequential walk finds), then
// the V rows of the chosen tokens with token groups in parallel, one inverse
// transform.  Longer caches use the device-wide segmented sort instead.
#pragma once
#include "common.cuh"
#include "compute_general.cuh"
#include <cub/block/block_radix_sort.cuh>

namespace aq {

constexpr int SP_THREADS = 512;

template <int ITEMS> struct SparseSmem {
  using Sort = cub::BlockRadixSort<float, SP_THREADS, ITEMS, int>;
  static constexpr int CAP = SP_THREADS * ITEMS;
  // sort scratch (later reused for the block sums and the group fold) | weights | tokens | vec[1024] | red[64]
  static constexpr size_t sort_bytes = (sizeof(typename Sort::TempStorage) + 15) / 16 * 16;
  static constexpr size_t scratch_bytes = sort_bytes > (size_t)CAP ? sort_bytes : (size_t)CAP; // >= CAP/4 floats and >= SP_THREADS floats
  static constexpr size_t bytes = scratch_bytes + (size_t)CAP * 8 + 1024 * 4 + 64 * 4;
};

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

template <int ITEMS>
__global__ void __launch_bounds__(SP_THREADS) sparse_fused_kernel(const float *logits, int w_stride, int n, int rot, CacheView c,
                                                                  int head0, int nq, float *out, int *status) {
  using S = SparseSmem<ITEMS>;
  using Sort = typename S::Sort;
  extern __shared__ __align__(16) unsigned char smem_sp[];
  typename Sort::TempStorage &sort_tmp = *reinterpret_cast<typename Sort::TempStorage *>(smem_sp);
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
  const float *lg = logits + (size_t)item * w_stride;

  // ---- softmax weights, exactly as the unfused path: e = exp(l - max), w = e * (1/sum) ----
  float key[ITEMS];
  int val[ITEMS];
  float mx = -1e30f;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = tid * ITEMS + k;
    key[k] = i < n ? lg[i] : -INFINITY;
    val[k] = i + rot < c.cap ? i + rot : i + rot - c.cap; // logits are in logical order; the V rows are read by slot
    mx = fmaxf(mx, key[k]);
  }
  mx = sp_block_reduce(mx, red, true);
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = tid * ITEMS + k;
    key[k] = i < n ? expf(key[k] - mx) : 0.f;
    s += key[k];
  }
  s = sp_block_reduce(s, red, false);
  const float inv = 1.f / s;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = tid * ITEMS + k;
    key[k] = i < n ? key[k] * inv : -1.f; // padding sorts behind every real weight (weights are >= 0)
  }
  // ---- stable descending sort of (weight, token) ------------------------------------------
  __syncthreads();
  Sort(sort_tmp).SortDescending(key, val);
  __syncthreads();
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    s_w[tid * ITEMS + k] = key[k];
    s_tok[tid * ITEMS + k] = val[k];
  }
  __syncthreads();
  // ---- the cut: blocks of four while four remain and the mass is short, then singles -------
  float *bsum = scratch; // the sort scratch is free now
  const int n4 = n / 4;
  for (int b = tid; b < n4; b += SP_THREADS)
    bsum[b] = __fadd_rn(__fadd_rn(__fadd_rn(s_w[4 * b], s_w[4 * b + 1]), s_w[4 * b + 2]), s_w[4 * b + 3]);
  __syncthreads();
  if (tid == 0) {
    float mass = 0.f;
    int ii = 0;
    if (c.sparse_block == 4)
      for (; ii + 3 < n && mass < c.v_mass; ii += 4) mass = __fadd_rn(mass, bsum[ii >> 2]);
    for (; ii < n && mass < c.v_mass; ++ii) mass = __fadd_rn(mass, s_w[ii]);
    s_count = ii;
  }
  __syncthreads();
  const int count = s_count;
  // ---- per-token factor w * vscale * (1/sqrt p), in place ------------------------------------
  const uint8_t *vbase = c.v_slab + (size_t)h * c.v_stride;
  const float *vsc = c.v_scale + (size_t)h * c.s_stride;
  const float *vcb = c_cb[c.v_bits - 2];
  const float isp = 1.f / sqrtf((float)P);
  for (int i = tid; i < count; i += SP_THREADS)
    if (AQ_CHECK(status, s_tok[i] >= 0 && s_tok[i] < c.cap, 15)) s_w[i] = s_w[i] * vsc[s_tok[i]] * isp;
  __syncthreads();
  // ---- V rows of the chosen tokens: thread = (column, token group) ----------------------------
  const int TG = P < SP_THREADS ? SP_THREADS / P : 1;
  const int jcol = P < SP_THREADS ? tid % P : tid;
  const int tg = P < SP_THREADS ? tid / P : 0;
  constexpr int MAXR = 2; // P <= 1024
  float acc[MAXR] = {0.f, 0.f};
#pragma unroll
  for (int r = 0; r < MAXR; ++r) {
    const int j = jcol + r * SP_THREADS;
    if (j >= P || (P < SP_THREADS && r > 0)) break;
    float av = 0.f;
#pragma unroll 4
    for (int i = tg; i < count; i += TG) {
      if (!AQ_CHECK(status, s_tok[i] >= 0 && s_tok[i] < c.cap, 15)) continue;
      av += s_w[i] * vcb[unpack_at(vbase + (size_t)s_tok[i] * c.v_row, j, c.v_bits)];
    }
    acc[r] = av;
  }
  __syncthreads(); // bsum is dead; reuse the scratch for the fold
  if (P < SP_THREADS) {
    scratch[tid] = acc[0];
    __syncthreads();
    if (tid < P) {
      float t = 0.f;
      for (int g = 0; g < TG; ++g) t += scratch[g * P + tid];
      vec[tid] = t;
    }
  } else {
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
      const int j = jcol + r * SP_THREADS;
      if (j < P) vec[j] = acc[r];
    }
  }
  __syncthreads();
  block_butterflies(vec, P);
  const uint32_t *sg = c.signs + (size_t)h * c.sign_words;
  float *o = out + (size_t)item * dim;
  for (int j = tid; j < dim; j += SP_THREADS) o[j] = vec[j] * isp * sign_of(sg, j);
}

} // namespace aq
