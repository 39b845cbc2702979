// Device side of upstream's second stack (the "V2" plugin runtime): the compute
// primitives of its kernel interface adaptq::IKernelBackend
// (include/adaptq/kernel.h:24-94; scalar reference in
// kernels/scalar/kdot_scalar.cpp:21-168) as CUDA kernels over rows that lie at
// a fixed stride in device memory -- the layout of upstream's slab storage
// (storage/contiguous_slab.h:19-153).
//
//   fwht_forward   x <- (1/sqrt p) H D x                (core/fwht.cpp:88-104)
//   fwht_inverse   x <- D (1/sqrt p) H x                (core/fwht.cpp:106-134)
//   kdot_batch     logits[i] = (sum_j q_rot[j] * centroid[idx_i[j]]) * scale_i / p
//   vaccum_batch   acc[j]    = sum_i weights[i] * scale_i * centroid[idx_i[j]]
//
// These are interface-compatibility kernels (the whole-head attention of that
// stack, HARFixedStrategy::compute_full, strategies/har_fixed.cpp:197-289, runs
// on the fused decode kernels through adaptq_runtime_compute); they are written
// for correctness and coalesced row reads, not tuned further.
#pragma once
#include "common.cuh"

namespace aq {

constexpr int KB_THREADS = 256;

// One block per vector.  inverse == 0: x*D, butterflies, *1/sqrt(p); else butterflies, *(1/sqrt(p))*D.
__global__ void __launch_bounds__(KB_THREADS) fwht_vectors_kernel(float *x, const int8_t *D, int padded, int inverse) {
  extern __shared__ __align__(16) unsigned char smem_kb[];
  float *buf = reinterpret_cast<float *>(smem_kb);
  float *v = x + (size_t)blockIdx.x * padded;
  for (int i = threadIdx.x; i < padded; i += KB_THREADS) buf[i] = inverse ? v[i] : v[i] * (float)D[i];
  __syncthreads();
  block_butterflies(buf, padded);
  const float s = 1.f / sqrtf((float)padded);
  for (int i = threadIdx.x; i < padded; i += KB_THREADS) v[i] = inverse ? buf[i] * s * (float)D[i] : buf[i] * s;
}

// One warp per row: logits[i] = dot * scale[i] / padded  (kernels/scalar/kdot_scalar.cpp:35-49).
__global__ void __launch_bounds__(KB_THREADS) kdot_rows_kernel(const float *q_rot, const uint8_t *rows, size_t row_stride,
                                                               const float *scales, int n, int padded, int bits,
                                                               float *logits) {
  extern __shared__ __align__(16) unsigned char smem_kb[];
  float *lut = reinterpret_cast<float *>(smem_kb); // [level][padded]
  const int levels = 1 << bits;
  const float *cb = c_cb[bits - 2];
  for (int i = threadIdx.x; i < padded * levels; i += KB_THREADS) lut[i] = q_rot[i % padded] * cb[i / padded];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv = 1.f / (float)padded;
  for (int i = blockIdx.x * (KB_THREADS / 32) + warp; i < n; i += gridDim.x * (KB_THREADS / 32)) {
    const uint8_t *row = rows + (size_t)i * row_stride;
    float s = 0.f;
    for (int j = lane; j < padded; j += 32) s += lut[unpack_at(row, j, bits) * padded + j];
    s = warp_sum(s);
    if (lane == 0) logits[i] = s * scales[i] * inv;
  }
}

// Block b accumulates its slice of the tokens into partial[b][padded]; the second
// kernel adds the partials in block order (deterministic).
__global__ void __launch_bounds__(KB_THREADS) vaccum_rows_kernel(const uint8_t *rows, size_t row_stride, const float *scales,
                                                                 const float *weights, int n, int padded, int bits,
                                                                 float *partial) {
  const float *cb = c_cb[bits - 2];
  const int per = (n + gridDim.x - 1) / gridDim.x;
  const int t0 = blockIdx.x * per, t1 = min(n, t0 + per);
  for (int j = threadIdx.x; j < padded; j += KB_THREADS) {
    float a = 0.f;
    for (int i = t0; i < t1; ++i) {
      const float w = weights[i];
      if (w == 0.f) continue; // as upstream skips them (kdot_scalar.cpp:63)
      a += (w * scales[i]) * cb[unpack_at(rows + (size_t)i * row_stride, j, bits)];
    }
    partial[(size_t)blockIdx.x * padded + j] = a;
  }
}
__global__ void __launch_bounds__(KB_THREADS) vaccum_fold_kernel(const float *partial, int n_parts, int padded, float *acc) {
  for (int j = blockIdx.x * KB_THREADS + threadIdx.x; j < padded; j += gridDim.x * KB_THREADS) {
    float a = 0.f;
    for (int p = 0; p < n_parts; ++p) a += partial[(size_t)p * padded + j];
    acc[j] = a;
  }
}

} // namespace aq
