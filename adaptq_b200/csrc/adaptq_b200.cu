// Host runtime and C ABI of the B200 AdapTQ engine (libadaptq_b200.so).
//
// Implements include/adaptq.h (the interface of upstream
// core/adaptq_c_api.cpp) and include/adaptq_b200.h over the CUDA kernels in
// this directory.  There is no CPU compute path: if no CUDA device is usable
// every constructor fails with an error string.
#include "../../include/adaptq_b200.h"
#include "../../include/adaptq_runtime.h"
#include "append.cuh"
#include "compute_general.cuh"
#include "compute_sparse.cuh"
#include "compute_stream.cuh"
#include "runtime_v2.cuh"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cub/device/device_segmented_radix_sort.cuh>
#include <mutex>
#include <new>
#include <vector>

using namespace aq;

// ---------------------------------------------------------------------------
// error string (per thread, 256 bytes, as upstream core/adaptq_c_api.cpp:15-21)
// ---------------------------------------------------------------------------
static thread_local char tl_error[256] = "";
static void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
}
static void clear_error() { tl_error[0] = '\0'; }
extern "C" const char *adaptq_last_error(void) { return tl_error; }

static std::atomic<unsigned long long> g_launches{0};
static std::atomic<int> g_policy{0};
extern "C" unsigned long long adaptq_kernel_launches(void) { return g_launches.load(); }
extern "C" int adaptq_set_kernel_policy(int policy) {
  if (policy < 0 || policy > 2) { set_error("adaptq_set_kernel_policy: policy must be 0, 1 or 2"); return -1; }
  g_policy.store(policy);
  return 0;
}

// ---------------------------------------------------------------------------
// Failure seam for tests: the three host-side calls whose failure the library must
// survive -- device allocation, page-locked host allocation, kernel launch -- go
// through these wrappers.  adaptq_inject_failure(kind, nth) makes the nth upcoming
// call of that kind report failure WITHOUT touching the device (nothing faults,
// nothing is launched), so the error paths can be exercised on a healthy GPU.
// ---------------------------------------------------------------------------
enum { FAIL_DEVICE_ALLOC = 1, FAIL_PINNED_ALLOC = 2, FAIL_LAUNCH = 3 };
static std::atomic<int> g_fail_in[4] = {};
static bool injected(int kind) {
  int v = g_fail_in[kind].load();
  while (v > 0) {
    if (g_fail_in[kind].compare_exchange_weak(v, v - 1)) return v == 1;
  }
  return false;
}
extern "C" int adaptq_inject_failure(int kind, int nth) {
  if (kind < FAIL_DEVICE_ALLOC || kind > FAIL_LAUNCH || nth < 0) { set_error("adaptq_inject_failure: kind must be 1..3 and nth >= 0"); return -1; }
  g_fail_in[kind].store(nth);
  return 0;
}
static cudaError_t device_malloc(void **p, size_t bytes) {
  if (injected(FAIL_DEVICE_ALLOC)) { *p = nullptr; return cudaErrorMemoryAllocation; }
  return cudaMalloc(p, bytes);
}
static cudaError_t pinned_malloc(void **p, size_t bytes) {
  if (injected(FAIL_PINNED_ALLOC)) { *p = nullptr; return cudaErrorMemoryAllocation; }
  return cudaMallocHost(p, bytes);
}
// The status of the launch just made (cudaGetLastError), or an injected failure.
static cudaError_t launch_status() {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && injected(FAIL_LAUNCH)) return cudaErrorLaunchFailure;
  return e;
}

#define CUDA_TRY(expr, what)                                                            \
  do {                                                                                  \
    cudaError_t e__ = (expr);                                                           \
    if (e__ != cudaSuccess) {                                                           \
      set_error("%s: CUDA error: %s", what, cudaGetErrorString(e__));                   \
      return false;                                                                     \
    }                                                                                   \
  } while (0)

// ---------------------------------------------------------------------------
// handle
// ---------------------------------------------------------------------------
namespace {

constexpr uint32_t MAGIC = 0xA0DA97B2u;

struct RingState { int head, size, mirror; };

struct Group {
  uint32_t magic = MAGIC;
  bool single = false;
  // The decode-step entry points store the library's launch count here right after they have
  // launched the append kernel on `stream`.  An attention launch that finds the count unchanged
  // is the very next launch, so the append kernel is its predecessor in the stream and it may
  // start beside it (programmatic dependent launch); any other launch in between voids it.
  std::atomic<unsigned long long> append_ticket{~0ull};
  CacheView c{};
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  std::vector<uint64_t> seeds;
  // ring state: one value while all heads move together, else one per head
  bool uniform = true;
  RingState u{0, 0, 0};
  std::vector<RingState> per_head;
  // device staging for host-pointer calls, and scratch for partials / sparse V
  void *d_stage = nullptr; size_t stage_bytes = 0;
  void *h_stage = nullptr; size_t h_stage_bytes = 0;
  void *d_scratch_base = nullptr; // header + scratch, one allocation
  void *d_scratch = nullptr; size_t scratch_bytes = 0;
  int *d_counters = nullptr;
  int *d_status = nullptr;
  size_t device_bytes = 0;
  std::mutex mu;
#ifdef ADAPTQ_CHECKED
  std::vector<std::pair<const unsigned char *, const char *>> canaries; // (first byte behind a buffer, its name)
#endif
  // decode-step pipeline (host buffers): copy streams and per-chunk events, made on first use
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  std::vector<cudaEvent_t> ev;

  RingState state(int h) const { return uniform ? u : per_head[h]; }
  void split_state() {
    if (uniform) { per_head.assign(c.n_heads, u); uniform = false; }
  }
  void try_unify() {
    if (uniform) return;
    for (int i = 1; i < c.n_heads; ++i)
      if (per_head[i].head != per_head[0].head || per_head[i].size != per_head[0].size ||
          per_head[i].mirror != per_head[0].mirror)
        return;
    u = per_head[0]; uniform = true; per_head.clear();
  }
};

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
  ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

int next_pow2(int n) { // upstream core/fwht.cpp:13-19
  if (n <= 1) return 1;
  if (n > (1 << 30)) return 1 << 30;
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

bool valid_bits(int b) { return b == 16 || (b >= 2 && b <= 4); }

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

__global__ void fill_f32_kernel(float *p, size_t n, float v) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}
__global__ void segment_offsets_kernel(int *begin, int *end, int n_seg, int stride, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_seg) { begin[i] = i * stride; end[i] = i * stride + n; }
}

void free_group(Group *g) {
  if (!g) return;
  DeviceGuard dg(g->device);
  // wait for this handle's own work only (the legacy stream when no stream was set)
  cudaStreamSynchronize(g->stream);
  if (g->copy_in) cudaStreamSynchronize(g->copy_in);
  if (g->copy_out) cudaStreamSynchronize(g->copy_out);
  cudaFree(g->c.k_slab); cudaFree(g->c.v_slab); cudaFree(g->c.k_scale); cudaFree(g->c.v_scale);
  cudaFree((void *)g->c.signs); cudaFree(g->c.mirror);
  cudaFree(g->d_stage); cudaFree(g->d_scratch_base); cudaFree(g->d_status);
  if (g->h_stage) cudaFreeHost(g->h_stage);
  if (g->copy_in) cudaStreamDestroy(g->copy_in);
  if (g->copy_out) cudaStreamDestroy(g->copy_out);
  for (cudaEvent_t e : g->ev) cudaEventDestroy(e);
  g->magic = 0;
  delete g;
}

// Checked build: every buffer of a handle is followed by AQ_CANARY_BYTES of a fixed pattern
// that adaptq_mha_synchronize verifies; a kernel that writes past a buffer is caught there.
#ifdef ADAPTQ_CHECKED
constexpr size_t AQ_CANARY_BYTES = 256;
constexpr int AQ_CANARY_BYTE = 0xA5;
#endif

bool alloc(void **p, size_t bytes, Group *g, const char *what) {
  *p = nullptr;
  if (bytes == 0) bytes = 16;
#ifdef ADAPTQ_CHECKED
  const size_t tail = AQ_CANARY_BYTES;
#else
  const size_t tail = 0;
#endif
  cudaError_t e = device_malloc(p, bytes + tail);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error("%s: device allocation of %zu bytes failed: %s", what, bytes, cudaGetErrorString(e));
    return false;
  }
#ifdef ADAPTQ_CHECKED
  cudaMemset(static_cast<unsigned char *>(*p) + bytes, AQ_CANARY_BYTE, tail);
  g->canaries.emplace_back(static_cast<unsigned char *>(*p) + bytes, what);
#endif
  g->device_bytes += bytes;
  return true;
}

#ifdef ADAPTQ_CHECKED
void forget_canary(Group *g, const void *base) { // the buffer is about to be freed
  // buffers are separate allocations, so the closest guard above `base` is the one behind it
  size_t best = g->canaries.size();
  for (size_t i = 0; i < g->canaries.size(); ++i)
    if (g->canaries[i].first > static_cast<const unsigned char *>(base) &&
        (best == g->canaries.size() || g->canaries[i].first < g->canaries[best].first))
      best = i;
  if (best != g->canaries.size()) g->canaries.erase(g->canaries.begin() + best);
}
#else
inline void forget_canary(Group *, const void *) {}
#endif

// Rademacher signs as upstream core/fwht.cpp:21-27, stored one bit per sign.
void sign_words_for(uint64_t seed, int padded, uint32_t *words, int n_words) {
  uint64_t s = seed ? seed : 0xdeadbeefcafe1234ULL;
  for (int i = 0; i < n_words; ++i) words[i] = 0;
  for (int i = 0; i < padded; ++i) {
    s ^= s << 13; s ^= s >> 7; s ^= s << 17;
    if (!(s & 1)) words[i >> 5] |= 1u << (i & 31);
  }
}

Group *create_group(const char *fn, const char *bad_args_msg, int n_heads, const uint64_t *seeds, int dim,
                    int k_bits, int v_bits, int capacity, float v_mass, int hyb, bool single) {
  if (n_heads <= 0 || dim <= 0 || !valid_bits(k_bits) || !valid_bits(v_bits) || capacity < 0 || hyb < 0) {
    set_error("%s", bad_args_msg);
    return nullptr;
  }
  const int P = next_pow2(dim);
  if (P > 1024) { // upstream throws here (core/quantizer.cpp:27-31); the C ABI must not
    set_error("%s: head dimension %d pads to %d, above the supported 1024", fn, dim, P);
    return nullptr;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    set_error("%s: no usable CUDA device (this library has no CPU path)", fn);
    return nullptr;
  }
  Group *g = new (std::nothrow) Group();
  if (!g) { set_error("%s: out of host memory", fn); return nullptr; }
  g->single = single;
  g->device = dev;
  cudaDeviceGetAttribute(&g->sm_count, cudaDevAttrMultiProcessorCount, dev);
  g->seeds.assign(seeds, seeds + n_heads);
  CacheView &c = g->c;
  c.n_heads = n_heads; c.dim = dim; c.padded = P; c.k_bits = k_bits; c.v_bits = v_bits;
  c.log2p = 0; while ((1 << c.log2p) < P) ++c.log2p;
  c.k_row = row_bytes(P, k_bits); c.v_row = row_bytes(P, v_bits);
  c.cap = capacity; c.hyb = hyb; c.v_mass = v_mass;
  c.sparse_block = 4;
  // +128 slack: bulk copies of the last tile round their size up to 16 bytes
  c.k_stride = round_up((size_t)capacity * c.k_row, 128) + 128;
  c.v_stride = round_up((size_t)capacity * c.v_row, 128) + 128;
  c.s_stride = (int)round_up((size_t)capacity, 32) + 32;
  c.sign_words = (P + 31) / 32;
  c.mirror_stride = (size_t)hyb * 2 * dim;
  const char *what = fn;
  bool ok = alloc((void **)&c.k_slab, c.k_stride * n_heads, g, what) &&
            alloc((void **)&c.v_slab, c.v_stride * n_heads, g, what) &&
            alloc((void **)&c.k_scale, (size_t)c.s_stride * n_heads * 4, g, what) &&
            alloc((void **)&c.v_scale, (size_t)c.s_stride * n_heads * 4, g, what) &&
            alloc((void **)&c.signs, (size_t)c.sign_words * n_heads * 4, g, what) &&
            alloc((void **)&g->d_status, 16, g, what);
  if (ok && hyb > 0) ok = alloc((void **)&c.mirror, c.mirror_stride * n_heads * 4, g, what);
  if (!ok) { free_group(g); return nullptr; }
  std::vector<uint32_t> words((size_t)c.sign_words * n_heads);
  for (int h = 0; h < n_heads; ++h) sign_words_for(seeds[h], P, words.data() + (size_t)h * c.sign_words, c.sign_words);
  cudaError_t e = cudaMemcpy((void *)c.signs, words.data(), words.size() * 4, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(c.k_slab, 0, c.k_stride * n_heads);
  if (e == cudaSuccess) e = cudaMemset(c.v_slab, 0, c.v_stride * n_heads);
  if (e == cudaSuccess) e = cudaMemset(g->d_status, 0, 16);
  if (e == cudaSuccess) {
    size_t ns = (size_t)c.s_stride * n_heads;
    fill_f32_kernel<<<(int)std::min<size_t>((ns + 255) / 256, 4096), 256>>>(c.k_scale, ns, 1.0f);
    fill_f32_kernel<<<(int)std::min<size_t>((ns + 255) / 256, 4096), 256>>>(c.v_scale, ns, 1.0f);
    g_launches += 2;
    e = cudaDeviceSynchronize();
  }
  if (e != cudaSuccess) {
    set_error("%s: CUDA error during set-up: %s", fn, cudaGetErrorString(e));
    cudaGetLastError();
    free_group(g);
    return nullptr;
  }
  return g;
}

Group *as_group(void *h) {
  Group *g = static_cast<Group *>(h);
  return (g && g->magic == MAGIC) ? g : nullptr;
}

enum PtrKind { PK_HOST_PAGEABLE, PK_HOST_PINNED, PK_DEVICE };
PtrKind ptr_kind(const void *p) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return PK_HOST_PAGEABLE; }
  if (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) return PK_DEVICE;
  if (at.type == cudaMemoryTypeHost) return PK_HOST_PINNED;
  return PK_HOST_PAGEABLE;
}

bool ensure_stage(Group *g, size_t dev_bytes, size_t host_bytes) {
  if (dev_bytes > g->stage_bytes) {
    CUDA_TRY(cudaStreamSynchronize(g->stream), "staging");
    if (g->d_stage) { forget_canary(g, g->d_stage); cudaFree(g->d_stage); g->device_bytes -= g->stage_bytes; }
    g->d_stage = nullptr; g->stage_bytes = 0;
    size_t nb = round_up(dev_bytes, 256);
    if (!alloc(&g->d_stage, nb, g, "staging")) return false;
    g->stage_bytes = nb;
  }
  if (host_bytes > g->h_stage_bytes) {
    CUDA_TRY(cudaStreamSynchronize(g->stream), "staging");
    if (g->h_stage) cudaFreeHost(g->h_stage);
    g->h_stage = nullptr; g->h_stage_bytes = 0;
    size_t nb = round_up(host_bytes, 4096);
    CUDA_TRY(pinned_malloc(&g->h_stage, nb), "staging (pinned host)");
    g->h_stage_bytes = nb;
  }
  return true;
}

// Scratch = a zeroed header of arrival counters (kernels that use them leave them at
// zero) followed by the space for partials / sparse-V work arrays.
constexpr size_t SCRATCH_HEADER = 65536;
constexpr int MAX_COUNTED_ITEMS = (int)(SCRATCH_HEADER / sizeof(int));
bool ensure_scratch(Group *g, size_t bytes) {
  if (bytes <= g->scratch_bytes) return true;
  CUDA_TRY(cudaStreamSynchronize(g->stream), "scratch");
  if (g->d_scratch_base) { forget_canary(g, g->d_scratch_base); cudaFree(g->d_scratch_base); g->device_bytes -= g->scratch_bytes + SCRATCH_HEADER; }
  g->d_scratch_base = nullptr; g->d_scratch = nullptr; g->d_counters = nullptr; g->scratch_bytes = 0;
  size_t nb = round_up(bytes + bytes / 4, 256);
  if (!alloc(&g->d_scratch_base, nb + SCRATCH_HEADER, g, "scratch")) return false;
  CUDA_TRY(cudaMemsetAsync(g->d_scratch_base, 0, SCRATCH_HEADER, g->stream), "scratch");
  g->d_counters = static_cast<int *>(g->d_scratch_base);
  g->d_scratch = static_cast<char *>(g->d_scratch_base) + SCRATCH_HEADER;
  g->scratch_bytes = nb;
  return true;
}

// Bring `bytes` at `src` to the device: device pointers pass through, pinned
// host memory is copied asynchronously, pageable memory goes through the
// handle's pinned buffer.  `slot_off` places it inside the staging buffer.
const float *to_device(Group *g, const void *src, size_t bytes, size_t slot_off, bool &ok) {
  ok = true;
  PtrKind k = ptr_kind(src);
  if (k == PK_DEVICE) return static_cast<const float *>(src);
  char *dst = static_cast<char *>(g->d_stage) + slot_off;
  cudaError_t e;
  if (k == PK_HOST_PINNED) {
    e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, g->stream);
  } else {
    char *hp = static_cast<char *>(g->h_stage) + slot_off;
    memcpy(hp, src, bytes);
    e = cudaMemcpyAsync(dst, hp, bytes, cudaMemcpyHostToDevice, g->stream);
  }
  if (e != cudaSuccess) { set_error("host-to-device copy failed: %s", cudaGetErrorString(e)); ok = false; }
  return reinterpret_cast<const float *>(dst);
}

bool check_status(Group *g, const char *fn) {
  int st[4] = {0, 0, 0, 0};
  CUDA_TRY(cudaMemcpyAsync(st, g->d_status, sizeof(int), cudaMemcpyDeviceToHost, g->stream), fn);
  CUDA_TRY(cudaStreamSynchronize(g->stream), fn);
  if (st[0] != 0) {
    if (st[0] >= 10) set_error("%s: a device-side index check failed (status %d); the access was skipped", fn, st[0]);
    else set_error("%s: a kernel gave up waiting for a memory transfer (status %d)", fn, st[0]);
    cudaMemsetAsync(g->d_status, 0, sizeof(int), g->stream);
    return false;
  }
#ifdef ADAPTQ_CHECKED
  unsigned char tail[AQ_CANARY_BYTES];
  for (auto &cn : g->canaries) {
    CUDA_TRY(cudaMemcpy(tail, cn.first, AQ_CANARY_BYTES, cudaMemcpyDeviceToHost), fn);
    for (size_t i = 0; i < AQ_CANARY_BYTES; ++i)
      if (tail[i] != AQ_CANARY_BYTE) {
        set_error("%s: the guard bytes behind a device buffer (%s) were overwritten at offset %zu", fn, cn.second, i);
        return false;
      }
  }
#endif
  return true;
}

// Dynamic shared-memory limit of a kernel, raised once per device (and again only
// when a larger size is asked for).  `slot` is the caller's per-kernel table; calls
// hold different handles' mutexes, so the table has its own lock.
constexpr int MAX_DEVICES = 64;
std::mutex g_attr_mu;
template <typename K>
bool ensure_smem_limit(K kern, int (&slot)[MAX_DEVICES], int device, size_t bytes, const char *what) {
  std::lock_guard<std::mutex> lk(g_attr_mu);
  if (device < 0 || device >= MAX_DEVICES) { set_error("%s: device ordinal %d is not supported (0..%d)", what, device, MAX_DEVICES - 1); return false; }
  if ((int)bytes > slot[device]) {
    CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), what);
    slot[device] = (int)bytes;
  }
  return true;
}

// Launch an attention kernel.  Directly behind this handle's append kernel (g->after_append)
// the launch carries the programmatic-stream-serialisation attribute: the kernel may start
// while the append still runs and waits inside (griddep_wait) before it reads the cache.
template <typename Kern, typename... Args>
void launch_attention(Group *g, Kern kern, dim3 grid, int threads, size_t smem, Args... args) {
  const bool pdl = g->append_ticket.exchange(~0ull) == g_launches.load();
  if (!pdl) {
    kern<<<grid, threads, smem, g->stream>>>(args...);
    return;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = g->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, args...); // the caller reads the launch status
}

// ---------------------------------------------------------------------------
// append
// ---------------------------------------------------------------------------
template <int P, int BITS>
bool launch_rows(Group *g, const AppendLaunch &a) {
  constexpr size_t SMEM = ((size_t)AT_TILE * (P + 4) + (size_t)(AT_THREADS / 32) * P) * sizeof(float);
  static int configured[MAX_DEVICES] = {};
  auto kern = append_tile_kernel<P, BITS>;
  if (!ensure_smem_limit(kern, configured, g->device, SMEM, "append")) return false;
  long long items = (long long)a.heads_in_call * a.n_tokens;
  long long tiles = (items + AT_TILE - 1) / AT_TILE;
  int grid = (int)std::min<long long>(tiles, (long long)g->sm_count * AT_BLOCKS_PER_SM);
  kern<<<grid, AT_THREADS, SMEM, g->stream>>>(a);
  ++g_launches;
  CUDA_TRY(launch_status(), "append");
  return true;
}

template <int P>
bool launch_rows_bits(Group *g, const AppendLaunch &a, int bits) {
  switch (bits) {
  case 2: return launch_rows<P, 2>(g, a);
  case 3: return launch_rows<P, 3>(g, a);
  case 4: return launch_rows<P, 4>(g, a);
  default: return launch_rows<P, 16>(g, a);
  }
}

// Keys and values together (values quantised, keys quantised or FP32): one launch, blockIdx.y = side.
template <int P, int KB, int VB>
bool launch_pair(Group *g, const AppendLaunch &ak, const AppendLaunch &av) {
  constexpr size_t SMEM = ((size_t)AT_TILE * (P + 4) + (size_t)(AT_THREADS / 32) * P) * sizeof(float);
  static int configured[MAX_DEVICES] = {};
  auto kern = append_pair_kernel<P, KB, VB>;
  if (!ensure_smem_limit(kern, configured, g->device, SMEM, "append")) return false;
  long long items = (long long)ak.heads_in_call * ak.n_tokens;
  long long tiles = (items + AT_TILE - 1) / AT_TILE;
  int gx = (int)std::min<long long>(tiles, (long long)g->sm_count * (AT_BLOCKS_PER_SM / 2));
  kern<<<dim3(gx, 2), AT_THREADS, SMEM, g->stream>>>(ak, av.src);
  ++g_launches;
  CUDA_TRY(launch_status(), "append");
  return true;
}
template <int P, int KB>
bool launch_pair_v(Group *g, const AppendLaunch &ak, const AppendLaunch &av, int vb) {
  switch (vb) {
  case 2: return launch_pair<P, KB, 2>(g, ak, av);
  case 3: return launch_pair<P, KB, 3>(g, ak, av);
  default: return launch_pair<P, KB, 4>(g, ak, av);
  }
}
template <int P>
bool launch_pair_kv(Group *g, const AppendLaunch &ak, const AppendLaunch &av, int kb, int vb) {
  switch (kb) {
  case 2: return launch_pair_v<P, 2>(g, ak, av, vb);
  case 3: return launch_pair_v<P, 3>(g, ak, av, vb);
  case 16: return launch_pair_v<P, 16>(g, ak, av, vb); // FP32 keys (layer-0 passthrough) beside quantised values
  default: return launch_pair_v<P, 4>(g, ak, av, vb);
  }
}

bool tile_kernel_applies(Group *g, const AppendLaunch &a, int src_row_align_ok) {
  const CacheView &c = g->c;
  const bool small = (long long)a.heads_in_call * a.n_tokens < (1ll << 31) && (long long)a.ring_head + a.n_tokens < (1ll << 31);
  return g_policy.load() != 1 && (c.padded == 64 || c.padded == 128) && (c.dim % 4 == 0) && src_row_align_ok && small;
}

bool launch_append_one(Group *g, AppendLaunch a, int src_row_align_ok) {
  const CacheView &c = g->c;
  const int bits = a.which ? c.v_bits : c.k_bits;
  const int policy = g_policy.load();
  const bool fast = tile_kernel_applies(g, a, src_row_align_ok);
  if (fast) return c.padded == 128 ? launch_rows_bits<128>(g, a, bits) : launch_rows_bits<64>(g, a, bits);
  if (policy == 2) { set_error("append: shape not covered by the specialised kernel"); return false; }
  long long items = (long long)a.heads_in_call * a.n_tokens;
  int grid = (int)std::min<long long>((items + GEN_WARPS - 1) / GEN_WARPS, (long long)g->sm_count * 16);
  size_t smem = (size_t)GEN_WARPS * c.padded * sizeof(float);
  append_general_kernel<<<grid, GEN_WARPS * 32, smem, g->stream>>>(a);
  ++g_launches;
  CUDA_TRY(launch_status(), "append");
  return true;
}

// (magic, shift, add) with  x / d == umulhi(x + add, magic) >> shift  for 0 <= x < 2^31
// (round-down multiplier; the +1 on the dividend makes it exact).
void magic_div(uint32_t d, uint32_t &magic, uint32_t &shift, uint32_t &add) {
  if (d <= 1) { magic = 0xFFFFFFFFu; shift = 0; add = 1; return; }
  uint32_t l = 0;
  while ((1ull << l) < d) ++l; // ceil(log2 d)
  if ((d & (d - 1)) == 0) { magic = 0x80000000u; shift = l - 1; add = 0; return; }
  magic = (uint32_t)((1ull << (32 + l - 1)) / d);
  shift = l - 1;
  add = 1;
}

RingState advance(const CacheView &c, RingState s, int T) { // cache/ring_buffer.cpp:105-119, attention.cpp:354-365
  RingState r = s;
  if (c.cap > 0) {
    r.head = (int)(((long long)s.head + T) % c.cap);
    r.size = (int)std::min<long long>((long long)s.size + T, c.cap);
  }
  if (c.hyb > 0) {
    bool evicts = (long long)s.size + T > c.cap;
    if (evicts) r.mirror = 0;
    else r.mirror = s.mirror + std::min(T, std::max(0, c.hyb - s.mirror));
  }
  return r;
}

// keys/vals on the device: [n_tokens] rows of `token_stride` floats, head hl at +hl*dim
bool append_device(Group *g, const float *dk, const float *dv, int head0, int heads_in_call, int n_tokens,
                   size_t token_stride, RingState st) {
  if (n_tokens <= 0 || heads_in_call <= 0) return true;
  AppendLaunch a;
  a.c = g->c;
  a.head0 = head0; a.heads_in_call = heads_in_call; a.n_tokens = n_tokens;
  a.ring_head = st.head; a.ring_size = st.size; a.mirror_cnt = st.mirror;
  // One contiguous block of rows (the call covers whole tokens, no padding): walk it
  // token-major so that a tile is one stretch of memory; otherwise walk the tokens of
  // a head so that its packed rows leave in order.
  a.contig = (token_stride == (size_t)heads_in_call * g->c.dim && g->c.dim == g->c.padded) ? 1 : 0;
  a.head_major = a.contig ? 0 : (n_tokens >= 32);
  a.status = g->d_status;
  a.src_token_stride = token_stride;
  magic_div((uint32_t)(a.head_major ? n_tokens : heads_in_call), a.div_magic, a.div_shift, a.div_add);
  magic_div((uint32_t)std::max(1, g->c.cap), a.cap_magic, a.cap_shift, a.cap_add);
  {
    volatile float sq = sqrtf((float)g->c.padded); // IEEE sqrt, then IEEE divide, as upstream computes them
    volatile float isq = 1.0f / sq;
    a.sqrt_p = sq; a.inv_sqrt_p = isq;
  }
  const int align_k = ((reinterpret_cast<uintptr_t>(dk) & 15) == 0) && (token_stride % 4 == 0);
  const int align_v = ((reinterpret_cast<uintptr_t>(dv) & 15) == 0) && (token_stride % 4 == 0);
  if (g->c.v_bits != 16) {
    AppendLaunch ak = a, av = a;
    ak.which = 0; ak.src = dk;
    av.which = 1; av.src = dv;
    if (tile_kernel_applies(g, ak, align_k) && tile_kernel_applies(g, av, align_v))
      return g->c.padded == 128 ? launch_pair_kv<128>(g, ak, av, g->c.k_bits, g->c.v_bits)
                                : launch_pair_kv<64>(g, ak, av, g->c.k_bits, g->c.v_bits);
  }
  for (int which = 0; which < 2; ++which) {
    a.which = which;
    a.src = which ? dv : dk;
    if (!launch_append_one(g, a, which ? align_v : align_k)) return false;
  }
  return true;
}

// ---------------------------------------------------------------------------
// compute
// ---------------------------------------------------------------------------
size_t partial_floats(const CacheView &c) { return (size_t)2 + c.padded; }

// The general kernel's dynamic shared memory limit only ever grows (per device and variant).
template <bool KW, bool VW>
bool launch_general_variant(Group *g, const ComputeLaunch &a, dim3 grid, size_t smem, const char *what) {
  static int smem_set[MAX_DEVICES] = {};
  auto kern = compute_general_kernel<KW, VW>;
  if (!ensure_smem_limit(kern, smem_set, g->device, smem, what)) return false;
  launch_attention(g, kern, grid, CG_THREADS, smem, a);
  ++g_launches;
  CUDA_TRY(launch_status(), what);
  return true;
}

// Packed rows are read by words where they are whole words (padded dimension a multiple of 32).
bool general_by_words(const CacheView &c, bool side_f32) { return !side_f32 && c.padded % 32 == 0; }

// Tokens per shared-memory pass; the by-words fold of V needs 8 rows of the padded dimension there.
int general_chunk(const CacheView &c, int span, bool vw) {
  return std::max(std::max(CG_THREADS, std::min(span, 2048)), vw ? 8 * c.padded : 0);
}

bool launch_general_kernel(Group *g, const ComputeLaunch &a, dim3 grid, size_t smem, bool kw, bool vw, const char *what) {
  if (kw) return vw ? launch_general_variant<true, true>(g, a, grid, smem, what) : launch_general_variant<true, false>(g, a, grid, smem, what);
  return vw ? launch_general_variant<false, true>(g, a, grid, smem, what) : launch_general_variant<false, false>(g, a, grid, smem, what);
}

bool launch_general(Group *g, ComputeLaunch &a, bool want_partial_out, float *partial_out) {
  const CacheView &c = g->c;
  const bool mirror = a.use_mirror != 0;
  const bool k_f32 = mirror || c.k_bits == 16;
  const bool v_f32 = mirror || c.v_bits == 16;
  const int items = a.heads_in_call * a.nq;
  int want = std::max(1, (2 * g->sm_count + items - 1) / items); // measured: more blocks per SM bring nothing
  int max_splits = std::max(1, (a.n + 63) / 64); // short spans: these shapes are latency-bound, so spread them wide
  a.n_splits = std::min(want, max_splits);
  a.span = (int)round_up((size_t)(a.n + a.n_splits - 1) / a.n_splits, 32);
  a.n_splits = (a.n + a.span - 1) / a.span;
  const bool kw = general_by_words(c, k_f32), vw = general_by_words(c, v_f32);
  a.chunk = std::max(CG_THREADS, std::min(a.span, 2048));
  const int kcb = k_f32 ? 0 : (1 << c.k_bits);
  size_t smem = cg_smem_floats(c.padded, kcb, general_chunk(c, a.span, vw)) * sizeof(float);
  const bool direct = a.n_splits == 1 && !want_partial_out;
  if (!direct) {
    if (!ensure_scratch(g, (size_t)a.n_splits * items * partial_floats(c) * sizeof(float))) return false;
    a.partial = static_cast<float *>(g->d_scratch);
    a.mode = 1;
  } else {
    a.mode = 0;
  }
  // few items: the last block to finish an item merges its partials inside the same launch
  const bool fused = !direct && items <= MAX_COUNTED_ITEMS;
  a.counters = fused ? g->d_counters : nullptr;
  a.final_out = want_partial_out ? partial_out : a.out;
  a.final_to_partial = want_partial_out ? 1 : 0;
  dim3 grid(a.n_splits, a.heads_in_call, a.nq);
  if (!launch_general_kernel(g, a, grid, smem, kw, vw, "compute")) return false;
  if (!direct && !fused) {
    merge_partials_kernel<<<items, CG_THREADS, c.padded * sizeof(float), g->stream>>>(
        a.partial, (size_t)items * partial_floats(c), a.n_splits, c, a.head0, a.nq,
        want_partial_out ? partial_out : a.out, v_f32 ? 1 : 0, want_partial_out ? 1 : 0, mirror ? a.n : 0);
    ++g_launches;
    CUDA_TRY(launch_status(), "compute (merge)");
  }
  return true;
}

// Logits of every (head, query) into w[items][ws] with the general kernel (mode 2).
bool launch_logits(Group *g, ComputeLaunch &a, float *w, int ws) {
  const CacheView &c = g->c;
  const int items = a.heads_in_call * a.nq;
  a.weights = w; a.w_stride = ws; a.mode = 2;
  a.n_splits = std::max(1, std::min((2 * g->sm_count + items - 1) / items, (a.n + 63) / 64));
  a.span = (int)round_up((size_t)(a.n + a.n_splits - 1) / a.n_splits, 32);
  a.n_splits = (a.n + a.span - 1) / a.span;
  a.chunk = std::max(CG_THREADS, std::min(a.span, 2048));
  size_t smem = cg_smem_floats(c.padded, 1 << c.k_bits, a.chunk) * sizeof(float);
  return launch_general_kernel(g, a, dim3(a.n_splits, a.heads_in_call, a.nq), smem, general_by_words(c, false), false,
                               "compute (logits)");
}

template <int ITEMS>
bool launch_sparse_fused_t(Group *g, const ComputeLaunch &a, const float *w, int ws, const float *q) {
  const size_t smem = SparseSmem<ITEMS>::bytes + sparse_fold_bytes(g->c.padded, g->c.v_bits);
  static int configured[MAX_DEVICES] = {};
  auto kern = sparse_fused_kernel<ITEMS>;
  if (!ensure_smem_limit(kern, configured, g->device, smem, "compute (sparse V)")) return false;
  launch_attention(g, kern, dim3((unsigned)(a.heads_in_call * a.nq)), SP_THREADS, smem, w, ws, a.n, a.rot, g->c, a.head0, a.nq, a.out, g->d_status, q);
  ++g_launches;
  CUDA_TRY(launch_status(), "compute (sparse V)");
  return true;
}

bool launch_sparse(Group *g, ComputeLaunch &a) {
  const CacheView &c = g->c;
  const int items = a.heads_in_call * a.nq;
  const int ws = (int)round_up((size_t)a.n, 32);
  const size_t cells = (size_t)items * ws;
  if (cells > (size_t)0x7fffffff) { set_error("compute: sparse-V workspace too large for one call"); return false; }
  if (a.n <= SP_THREADS * 16) { // one block per (head, query) sorts and accumulates in shared memory
    // few items: the block also forms its logits (one launch); many items: the logits come from
    // the general kernel, which spreads each item's rows over many blocks
    const bool in_block = sparse_logits_in_block(c.padded) && g_policy.load() != 1 && items <= 2 * g->sm_count;
    float *w = nullptr;
    if (!in_block) {
      if (!ensure_scratch(g, cells * 4 + 256)) return false;
      w = static_cast<float *>(g->d_scratch);
      if (!launch_logits(g, a, w, ws)) return false;
    }
    const float *q = in_block ? a.q : nullptr;
    if (a.n <= SP_THREADS * 4) return launch_sparse_fused_t<4>(g, a, w, ws, q);
    if (a.n <= SP_THREADS * 8) return launch_sparse_fused_t<8>(g, a, w, ws, q);
    return launch_sparse_fused_t<16>(g, a, w, ws, q);
  }
  size_t temp_bytes = 0;
  cub::DeviceSegmentedRadixSort::SortPairsDescending(nullptr, temp_bytes, (const float *)nullptr, (float *)nullptr,
                                                     (const int *)nullptr, (int *)nullptr, (int)cells, items,
                                                     (const int *)nullptr, (const int *)nullptr, 0, 32, g->stream);
  size_t off_w = 0, off_o = off_w + cells * 4, off_sw = off_o + cells * 4, off_so = off_sw + cells * 4;
  size_t off_b = off_so + cells * 4, off_e = off_b + round_up((size_t)items * 4, 256);
  size_t off_t = off_e + round_up((size_t)items * 4, 256);
  if (!ensure_scratch(g, off_t + temp_bytes + 256)) return false;
  char *base = static_cast<char *>(g->d_scratch);
  float *w = (float *)(base + off_w), *sw = (float *)(base + off_sw);
  int *o = (int *)(base + off_o), *so = (int *)(base + off_so);
  int *sb = (int *)(base + off_b), *se = (int *)(base + off_e);
  // 1. logits into the weight buffer (general kernel, mode 2)
  if (!launch_logits(g, a, w, ws)) return false;
  // 2. softmax weights, 3. stable descending sort per (head, query), 4. cut + accumulate
  softmax_weights_kernel<<<items, CG_THREADS, 0, g->stream>>>(w, o, ws, a.n, a.rot, c.cap);
  segment_offsets_kernel<<<(items + 255) / 256, 256, 0, g->stream>>>(sb, se, items, ws, a.n);
  g_launches += 2;
  cudaError_t e = cub::DeviceSegmentedRadixSort::SortPairsDescending(base + off_t, temp_bytes, w, sw, o, so, (int)cells,
                                                                     items, sb, se, 0, 32, g->stream);
  g_launches += 1;
  CUDA_TRY(e, "compute (sparse-V sort)");
  sparse_accumulate_kernel<<<items, CG_THREADS, c.padded * sizeof(float), g->stream>>>(sw, so, ws, a.n, c, a.head0, a.nq, a.out);
  ++g_launches;
  CUDA_TRY(launch_status(), "compute (sparse V)");
  return true;
}


// ---- streaming kernel dispatch ---------------------------------------------
template <int KB, int KW, int VB, int VW>
bool launch_stream_t(Group *g, const StreamLaunch &a, int grid) {
  void (*kern)(const StreamLaunch);
  if constexpr (KB == 3 || VB == 3) kern = compute_stream_kernel_fields<KB, KW, VB, VW>;
  else kern = compute_stream_kernel<KB, KW, VB, VW>;
  static int configured[MAX_DEVICES] = {};
  if (!ensure_smem_limit(kern, configured, g->device, CS_SMEM_BYTES, "compute")) return false;
  launch_attention(g, kern, dim3((unsigned)grid), CS_THREADS, CS_SMEM_BYTES, a);
  ++g_launches;
  CUDA_TRY(launch_status(), "compute");
  return true;
}

bool stream_supported(const CacheView &c) {
  const bool v_ok = c.v_bits == 4 || c.v_bits == 3 || c.v_bits == 2;
  if (c.padded == 128) return (c.k_bits == 4 || c.k_bits == 3 || c.k_bits == 2) && v_ok;
  if (c.padded == 64) return (c.k_bits == 4 || c.k_bits == 3) && v_ok;
  return false;
}

// The streaming kernel's instantiation for a handle's shape (stream_supported() holds),
// one persistent block per SM or per work item, whichever is fewer.
template <int KB, int KW, int P>
bool launch_stream_v(Group *g, const StreamLaunch &a, int grid) {
  switch (a.c.v_bits) {
  case 2: return launch_stream_t<KB, KW, 2, P / 16>(g, a, grid);
  case 3: return launch_stream_t<KB, KW, 3, 3 * P / 32>(g, a, grid);
  default: return launch_stream_t<KB, KW, 4, P / 8>(g, a, grid);
  }
}

bool launch_stream_for_shape(Group *g, const StreamLaunch &a) {
  const CacheView &c = a.c;
  const long long items = (long long)a.heads_in_call * a.nq * a.n_splits;
  const int grid = (int)std::min<long long>(items, g->sm_count);
  if (c.padded == 128) {
    if (c.k_bits == 4) return launch_stream_v<4, 16, 128>(g, a, grid);
    if (c.k_bits == 3) return launch_stream_v<3, 12, 128>(g, a, grid);
    return launch_stream_v<2, 8, 128>(g, a, grid);
  }
  if (c.k_bits == 3) return launch_stream_v<3, 6, 64>(g, a, grid);
  return launch_stream_v<4, 8, 64>(g, a, grid);
}

// Pick the number of KV spans per (head, query): spans are multiples of 64
// tokens (16-byte aligned rows and scales; a span's last stage tile may be
// partial) of nearly equal length, at most CS_SPAN_MAX, not needlessly short,
// and the item count should fill whole waves of persistent blocks.
void plan_spans(int n, int items_base, int sms, int &n_splits, int &span) {
  const int G = 64;

  const int n_pad = (int)round_up((size_t)n, G);
  const int min_splits = (n + CS_SPAN_MAX - 1) / CS_SPAN_MAX;
  double best = -1.0;
  n_splits = min_splits;
  span = std::min(CS_SPAN_MAX, n_pad);
  for (int r = 1; r <= 16; ++r) {
    int s = std::max(std::max(1, min_splits), (sms * r) / std::max(1, items_base));
    int sp = (int)round_up((size_t)(n + s - 1) / s, G);
    sp = std::max(sp, std::min(1024, n_pad));
    sp = std::min(sp, CS_SPAN_MAX);
    const int s2 = (n + sp - 1) / sp;
    const long long items = (long long)items_base * s2;
    const long long waves = (items + sms - 1) / sms;
    const double fill = (double)items / (double)(waves * sms);
    // per-item cost beside the streaming (softmax pass over a fixed register tile, bucket fold,
    // partial write, table build): measured sweeps over the number of spans at 16 k to 128 k
    // tokens per head are matched by about 1500 token-equivalents
    const double overhead = (double)sp / (double)(sp + 1500);
    const double score = fill * overhead;
    if (score > best + 1e-9) { best = score; n_splits = s2; span = sp; }
  }
}


// Peer destinations of the next streaming launch (set by adaptq_mha_compute_partial_to_peers
// around its call, under the handle's mutex).
struct PeerSpec { int n = 0, rank = 0; float *out[8] = {}; unsigned int *flag[8] = {}; };
static thread_local const PeerSpec *tl_peers = nullptr;

bool launch_stream(Group *g, const ComputeLaunch &ca, bool want_partial_out, float *partial_out) {
  const CacheView &c = g->c;
  StreamLaunch a{};
  a.c = c; a.q = ca.q; a.out = ca.out; a.head0 = ca.head0; a.heads_in_call = ca.heads_in_call; a.nq = ca.nq;
  a.n = ca.n; a.status = g->d_status;
  const int items_base = a.heads_in_call * a.nq;
  plan_spans(a.n, items_base, g->sm_count, a.n_splits, a.span);
  const bool direct = a.n_splits == 1 && !want_partial_out;
  if (!direct) {
    if (a.n_splits == 1) {
      a.partial = partial_out; // a single span already is the combined partial
    } else {
      if (!ensure_scratch(g, (size_t)a.n_splits * items_base * partial_floats(c) * sizeof(float))) return false;
      a.partial = static_cast<float *>(g->d_scratch);
    }
  }
  const int force_partial = (!direct && a.n_splits == 1) ? 1 : 0;
  a.force_partial = force_partial;
  const bool fused = a.n_splits > 1 && items_base <= MAX_COUNTED_ITEMS;
  a.counters = fused ? g->d_counters : nullptr;
  a.final_out = want_partial_out ? partial_out : a.out;
  a.final_to_partial = want_partial_out ? 1 : 0;
  if (tl_peers) {
    if (a.n_splits > 1 && !fused) { set_error("compute: too many (head, query) items for the peer exchange"); return false; }
    a.n_peers = tl_peers->n; a.my_rank = tl_peers->rank;
    for (int r = 0; r < tl_peers->n; ++r) { a.peer_out[r] = tl_peers->out[r]; a.peer_flag[r] = tl_peers->flag[r]; }
  }
  if (!launch_stream_for_shape(g, a)) return false;
  if (a.n_splits > 1 && !fused) {
    merge_partials_kernel<<<items_base, CG_THREADS, c.padded * sizeof(float), g->stream>>>(
        a.partial, (size_t)items_base * partial_floats(c), a.n_splits, c, a.head0, a.nq,
        want_partial_out ? partial_out : a.out, 0, want_partial_out ? 1 : 0, 0);
    ++g_launches;
    CUDA_TRY(launch_status(), "compute (merge)");
  }
  return true;
}

bool launch_general_or_stream(Group *g, ComputeLaunch &a, bool want_partial_out, float *partial_out) {
  const CacheView &c = g->c;
  const int policy = g_policy.load();
  const bool can_stream = !a.use_mirror && stream_supported(c);
  if (can_stream && policy != 1) return launch_stream(g, a, want_partial_out, partial_out);
  if (policy == 2) { set_error("compute: shape not covered by the streaming kernel"); return false; }
  return launch_general(g, a, want_partial_out, partial_out);
}

// dq, dout on the device.  All heads of the call share `st`.
bool compute_device(Group *g, const float *dq, float *dout, int head0, int heads_in_call, int nq, RingState st,
                    bool partial_out) {
  const CacheView &c = g->c;
  if (heads_in_call <= 0 || nq <= 0) return true;
  const size_t out_floats = (size_t)heads_in_call * nq * (partial_out ? partial_floats(c) : (size_t)c.dim);
  if (st.size == 0) {
    g->append_ticket = ~0ull;
    CUDA_TRY(cudaMemsetAsync(dout, 0, out_floats * 4, g->stream), "compute");
    return true;
  }
  ComputeLaunch a{};
  a.c = c; a.q = dq; a.out = dout; a.head0 = head0; a.heads_in_call = heads_in_call; a.nq = nq; a.n = st.size;
  a.rot = (int)(((long long)st.head - st.size + c.cap) % c.cap); // st.size > 0, so c.cap > 0
  a.status = g->d_status;
  a.use_mirror = (c.hyb > 0 && st.size <= c.hyb && st.mirror == st.size) ? 1 : 0;
  const bool quant = c.k_bits != 16 && c.v_bits != 16;
  if (partial_out) return launch_general_or_stream(g, a, true, dout);
  if (!a.use_mirror && c.v_mass > 0.f && quant) return launch_sparse(g, a);
  return launch_general_or_stream(g, a, false, nullptr);
}

} // namespace

// ===========================================================================
// C ABI
// ===========================================================================
namespace {

bool require_handle(const void *h, const char *op) {
  if (h) return true;
  set_error("%s: null handle", op);
  return false;
}
bool require_pointer(const void *p, const char *op, const char *param) {
  if (p) return true;
  set_error("%s: null %s", op, param);
  return false;
}

// One head, one token, host or device pointers.
void append_one(Group *g, int head, const float *key, const float *val, const char *fn) {
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  const size_t vb = (size_t)g->c.dim * 4;
  if (!ensure_stage(g, 2 * round_up(vb, 256), 2 * round_up(vb, 256))) return;
  bool ok1, ok2;
  const float *dk = to_device(g, key, vb, 0, ok1);
  const float *dv = to_device(g, val, vb, round_up(vb, 256), ok2);
  if (!ok1 || !ok2) return;
  RingState st = g->state(head);
  if (!append_device(g, dk, dv, head, 1, 1, (size_t)g->c.dim, st)) return;
  RingState ns = advance(g->c, st, 1);
  if (g->c.n_heads == 1) g->u = ns;
  else { g->split_state(); g->per_head[head] = ns; g->try_unify(); }
  // host buffers may be reused by the caller as soon as we return
  if (ptr_kind(key) != PK_DEVICE || ptr_kind(val) != PK_DEVICE) {
    cudaError_t e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) set_error("%s: CUDA error: %s", fn, cudaGetErrorString(e));
  }
}

// nq queries of one head.  Returns tokens used or -1.
int compute_one(Group *g, int head, const float *queries, int nq, float *outs, const char *fn) {
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  RingState st = g->state(head);
  if (nq == 0) return st.size;
  const size_t qb = (size_t)nq * g->c.dim * 4;
  const size_t off_out = round_up(qb, 256);
  if (!ensure_stage(g, off_out + round_up(qb, 256), off_out + round_up(qb, 256))) return -1;
  bool ok;
  const float *dq = to_device(g, queries, qb, 0, ok);
  if (!ok) return -1;
  const PtrKind ok_kind = ptr_kind(outs);
  float *dout = ok_kind == PK_DEVICE ? outs : reinterpret_cast<float *>(static_cast<char *>(g->d_stage) + off_out);
  if (!compute_device(g, dq, dout, head, 1, nq, st, false)) return -1;
  if (ok_kind != PK_DEVICE) {
    void *hdst = ok_kind == PK_HOST_PINNED ? (void *)outs : (void *)(static_cast<char *>(g->h_stage) + off_out);
    cudaError_t e = cudaMemcpyAsync(hdst, dout, qb, cudaMemcpyDeviceToHost, g->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) { set_error("%s: CUDA error: %s", fn, cudaGetErrorString(e)); return -1; }
    if (ok_kind != PK_HOST_PINNED) memcpy(outs, hdst, qb);
  } else if (ptr_kind(queries) != PK_DEVICE) {
    cudaStreamSynchronize(g->stream);
  }
  return st.size;
}

void reset_group(Group *g) { // upstream core/adaptq_c_api.cpp:128-137: counters only, data stays
  std::lock_guard<std::mutex> lk(g->mu);
  g->uniform = true;
  g->per_head.clear();
  g->u = RingState{0, 0, 0};
}

size_t kv_bytes_group(Group *g) { // include/ring_buffer.h:93 summed over heads
  std::lock_guard<std::mutex> lk(g->mu);
  const size_t per_tok = (size_t)g->c.k_row + g->c.v_row;
  if (g->uniform) return (size_t)g->u.size * per_tok * g->c.n_heads;
  size_t t = 0;
  for (auto &s : g->per_head) t += (size_t)s.size * per_tok;
  return t;
}

} // namespace

extern "C" {

adaptq_ctx_t adaptq_create(int dim, int k_bits, int v_bits, int capacity, uint64_t seed, float v_mass,
                           int hybrid_thresh) {
  return create_group("adaptq_create", "adaptq_create: invalid dimensions or capacity", 1, &seed, dim, k_bits, v_bits,
                      capacity, v_mass, hybrid_thresh, true);
}

void adaptq_destroy(adaptq_ctx_t h) { free_group(as_group(h)); }

void adaptq_append(adaptq_ctx_t h, const float *key, const float *val, int /*token_pos*/) {
  if (!require_handle(h, "adaptq_append") || !require_pointer(key, "adaptq_append", "key") ||
      !require_pointer(val, "adaptq_append", "val"))
    return;
  Group *g = as_group(h);
  if (!g) { set_error("adaptq_append: not a live handle"); return; }
  append_one(g, 0, key, val, "adaptq_append");
}

int adaptq_compute(adaptq_ctx_t h, const float *query, float *out) {
  if (!require_handle(h, "adaptq_compute") || !require_pointer(query, "adaptq_compute", "query") ||
      !require_pointer(out, "adaptq_compute", "out"))
    return -1;
  Group *g = as_group(h);
  if (!g) { set_error("adaptq_compute: not a live handle"); return -1; }
  return compute_one(g, 0, query, 1, out, "adaptq_compute");
}

int adaptq_compute_batch(adaptq_ctx_t h, const float *queries, int num_queries, float *outs) {
  if (!require_handle(h, "adaptq_compute_batch")) return -1;
  if (num_queries < 0) { set_error("adaptq_compute_batch: negative num_queries"); return -1; }
  if (num_queries > 0 && (!require_pointer(queries, "adaptq_compute_batch", "queries") ||
                          !require_pointer(outs, "adaptq_compute_batch", "outs")))
    return -1;
  Group *g = as_group(h);
  if (!g) { set_error("adaptq_compute_batch: not a live handle"); return -1; }
  return compute_one(g, 0, queries, num_queries, outs, "adaptq_compute_batch");
}

void adaptq_reset(adaptq_ctx_t h) {
  if (!require_handle(h, "adaptq_reset")) return;
  Group *g = as_group(h);
  if (!g) { set_error("adaptq_reset: not a live handle"); return; }
  reset_group(g);
  clear_error();
}

size_t adaptq_kv_bytes(adaptq_ctx_t h) {
  if (!require_handle(h, "adaptq_kv_bytes")) return 0;
  Group *g = as_group(h);
  return g ? kv_bytes_group(g) : 0;
}

adaptq_mha_t adaptq_mha_create(int n_heads, int dim, int k_bits, int v_bits, int capacity, uint64_t base_seed,
                               float v_mass, int hybrid_thresh) {
  if (n_heads <= 0) { set_error("adaptq_mha_create: invalid parameters"); return nullptr; }
  std::vector<uint64_t> seeds((size_t)n_heads);
  for (int i = 0; i < n_heads; ++i) seeds[i] = base_seed ^ ((uint64_t)i * 0xDEADBEEFCAFEULL);
  return create_group("adaptq_mha_create", "adaptq_mha_create: invalid parameters", n_heads, seeds.data(), dim, k_bits,
                      v_bits, capacity, v_mass, hybrid_thresh, false);
}

adaptq_mha_t adaptq_mha_create_seeded(int n_heads, const uint64_t *seeds, int dim, int k_bits, int v_bits,
                                      int capacity, float v_mass, int hybrid_thresh) {
  if (n_heads <= 0 || !seeds) { set_error("adaptq_mha_create_seeded: invalid parameters"); return nullptr; }
  return create_group("adaptq_mha_create_seeded", "adaptq_mha_create_seeded: invalid parameters", n_heads, seeds, dim,
                      k_bits, v_bits, capacity, v_mass, hybrid_thresh, false);
}

void adaptq_mha_destroy(adaptq_mha_t h) { free_group(as_group(h)); }

#define MHA_PROLOGUE(fn, fail)                                                     \
  if (!require_handle(h, fn)) return fail;                                         \
  Group *g = as_group(h);                                                          \
  if (!g) { set_error("%s: not a live handle", fn); return fail; }

void adaptq_mha_append(adaptq_mha_t h, int head_idx, const float *key, const float *val, int /*token_pos*/) {
  MHA_PROLOGUE("adaptq_mha_append", )
  if (head_idx < 0 || head_idx >= g->c.n_heads) { set_error("adaptq_mha_append: head_idx out of range"); return; }
  if (!require_pointer(key, "adaptq_mha_append", "key") || !require_pointer(val, "adaptq_mha_append", "val")) return;
  clear_error();
  append_one(g, head_idx, key, val, "adaptq_mha_append");
}

int adaptq_mha_compute(adaptq_mha_t h, int head_idx, const float *query, float *out) {
  MHA_PROLOGUE("adaptq_mha_compute", -1)
  if (head_idx < 0 || head_idx >= g->c.n_heads) { set_error("adaptq_mha_compute: head_idx out of range"); return -1; }
  if (!require_pointer(query, "adaptq_mha_compute", "query") || !require_pointer(out, "adaptq_mha_compute", "out"))
    return -1;
  clear_error();
  return compute_one(g, head_idx, query, 1, out, "adaptq_mha_compute");
}

int adaptq_mha_compute_batch(adaptq_mha_t h, int head_idx, const float *queries, int num_queries, float *outs) {
  MHA_PROLOGUE("adaptq_mha_compute_batch", -1)
  if (head_idx < 0 || head_idx >= g->c.n_heads) {
    set_error("adaptq_mha_compute_batch: head_idx out of range");
    return -1;
  }
  if (num_queries < 0) { set_error("adaptq_mha_compute_batch: negative num_queries"); return -1; }
  if (num_queries > 0 && (!require_pointer(queries, "adaptq_mha_compute_batch", "queries") ||
                          !require_pointer(outs, "adaptq_mha_compute_batch", "outs")))
    return -1;
  clear_error();
  return compute_one(g, head_idx, queries, num_queries, outs, "adaptq_mha_compute_batch");
}

void adaptq_mha_reset(adaptq_mha_t h) {
  MHA_PROLOGUE("adaptq_mha_reset", )
  reset_group(g);
  clear_error();
}

size_t adaptq_mha_total_kv_bytes(adaptq_mha_t h) {
  MHA_PROLOGUE("adaptq_mha_total_kv_bytes", 0)
  return kv_bytes_group(g);
}

unsigned int adaptq_features(void) { return ADAPTQ_FEAT_HYBRID | ADAPTQ_FEAT_SPARSE_V | ADAPTQ_FEAT_CUDA_SM100; }
#ifdef ADAPTQ_CHECKED
const char *adaptq_version(void) { return "3.2.0-sm100a-checked"; }
#else
const char *adaptq_version(void) { return "3.2.0-sm100a"; }
#endif

// ---- batched additions ---------------------------------------------------------------

int adaptq_mha_append_batch(adaptq_mha_t h, const float *keys, const float *vals, int n_tokens, int /*token_pos0*/) {
  MHA_PROLOGUE("adaptq_mha_append_batch", -1)
  if (n_tokens < 0) { set_error("adaptq_mha_append_batch: negative n_tokens"); return -1; }
  if (n_tokens == 0) return 0;
  if (!require_pointer(keys, "adaptq_mha_append_batch", "keys") || !require_pointer(vals, "adaptq_mha_append_batch", "vals"))
    return -1;
  clear_error();
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  const CacheView &c = g->c;
  const size_t bytes = (size_t)n_tokens * c.n_heads * c.dim * 4, slot = round_up(bytes, 256);
  const bool k_host = ptr_kind(keys) != PK_DEVICE, v_host = ptr_kind(vals) != PK_DEVICE;
  const bool pageable = ptr_kind(keys) == PK_HOST_PAGEABLE || ptr_kind(vals) == PK_HOST_PAGEABLE;
  if (k_host || v_host) {
    if (!ensure_stage(g, 2 * slot, pageable ? 2 * slot : 0)) return -1;
  }
  bool ok1 = true, ok2 = true;
  const float *dk = k_host ? to_device(g, keys, bytes, 0, ok1) : keys;
  const float *dv = v_host ? to_device(g, vals, bytes, slot, ok2) : vals;
  if (!ok1 || !ok2) return -1;
  const size_t tstride = (size_t)c.n_heads * c.dim;
  if (g->uniform) {
    if (!append_device(g, dk, dv, 0, c.n_heads, n_tokens, tstride, g->u)) return -1;
    g->u = advance(c, g->u, n_tokens);
  } else {
    for (int hd = 0; hd < c.n_heads; ++hd) {
      if (!append_device(g, dk + (size_t)hd * c.dim, dv + (size_t)hd * c.dim, hd, 1, n_tokens, tstride, g->per_head[hd]))
        return -1;
      g->per_head[hd] = advance(c, g->per_head[hd], n_tokens);
    }
    g->try_unify();
  }
  if (k_host || v_host) {
    cudaError_t e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) { set_error("adaptq_mha_append_batch: CUDA error: %s", cudaGetErrorString(e)); return -1; }
  }
  return 0;
}

static int compute_all_impl(Group *g, const float *queries, int qph, float *outs, bool partial, const char *fn) {
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  const CacheView &c = g->c;
  const size_t qb = (size_t)c.n_heads * qph * c.dim * 4;
  const size_t ob = (size_t)c.n_heads * qph * (partial ? partial_floats(c) : (size_t)c.dim) * 4;
  const size_t off_out = round_up(qb, 256);
  const PtrKind qk = ptr_kind(queries), okd = ptr_kind(outs);
  if (qk != PK_DEVICE || okd != PK_DEVICE) {
    const bool pageable = qk == PK_HOST_PAGEABLE || okd == PK_HOST_PAGEABLE;
    if (!ensure_stage(g, off_out + round_up(ob, 256), pageable ? off_out + round_up(ob, 256) : 0)) return -1;
  }
  bool ok = true;
  const float *dq = qk == PK_DEVICE ? queries : to_device(g, queries, qb, 0, ok);
  if (!ok) return -1;
  float *dout = okd == PK_DEVICE ? outs : reinterpret_cast<float *>(static_cast<char *>(g->d_stage) + off_out);
  int max_n = 0;
  if (g->uniform) {
    if (!compute_device(g, dq, dout, 0, c.n_heads, qph, g->u, partial)) return -1;
    max_n = g->u.size;
  } else {
    const size_t per_head_out = (size_t)qph * (partial ? partial_floats(c) : (size_t)c.dim);
    for (int hd = 0; hd < c.n_heads; ++hd) {
      if (!compute_device(g, dq + (size_t)hd * qph * c.dim, dout + (size_t)hd * per_head_out, hd, 1, qph, g->per_head[hd], partial))
        return -1;
      max_n = std::max(max_n, g->per_head[hd].size);
    }
  }
  if (okd != PK_DEVICE) {
    void *hdst = okd == PK_HOST_PINNED ? (void *)outs : (void *)(static_cast<char *>(g->h_stage) + off_out);
    cudaError_t e = cudaMemcpyAsync(hdst, dout, ob, cudaMemcpyDeviceToHost, g->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) { set_error("%s: CUDA error: %s", fn, cudaGetErrorString(e)); return -1; }
    if (okd != PK_HOST_PINNED) memcpy(outs, hdst, ob);
  } else if (qk != PK_DEVICE) {
    cudaStreamSynchronize(g->stream);
  }
  return max_n;
}

int adaptq_mha_compute_all(adaptq_mha_t h, const float *queries, int queries_per_head, float *outs) {
  MHA_PROLOGUE("adaptq_mha_compute_all", -1)
  if (queries_per_head < 0) { set_error("adaptq_mha_compute_all: negative queries_per_head"); return -1; }
  if (queries_per_head == 0) return g->uniform ? g->u.size : 0;
  if (!require_pointer(queries, "adaptq_mha_compute_all", "queries") || !require_pointer(outs, "adaptq_mha_compute_all", "outs"))
    return -1;
  clear_error();
  return compute_all_impl(g, queries, queries_per_head, outs, false, "adaptq_mha_compute_all");
}

// One decode step over all heads: append one token per head, then one query per
// head.  With pinned host buffers the heads are cut into chunks and the chunks
// are pipelined over three streams -- upload of chunk i+1, kernels of chunk i and
// download of chunk i-1 overlap -- so the PCIe time hides behind the kernels.
#define STEP_TRY(expr)                                                                         \
  do {                                                                                         \
    cudaError_t e__ = (expr);                                                                  \
    if (e__ != cudaSuccess) {                                                                  \
      set_error("adaptq_mha_decode_step: CUDA error: %s", cudaGetErrorString(e__));            \
      return -1;                                                                               \
    }                                                                                          \
  } while (0)
int adaptq_mha_decode_step(adaptq_mha_t h, const float *keys, const float *vals, const float *queries, float *outs,
                           int token_pos) {
  MHA_PROLOGUE("adaptq_mha_decode_step", -1)
  if (!require_pointer(keys, "adaptq_mha_decode_step", "keys") || !require_pointer(vals, "adaptq_mha_decode_step", "vals") ||
      !require_pointer(queries, "adaptq_mha_decode_step", "queries") || !require_pointer(outs, "adaptq_mha_decode_step", "outs"))
    return -1;
  clear_error();
  const CacheView &c = g->c;
  constexpr int CHUNKS = 12; // at most; about eight are used
  const bool pinned = ptr_kind(keys) == PK_HOST_PINNED && ptr_kind(vals) == PK_HOST_PINNED &&
                      ptr_kind(queries) == PK_HOST_PINNED && ptr_kind(outs) == PK_HOST_PINNED;
  std::unique_lock<std::mutex> lk(g->mu);
  const bool pipeline = pinned && g->uniform && c.v_mass <= 0.f && c.n_heads >= 4096;
  if (!pipeline) {
    const bool on_device = g->uniform && ptr_kind(keys) == PK_DEVICE && ptr_kind(vals) == PK_DEVICE &&
                           ptr_kind(queries) == PK_DEVICE && ptr_kind(outs) == PK_DEVICE;
    lk.unlock();
    if (adaptq_mha_append_batch(h, keys, vals, 1, token_pos) != 0) return -1;
    if (on_device) g->append_ticket = g_launches.load(); // no copy sits between the two kernels
    const int r = adaptq_mha_compute_all(h, queries, 1, outs);
    g->append_ticket = ~0ull;
    return r;
  }
  DeviceGuard dg(g->device);
  const size_t row = (size_t)c.dim, all = (size_t)c.n_heads * row * 4, slot = round_up(all, 256);
  if (!ensure_stage(g, 4 * slot, 0)) return -1;
  if (!g->copy_in) {
    STEP_TRY(cudaStreamCreateWithFlags(&g->copy_in, cudaStreamNonBlocking));
    STEP_TRY(cudaStreamCreateWithFlags(&g->copy_out, cudaStreamNonBlocking));
  }
  while (g->ev.size() < 2 * CHUNKS + 1) {
    cudaEvent_t e;
    STEP_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    g->ev.push_back(e);
  }
  char *st = static_cast<char *>(g->d_stage);
  float *dk = reinterpret_cast<float *>(st), *dv = reinterpret_cast<float *>(st + slot),
        *dq = reinterpret_cast<float *>(st + 2 * slot), *dout = reinterpret_cast<float *>(st + 3 * slot);
  // the staging buffer may still be in use by earlier work of this handle
  STEP_TRY(cudaEventRecord(g->ev[2 * CHUNKS], g->stream));
  STEP_TRY(cudaStreamWaitEvent(g->copy_in, g->ev[2 * CHUNKS], 0));
  const RingState before = g->u, after = advance(c, before, 1);
  // about an eighth of the heads per chunk, rounded down to whole waves of persistent
  // blocks (one head per SM per round) so that no chunk ends on a partly filled wave; with
  // enough heads the first and the last chunk are small (a 32nd), because the upload of the
  // first and the download of the last are the transfers that nothing hides
  int cut[CHUNKS + 1];
  int n_chunks = 0;
  {
    const int nh = c.n_heads, sm = g->sm_count;
    int small = nh / 32;
    small -= small % sm;
    cut[0] = 0;
    if (small >= sm) {
      int per = (nh - 2 * small + 7) / 8;
      if (per >= sm) per -= per % sm;
      per = std::max(per, (nh - 2 * small + CHUNKS - 3) / (CHUNKS - 2));
      int pos = small;
      cut[++n_chunks] = pos;
      while (pos < nh - small && n_chunks < CHUNKS - 1) {
        pos = std::min(pos + per, nh - small);
        cut[++n_chunks] = pos;
      }
      cut[++n_chunks] = nh;
    } else {
      int per = (nh + 7) / 8;
      if (per >= sm) per -= per % sm;
      per = std::max(per, (nh + CHUNKS - 1) / CHUNKS);
      for (int pos = 0; pos < nh;) {
        pos = std::min(pos + per, nh);
        cut[++n_chunks] = pos;
      }
    }
  }
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int h0 = cut[ch], hc = cut[ch + 1] - cut[ch];
    if (hc <= 0) continue;
    const size_t off = (size_t)h0 * row, bytes = (size_t)hc * row * 4;
    STEP_TRY(cudaMemcpyAsync(dk + off, keys + off, bytes, cudaMemcpyHostToDevice, g->copy_in));
    STEP_TRY(cudaMemcpyAsync(dv + off, vals + off, bytes, cudaMemcpyHostToDevice, g->copy_in));
    STEP_TRY(cudaMemcpyAsync(dq + off, queries + off, bytes, cudaMemcpyHostToDevice, g->copy_in));
    STEP_TRY(cudaEventRecord(g->ev[ch], g->copy_in));
    STEP_TRY(cudaStreamWaitEvent(g->stream, g->ev[ch], 0));
    if (!append_device(g, dk + off, dv + off, h0, hc, 1, (size_t)c.n_heads * row, before)) return -1;
    g->append_ticket = g_launches.load();
    const bool computed = compute_device(g, dq + off, dout + off, h0, hc, 1, after, false);
    g->append_ticket = ~0ull;
    if (!computed) return -1;
    STEP_TRY(cudaEventRecord(g->ev[CHUNKS + ch], g->stream));
    STEP_TRY(cudaStreamWaitEvent(g->copy_out, g->ev[CHUNKS + ch], 0));
    STEP_TRY(cudaMemcpyAsync(outs + off, dout + off, bytes, cudaMemcpyDeviceToHost, g->copy_out));
  }
  g->u = after;
  STEP_TRY(cudaStreamSynchronize(g->copy_out));
  STEP_TRY(cudaStreamSynchronize(g->stream));
  return after.size;
}

int adaptq_mha_partial_floats(adaptq_mha_t h) {
  MHA_PROLOGUE("adaptq_mha_partial_floats", -1)
  return (int)partial_floats(g->c);
}

int adaptq_mha_compute_partial(adaptq_mha_t h, const float *queries, int queries_per_head, float *partials) {
  MHA_PROLOGUE("adaptq_mha_compute_partial", -1)
  if (queries_per_head <= 0) { set_error("adaptq_mha_compute_partial: queries_per_head must be positive"); return -1; }
  if (!require_pointer(queries, "adaptq_mha_compute_partial", "queries") ||
      !require_pointer(partials, "adaptq_mha_compute_partial", "partials"))
    return -1;
  const CacheView &c = g->c;
  if (c.v_mass > 0.f || c.hyb > 0 || c.k_bits == 16 || c.v_bits == 16) {
    set_error("adaptq_mha_compute_partial: needs dense V, no hybrid window and quantized K and V");
    return -1;
  }
  clear_error();
  return compute_all_impl(g, queries, queries_per_head, partials, true, "adaptq_mha_compute_partial");
}

// A rank whose shard is empty still has to tell its peers so: (max, sum) = (-inf, 0).
__global__ void deliver_empty_kernel(PeerSpec ps, int items, int pf) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= items) return;
  for (int r = 0; r < ps.n; ++r) {
    float *po = ps.out[r] + ((size_t)ps.rank * items + i) * (size_t)pf;
    po[0] = -INFINITY;
    po[1] = 0.f;
  }
  __threadfence_system();
  for (int r = 0; r < ps.n; ++r) atomicAdd_system(ps.flag[r] + ps.rank, 1u);
}

int adaptq_mha_compute_partial_to_peers(adaptq_mha_t h, const float *queries, int queries_per_head,
                                        float *const *peer_bufs, unsigned int *const *peer_flags, int world, int rank) {
  MHA_PROLOGUE("adaptq_mha_compute_partial_to_peers", -1)
  const char *fn = "adaptq_mha_compute_partial_to_peers";
  if (queries_per_head <= 0) { set_error("%s: queries_per_head must be positive", fn); return -1; }
  if (!require_pointer(queries, fn, "queries") || !require_pointer(peer_bufs, fn, "peer_bufs") ||
      !require_pointer(peer_flags, fn, "peer_flags"))
    return -1;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) { set_error("%s: need 1 <= world <= 8 and 0 <= rank < world", fn); return -1; }
  const CacheView &c = g->c;
  if (c.v_mass > 0.f || c.hyb > 0 || !stream_supported(c) || g_policy.load() == 1) {
    set_error("%s: streaming-kernel shapes only (2- or 4-bit K and V, dim 64/128, dense V, no hybrid window)", fn);
    return -1;
  }
  if (ptr_kind(queries) != PK_DEVICE) { set_error("%s: queries must be device memory", fn); return -1; }
  clear_error();
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  if (!g->uniform) { set_error("%s: heads must hold the same number of tokens", fn); return -1; }
  PeerSpec ps;
  ps.n = world; ps.rank = rank;
  for (int r = 0; r < world; ++r) {
    if (!peer_bufs[r] || !peer_flags[r]) { set_error("%s: null peer pointer", fn); return -1; }
    ps.out[r] = peer_bufs[r];
    ps.flag[r] = peer_flags[r];
  }
  const int items = c.n_heads * queries_per_head;
  if (g->u.size == 0) {
    deliver_empty_kernel<<<(items + 127) / 128, 128, 0, g->stream>>>(ps, items, (int)partial_floats(c));
    ++g_launches;
    cudaError_t e = launch_status();
    if (e != cudaSuccess) { set_error("%s: CUDA error: %s", fn, cudaGetErrorString(e)); return -1; }
    return 0;
  }
  tl_peers = &ps;
  const bool ok = compute_device(g, queries, nullptr, 0, c.n_heads, queries_per_head, g->u, true);
  tl_peers = nullptr;
  return ok ? g->u.size : -1;
}

int adaptq_mha_merge_from_peers(adaptq_mha_t h, const float *gather_buf, const unsigned int *flags, int world,
                                unsigned int expected, int queries_per_head, float *outs) {
  MHA_PROLOGUE("adaptq_mha_merge_from_peers", -1)
  const char *fn = "adaptq_mha_merge_from_peers";
  if (queries_per_head <= 0 || world < 1 || world > 8) { set_error("%s: bad world or queries_per_head", fn); return -1; }
  if (!require_pointer(gather_buf, fn, "gather_buf") || !require_pointer(flags, fn, "flags") || !require_pointer(outs, fn, "outs"))
    return -1;
  if (ptr_kind(outs) != PK_DEVICE) { set_error("%s: outs must be device memory", fn); return -1; }
  clear_error();
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  const CacheView &c = g->c;
  const int items = c.n_heads * queries_per_head;
  merge_peers_kernel<<<(items + 3) / 4, 128, 4 * c.padded * sizeof(float), g->stream>>>(
      gather_buf, (size_t)items * partial_floats(c), world, flags, expected, g->d_status, c, 0, queries_per_head, items, outs);
  ++g_launches;
  cudaError_t e = launch_status();
  if (e != cudaSuccess) { set_error("%s: CUDA error: %s", fn, cudaGetErrorString(e)); return -1; }
  return 0;
}

int adaptq_mha_merge_partials(adaptq_mha_t h, const float *partials, int n_parts, int queries_per_head, float *outs) {
  MHA_PROLOGUE("adaptq_mha_merge_partials", -1)
  if (n_parts <= 0 || queries_per_head <= 0) { set_error("adaptq_mha_merge_partials: counts must be positive"); return -1; }
  if (!require_pointer(partials, "adaptq_mha_merge_partials", "partials") ||
      !require_pointer(outs, "adaptq_mha_merge_partials", "outs"))
    return -1;
  clear_error();
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  const CacheView &c = g->c;
  const int items = c.n_heads * queries_per_head;
  const size_t pb = (size_t)n_parts * items * partial_floats(c) * 4, ob = (size_t)items * c.dim * 4;
  const size_t off_out = round_up(pb, 256);
  const PtrKind pk = ptr_kind(partials), okd = ptr_kind(outs);
  if (pk != PK_DEVICE || okd != PK_DEVICE) {
    const bool pageable = pk == PK_HOST_PAGEABLE || okd == PK_HOST_PAGEABLE;
    if (!ensure_stage(g, off_out + round_up(ob, 256), pageable ? off_out + round_up(ob, 256) : 0)) return -1;
  }
  bool ok = true;
  const float *dp = pk == PK_DEVICE ? partials : to_device(g, partials, pb, 0, ok);
  if (!ok) return -1;
  float *dout = okd == PK_DEVICE ? outs : reinterpret_cast<float *>(static_cast<char *>(g->d_stage) + off_out);
  merge_partials_kernel<<<items, CG_THREADS, c.padded * sizeof(float), g->stream>>>(
      dp, (size_t)items * partial_floats(c), n_parts, c, 0, queries_per_head, dout, 0, 0, 0);
  ++g_launches;
  cudaError_t e = launch_status();
  if (e == cudaSuccess && okd != PK_DEVICE) {
    void *hdst = okd == PK_HOST_PINNED ? (void *)outs : (void *)(static_cast<char *>(g->h_stage) + off_out);
    e = cudaMemcpyAsync(hdst, dout, ob, cudaMemcpyDeviceToHost, g->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
    if (e == cudaSuccess && okd != PK_HOST_PINNED) memcpy(outs, hdst, ob);
  } else if (e == cudaSuccess && pk != PK_DEVICE) {
    e = cudaStreamSynchronize(g->stream);
  }
  if (e != cudaSuccess) { set_error("adaptq_mha_merge_partials: CUDA error: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

int adaptq_mha_set_stream(adaptq_mha_t h, void *cuda_stream) {
  MHA_PROLOGUE("adaptq_mha_set_stream", -1)
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  cudaStreamSynchronize(g->stream);
  g->stream = static_cast<cudaStream_t>(cuda_stream);
  return 0;
}

int adaptq_mha_synchronize(adaptq_mha_t h) {
  MHA_PROLOGUE("adaptq_mha_synchronize", -1)
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  return check_status(g, "adaptq_mha_synchronize") ? 0 : -1;
}

int adaptq_mha_info(adaptq_mha_t h, adaptq_mha_info_t *info) {
  MHA_PROLOGUE("adaptq_mha_info", -1)
  if (!require_pointer(info, "adaptq_mha_info", "info")) return -1;
  const CacheView &c = g->c;
  info->n_heads = c.n_heads; info->dim = c.dim; info->padded = c.padded; info->k_bits = c.k_bits; info->v_bits = c.v_bits;
  info->capacity = c.cap; info->hybrid_thresh = c.hyb; info->k_row_bytes = c.k_row; info->v_row_bytes = c.v_row;
  info->device = g->device; info->v_mass = c.v_mass; info->device_bytes = g->device_bytes;
  return 0;
}

int adaptq_mha_export_head(adaptq_mha_t h, int head_idx, uint8_t *k_rows, uint8_t *v_rows, float *k_scale, float *v_scale,
                           int8_t *signs, int *ring_head, int *ring_size, int *mirror_tokens) {
  MHA_PROLOGUE("adaptq_mha_export_head", -1)
  if (head_idx < 0 || head_idx >= g->c.n_heads) { set_error("adaptq_mha_export_head: head_idx out of range"); return -1; }
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  const CacheView &c = g->c;
  cudaError_t e = cudaStreamSynchronize(g->stream);
  auto d2h = [&](void *dst, const void *src, size_t n) {
    if (e == cudaSuccess && dst && n) e = cudaMemcpy(dst, src, n, cudaMemcpyDeviceToHost);
  };
  d2h(k_rows, c.k_slab + (size_t)head_idx * c.k_stride, (size_t)c.cap * c.k_row);
  d2h(v_rows, c.v_slab + (size_t)head_idx * c.v_stride, (size_t)c.cap * c.v_row);
  d2h(k_scale, c.k_scale + (size_t)head_idx * c.s_stride, (size_t)c.cap * 4);
  d2h(v_scale, c.v_scale + (size_t)head_idx * c.s_stride, (size_t)c.cap * 4);
  if (e != cudaSuccess) { set_error("adaptq_mha_export_head: CUDA error: %s", cudaGetErrorString(e)); return -1; }
  if (signs) {
    std::vector<uint32_t> w((size_t)c.sign_words);
    sign_words_for(g->seeds[head_idx], c.padded, w.data(), c.sign_words);
    for (int i = 0; i < c.padded; ++i) signs[i] = ((w[i >> 5] >> (i & 31)) & 1u) ? -1 : 1;
  }
  RingState st = g->state(head_idx);
  if (ring_head) *ring_head = st.head;
  if (ring_size) *ring_size = st.size;
  if (mirror_tokens) *mirror_tokens = st.mirror;
  return 0;
}

// ---------------------------------------------------------------------------
// adaptq_mha_compute_all_static: decode attention that allocates nothing.
//
// Some callers cannot let a library touch the device allocator once they are
// running: a serving engine that has handed every free byte of HBM to its own
// pool (a late cudaMalloc simply fails there), or a latency-critical decode
// loop that cannot tolerate the device-wide synchronisation an allocation or
// free may imply.  For them the split-KV partials go into a fixed array that
// is part of the library image instead of a lazily grown cudaMalloc buffer.
//
// The array is a file-scope __device__ object: every GPU that loads the
// library holds AQ_STATIC_SCRATCH_BYTES of it until the process exits.  In
// host code its name is only a handle, not a device address, so the address
// is looked up with cudaGetSymbolAddress -- once per device, by the first
// call made while that device is current.
// ---------------------------------------------------------------------------
#define AQ_STATIC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) float g_static_partials[AQ_STATIC_SCRATCH_BYTES / sizeof(float)];
static float *g_static_partials_addr[MAX_DEVICES] = {};
static std::mutex g_static_mu;

int adaptq_mha_compute_all_static(adaptq_mha_t h, const float *queries, int queries_per_head, float *outs) {
  MHA_PROLOGUE("adaptq_mha_compute_all_static", -1)
  if (queries_per_head <= 0) { set_error("adaptq_mha_compute_all_static: queries_per_head must be positive"); return -1; }
  if (!require_pointer(queries, "adaptq_mha_compute_all_static", "queries") ||
      !require_pointer(outs, "adaptq_mha_compute_all_static", "outs"))
    return -1;
  clear_error();
  std::lock_guard<std::mutex> lk(g->mu);
  DeviceGuard dg(g->device);
  const CacheView &c = g->c;
  if (ptr_kind(queries) != PK_DEVICE || ptr_kind(outs) != PK_DEVICE) {
    set_error("adaptq_mha_compute_all_static: queries and outs must be device memory (staging host buffers would allocate)");
    return -1;
  }
  if (g->device < 0 || g->device >= MAX_DEVICES) {
    set_error("adaptq_mha_compute_all_static: device ordinal %d is not supported (0..%d)", g->device, MAX_DEVICES - 1);
    return -1;
  }
  if (g_policy.load() == 1) {
    set_error("adaptq_mha_compute_all_static: kernel policy 1 (general kernels only) excludes the streaming kernel this call needs");
    return -1;
  }
  if (!stream_supported(c) || c.v_mass > 0.f || c.hyb > 0) {
    set_error("adaptq_mha_compute_all_static: needs 2/3/4-bit K and V at head dim 64/128 (no 2-bit K at 64), dense V, no hybrid window");
    return -1;
  }
  if (!g->uniform) {
    set_error("adaptq_mha_compute_all_static: heads hold different token counts; use adaptq_mha_compute_all");
    return -1;
  }
  const int n = g->u.size;
  const int items_base = c.n_heads * queries_per_head;
  if (n == 0) {
    cudaError_t e = cudaMemsetAsync(outs, 0, (size_t)items_base * c.dim * sizeof(float), g->stream);
    if (e != cudaSuccess) { set_error("adaptq_mha_compute_all_static: CUDA error: %s", cudaGetErrorString(e)); return -1; }
    return 0;
  }
  // device address of the static scratch, once per device (this device is current)
  float *scratch;
  {
    std::lock_guard<std::mutex> sl(g_static_mu);
    if (!g_static_partials_addr[g->device]) {
      void *p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_static_partials);
      if (e != cudaSuccess || !p) {
        set_error("adaptq_mha_compute_all_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        return -1;
      }
      g_static_partials_addr[g->device] = static_cast<float *>(p);
    }
    scratch = g_static_partials_addr[g->device];
  }
  StreamLaunch a{};
  a.c = c; a.q = queries; a.out = outs; a.head0 = 0; a.heads_in_call = c.n_heads; a.nq = queries_per_head;
  a.n = n; a.status = g->d_status;
  plan_spans(n, items_base, g->sm_count, a.n_splits, a.span);
  const size_t need = (size_t)a.n_splits * items_base * partial_floats(c) * sizeof(float);
  if (a.n_splits > 1 && need > AQ_STATIC_SCRATCH_BYTES) {
    set_error("adaptq_mha_compute_all_static: %zu bytes of split-KV partials exceed the %u-byte static scratch "
              "(fewer heads or queries per call, or use adaptq_mha_compute_all)", need, (unsigned)AQ_STATIC_SCRATCH_BYTES);
    return -1;
  }
  // Every (span, head, query) slot that the merge reads is written by the
  // streaming kernel first, so nothing in the array has to start at zero.
  a.partial = scratch;
  a.force_partial = 0;
  if (!launch_stream_for_shape(g, a)) return -1;
  if (a.n_splits > 1) {
    merge_partials_kernel<<<items_base, CG_THREADS, c.padded * sizeof(float), g->stream>>>(
        scratch, (size_t)items_base * partial_floats(c), a.n_splits, c, 0, queries_per_head, outs, 0, 0, 0);
    ++g_launches;
    cudaError_t e = launch_status();
    if (e != cudaSuccess) { set_error("adaptq_mha_compute_all_static: CUDA error: %s", cudaGetErrorString(e)); return -1; }
  }
  return n;
}



} // extern "C"

#include "runtime_v2_host.inc"
#include "stack_host.inc"
