// ref_v2_shim.cpp -- TEST INFRASTRUCTURE.
//
// C entry points over UPSTREAM's second stack as it stands in the upstream
// checkout: adaptq::RuntimeContext (runtime/runtime_context.h) with its default
// HARFixedStrategy + ContiguousSlabStorage, adaptq::SessionSnapshot
// (replay/session_snapshot.h) and the process-wide adaptq::IKernelBackend
// (include/adaptq/kernel.h).  Compiled by build_ref.sh together with the upstream
// sources into oracle/_ref/libadaptq_ref_v2.so; tests use it to check this
// repository's include/adaptq_runtime.h implementation against upstream itself.
#include "runtime/runtime_context.h"
#include "replay/session_snapshot.h"
#include "include/adaptq/kernel.h"
#include "include/adaptq/storage.h"

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>
#include <vector>

using namespace adaptq;

static thread_local char tl_msg[512] = "";
static void keep(const std::exception &e) { std::snprintf(tl_msg, sizeof(tl_msg), "%s", e.what()); }

extern "C" {

const char *refv2_last_error(void) { return tl_msg; }

void *refv2_create(int n_layers, int n_heads, int dim, int bits, int capacity, float v_mass) {
  try {
    RuntimeContextConfig cfg;
    cfg.n_layers = n_layers; cfg.n_heads = n_heads; cfg.dim = dim; cfg.bits = bits; cfg.capacity = capacity; cfg.v_mass = v_mass;
    cfg.log_tokens = false;
    auto *rt = new RuntimeContext();
    rt->init(cfg);
    return rt;
  } catch (const std::exception &e) { keep(e); return nullptr; }
}
void refv2_destroy(void *rt) { delete static_cast<RuntimeContext *>(rt); }

int refv2_append(void *rt, int layer, int head, const float *k, const float *v) {
  try { static_cast<RuntimeContext *>(rt)->append(layer, head, k, v); return 0; }
  catch (const std::exception &e) { keep(e); return -1; }
}
int refv2_compute(void *rt, int layer, int head, const float *q, float *out) {
  try { return static_cast<RuntimeContext *>(rt)->compute(layer, head, q, out).n_tokens_used; }
  catch (const std::exception &e) { keep(e); return -1; }
}
int refv2_token_pos(void *rt) { return static_cast<RuntimeContext *>(rt)->token_pos(); }

// SessionSnapshot::capture(ctx, false).save(path)
int refv2_snapshot_save(void *rt, const char *path) {
  try { SessionSnapshot::capture(*static_cast<RuntimeContext *>(rt), false).save(path); return 0; }
  catch (const std::exception &e) { keep(e); return -1; }
}
// SessionSnapshot::load(path): 0 and the header fields + per-head cache sizes (up to max_heads), or -1.
int refv2_snapshot_load(const char *path, int *hdr /* n_layers,n_heads,dim,bits,n_tokens,n_head_blocks,flags */,
                        int *cache_sizes, int max_heads) {
  try {
    SessionSnapshot s = SessionSnapshot::load(path);
    if (!s.is_valid()) { std::snprintf(tl_msg, sizeof(tl_msg), "not valid"); return -1; }
    hdr[0] = s.n_layers(); hdr[1] = s.n_heads(); hdr[2] = s.dim(); hdr[3] = s.bits(); hdr[4] = s.n_tokens();
    hdr[5] = (int)s.heads().size(); hdr[6] = (s.has_token_log() ? 1 : 0) | (s.has_strategy_state() ? 2 : 0);
    for (int i = 0; i < (int)s.heads().size() && i < max_heads; ++i) cache_sizes[i] = s.heads()[i].cache_size;
    return 0;
  } catch (const std::exception &e) { keep(e); return -1; }
}

// The process-wide kernel backend (kernels/kernel_selector.cpp:96-102).
const char *refv2_kernel_name(void) { return select_kernel_backend()->name(); }
void refv2_kernel_fwht(float *x, const int8_t *D, int padded, int inverse) {
  if (inverse) select_kernel_backend()->fwht_inverse(x, D, padded);
  else select_kernel_backend()->fwht_forward(x, D, padded);
}
static std::vector<CompressResult> as_results(const uint8_t *rows, size_t stride, const float *scales, int n, int bytes, int bits) {
  std::vector<CompressResult> r((size_t)n);
  for (int i = 0; i < n; ++i) r[i] = CompressResult{rows + (size_t)i * stride, bytes, scales[i], (uint8_t)bits, (StorageSlot)i};
  return r;
}
void refv2_kernel_kdot_batch(const float *q_rot, const uint8_t *rows, size_t stride, const float *scales, int n, int padded,
                             int bits, float *logits_out) {
  auto r = as_results(rows, stride, scales, n, (padded * bits + 7) / 8, bits);
  select_kernel_backend()->kdot_batch(q_rot, r.data(), n, padded, bits, logits_out);
}
void refv2_kernel_vaccum_batch(float *acc, const uint8_t *rows, size_t stride, const float *scales, const float *weights, int n,
                               int padded, int bits) {
  auto r = as_results(rows, stride, scales, n, (padded * bits + 7) / 8, bits);
  select_kernel_backend()->vaccum_batch(acc, r.data(), weights, n, padded, bits);
}

} // extern "C"
