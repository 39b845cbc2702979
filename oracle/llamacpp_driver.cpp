// llamacpp_driver.cpp -- TEST INFRASTRUCTURE.
//
// Drives upstream's LlamaCppAdaptQAdapter (adapters/adapter_llamacpp.h:12-41,
// compiled from the upstream file by build_ref_binding.sh) the way its header
// says llama.cpp would: feed_kv per token and head, attention per head,
// attention_batch, kv_bytes, reset.  Inputs come from a binary file, outputs go
// to another, so a test can compare them with the CPU oracle.
//
//   llamacpp_driver <in> <out>
//   in : int32 n_heads, head_dim, bits, capacity, n_tokens, n_queries, hybrid_thresh; float32 v_mass;
//        uint64 seed; float32 keys[n_tokens][n_heads][head_dim], vals[same], queries[n_heads][n_queries][head_dim]
//   out: float32 single[n_heads][head_dim] (attention with query 0), batch[n_heads][n_queries][head_dim];
//        uint64 kv_bytes, kv_bytes_after_reset; int32 tokens_used
#include "adapter_llamacpp.h"
#include <cstdint>
#include <cstdio>
#include <vector>

int main(int argc, char **argv) {
  if (argc != 3) { std::fprintf(stderr, "usage: %s <in> <out>\n", argv[0]); return 2; }
  FILE *fi = std::fopen(argv[1], "rb");
  if (!fi) { std::perror(argv[1]); return 2; }
  int32_t hdr[7];
  float v_mass;
  uint64_t seed;
  if (std::fread(hdr, 4, 7, fi) != 7 || std::fread(&v_mass, 4, 1, fi) != 1 || std::fread(&seed, 8, 1, fi) != 1) return 2;
  const int H = hdr[0], D = hdr[1], bits = hdr[2], cap = hdr[3], T = hdr[4], NQ = hdr[5], hyb = hdr[6];
  std::vector<float> keys((size_t)T * H * D), vals((size_t)T * H * D), qs((size_t)H * NQ * D);
  if (std::fread(keys.data(), 4, keys.size(), fi) != keys.size() || std::fread(vals.data(), 4, vals.size(), fi) != vals.size() ||
      std::fread(qs.data(), 4, qs.size(), fi) != qs.size())
    return 2;
  std::fclose(fi);

  LlamaCppAdaptQAdapter adapter(H, D, bits, cap, seed, v_mass, hyb);
  for (int t = 0; t < T; ++t)
    for (int h = 0; h < H; ++h)
      adapter.feed_kv(h, keys.data() + ((size_t)t * H + h) * D, vals.data() + ((size_t)t * H + h) * D, t);
  std::vector<float> single((size_t)H * D), batch((size_t)H * NQ * D);
  int32_t used = 0;
  for (int h = 0; h < H; ++h) {
    used = adapter.attention(h, qs.data() + (size_t)h * NQ * D, single.data() + (size_t)h * D);
    adapter.attention_batch(h, qs.data() + (size_t)h * NQ * D, NQ, batch.data() + (size_t)h * NQ * D);
  }
  const uint64_t bytes = adapter.kv_bytes();
  adapter.log_memory(cap);
  adapter.reset();
  const uint64_t bytes_after = adapter.kv_bytes();

  FILE *fo = std::fopen(argv[2], "wb");
  if (!fo) { std::perror(argv[2]); return 2; }
  std::fwrite(single.data(), 4, single.size(), fo);
  std::fwrite(batch.data(), 4, batch.size(), fo);
  std::fwrite(&bytes, 8, 1, fo);
  std::fwrite(&bytes_after, 8, 1, fo);
  std::fwrite(&used, 4, 1, fo);
  std::fclose(fo);
  return used < 0 ? 1 : 0;
}
