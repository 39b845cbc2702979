"""Generate the golden fixtures in this directory from the UPSTREAM build
(oracle/_ref/libadaptq_ref.so, made by oracle/build_ref.sh).  Run where the
upstream sources are available:

    python tests/golden/make_golden.py

Each .npz holds the seeded inputs and what upstream produced: packed K/V rows,
scales, ring state and attention outputs.  Tests check both the C restatement
(oracle/) and the CUDA library against them.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from oracle import loader  # noqa: E402
from helpers import make_kv  # noqa: E402

# name, dim, heads, k_bits, v_bits, capacity, tokens, v_mass, hybrid, dist, base_seed
CASES = [
    ("d64_k4v2_dense", 64, 2, 4, 2, 96, 80, 0.0, 0, "normal", 42),
    ("d64_k4v2_engine_defaults", 64, 2, 4, 2, 640, 600, 0.95, 512, "normal", 42),
    ("d64_k4v2_hybrid_window", 64, 2, 4, 2, 640, 100, 0.95, 512, "normal", 42),
    ("d128_k4v2_dense_outlier", 128, 2, 4, 2, 96, 96, 0.0, 0, "normal_outlier", 7),
    ("d128_k2v2_dense_student", 128, 2, 2, 2, 64, 64, 0.0, 0, "student3", 11),
    ("d128_k4v4_dense_student", 128, 2, 4, 4, 64, 50, 0.0, 0, "student3", 11),
    ("d64_k3v2_wrap", 64, 2, 3, 2, 48, 70, 0.0, 0, "lognormal_channel", 43),
    ("d64_k16v2_passthrough", 64, 2, 16, 2, 64, 40, 0.0, 0, "student4_outlier", 42),
    ("d96_k4v3_padded", 96, 2, 4, 3, 40, 33, 0.0, 0, "normal", 5),
    ("d64_k16v16_fp32", 64, 1, 16, 16, 32, 20, 0.0, 0, "normal", 9),
]


def main():
    R = loader.reference()
    for (name, dim, heads, kb, vb, cap, T, vm, hyb, dist, seed) in CASES:
        rng = np.random.default_rng(sum(map(ord, name)))
        keys, vals = make_kv(rng, T, heads, dim, dist)
        queries = rng.standard_normal((3, heads, dim)).astype(np.float32)
        out = {"dim": dim, "heads": heads, "k_bits": kb, "v_bits": vb, "capacity": cap, "v_mass": np.float32(vm),
               "hybrid_thresh": hyb, "base_seed": seed, "keys": keys, "vals": vals, "queries": queries}
        outs = np.zeros((3, heads, dim), dtype=np.float32)
        for h in range(heads):
            hd = loader.Head(R, dim, kb, vb, cap, loader.mha_head_seed(seed, h), vm, hyb)
            hd.append_many(keys[:, h], vals[:, h])
            out[f"k_rows_{h}"] = hd.k_data()
            out[f"v_rows_{h}"] = hd.v_data()
            out[f"k_scale_{h}"] = hd.k_scale()
            out[f"v_scale_{h}"] = hd.v_scale()
            out[f"signs_{h}"] = hd.signs()
            out[f"ring_{h}"] = np.array([hd.ring_head, hd.size, hd.mirror_tokens], dtype=np.int32)
            for i in range(3):
                outs[i, h], n = hd.compute(queries[i, h])
                assert n == hd.size
        out["outs"] = outs
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "ok")

    # math-layer known answers
    ka = {}
    ka["next_pow2_in"] = np.array([0, 1, 2, 3, 4, 5, 7, 8, 9, 63, 64, 65, 96, 100, 127, 128, 129, 255, 256, 1000, 1024], dtype=np.int32)
    ka["next_pow2_out"] = np.array([R.next_pow2(int(x)) for x in ka["next_pow2_in"]], dtype=np.int32)
    for s in (0, 1, 42, 0xDEADBEEF, 42 ^ 0xDEADBEEFCAFE):
        ka[f"signs_{s}"] = R.signs(128, s)
    rng = np.random.default_rng(2024)
    x = rng.standard_normal(128).astype(np.float32)
    sg = R.signs(128, 42)
    ka["fwht_x"] = x
    ka["fwht_fwd_128"] = R.fwht(x, sg)
    ka["fwht_inv_128"] = R.fwht(x, sg, inverse=True)
    ka["fwht_fwd_96"] = R.fwht(x[:96], R.signs(96, 42))
    grid = np.concatenate([np.linspace(-4, 4, 2001), [np.inf, -np.inf, np.nan, 0.0, -0.0, 3.4e38, -3.4e38, 1e-45]]).astype(np.float32)
    ka["q_grid"] = grid
    for b in (2, 3, 4):
        ka[f"q_idx_{b}"] = np.array([R.quantize_fast(float(v), b) for v in grid], dtype=np.uint8)
        ka[f"cb_{b}"] = R.centroids(b)
        idx = rng.integers(0, 1 << b, 128).astype(np.uint8)
        ka[f"pack_idx_{b}"] = idx
        ka[f"pack_bytes_{b}"] = R.pack(idx, b)
    np.savez_compressed(os.path.join(HERE, "math_known_answers.npz"), **ka)
    print("math_known_answers ok")


if __name__ == "__main__":
    main()
