"""Pins the C restatement (oracle/adaptq_oracle.c) against the upstream sources
compiled by oracle/build_ref.sh: packed rows, scales, ring state AND attention
outputs must agree bit for bit.  Skipped where the upstream build is absent;
tests/test_golden.py then carries the pin through the committed fixtures."""
import numpy as np
import pytest

from oracle import loader
from helpers import make_kv

CASES = [
    # dim, k_bits, v_bits, capacity, tokens, v_mass, hybrid, dist
    (64, 4, 2, 300, 257, 0.0, 0, "normal"),
    (64, 4, 2, 128, 300, 0.0, 0, "student4_outlier"),
    (128, 4, 2, 200, 333, 0.0, 0, "normal_outlier"),
    (128, 2, 2, 256, 256, 0.0, 0, "student3"),
    (128, 4, 4, 256, 255, 0.0, 0, "student3"),
    (128, 3, 3, 64, 100, 0.0, 0, "lognormal_channel"),
    (64, 3, 2, 96, 96, 0.0, 0, "lognormal_channel"),
    (64, 2, 4, 50, 49, 0.0, 0, "normal"),
    (64, 16, 2, 80, 100, 0.0, 0, "student4_outlier"),
    (64, 16, 16, 80, 60, 0.0, 0, "normal"),
    (128, 16, 4, 40, 40, 0.0, 0, "normal"),
    (64, 4, 2, 2048, 700, 0.95, 512, "normal"),   # Engine defaults past the hybrid window: sparse V
    (64, 4, 2, 2048, 300, 0.95, 512, "normal"),   # inside the hybrid window
    (96, 4, 2, 100, 150, 0.95, 512, "normal"),    # non-power-of-two dim, mirror dropped by eviction
    (96, 3, 3, 100, 70, 0.7, 64, "normal"),
    (40, 2, 4, 64, 37, 0.0, 0, "tiny"),           # tiny norms: the +-3 sigma clip bites
    (256, 4, 2, 64, 37, 0.0, 0, "normal"),
    (512, 3, 2, 32, 20, 0.0, 0, "normal"),
    (32, 4, 2, 64, 37, 0.7, 0, "normal"),
]


@pytest.mark.parametrize("dim,kb,vb,cap,T,vm,hyb,dist", CASES)
def test_oracle_equals_upstream_bitwise(orc, ref, dim, kb, vb, cap, T, vm, hyb, dist):
    rng = np.random.default_rng(dim * 7 + kb * 5 + vb * 3 + T)
    keys, vals = make_kv(rng, T, 1, dim, dist)
    ho = loader.Head(orc, dim, kb, vb, cap, 42, vm, hyb)
    hr = loader.Head(ref, dim, kb, vb, cap, 42, vm, hyb)
    ho.append_many(keys[:, 0], vals[:, 0])
    hr.append_many(keys[:, 0], vals[:, 0])
    assert (ho.size, ho.ring_head, ho.mirror_tokens) == (hr.size, hr.ring_head, hr.mirror_tokens)
    assert (ho.k_data() == hr.k_data()).all() and (ho.v_data() == hr.v_data()).all()
    assert (ho.k_scale().view(np.uint32) == hr.k_scale().view(np.uint32)).all()
    assert (ho.v_scale().view(np.uint32) == hr.v_scale().view(np.uint32)).all()
    assert (ho.signs() == hr.signs()).all()
    assert ho.kv_bytes == hr.kv_bytes
    for i in range(4):
        q = rng.standard_normal(dim).astype(np.float32)
        a, na = ho.compute(q)
        b, nb = hr.compute(q)
        assert na == nb
        assert (a.view(np.uint32) == b.view(np.uint32)).all(), f"query {i}: max |diff| {np.abs(a - b).max()}"


def test_special_values_match_upstream(orc, ref):
    """Zero, huge, NaN and Inf vectors go through append without a crash and
    pack to the same bytes (upstream tests/unit/test_api.cpp:334-358)."""
    dim = 64
    rows = np.zeros((6, dim), dtype=np.float32)
    rows[1] = 1e38
    rows[2, 3] = np.nan
    rows[3, 5] = np.inf
    rows[4] = np.where(np.arange(dim) % 2 == 0, 1.0, -1.0)
    rows[5] = 1e-30
    for bits in (2, 3, 4):
        ho = loader.Head(orc, dim, bits, bits, 8, 3)
        hr = loader.Head(ref, dim, bits, bits, 8, 3)
        ho.append_many(rows, rows)
        hr.append_many(rows, rows)
        assert (ho.k_data() == hr.k_data()).all()
        assert (ho.k_scale().view(np.uint32) == hr.k_scale().view(np.uint32)).all()


def test_math_layer_matches_upstream(orc, ref):
    rng = np.random.default_rng(1)
    for d in (16, 64, 96, 128, 200, 1024):
        x = rng.standard_normal(d).astype(np.float32)
        sg = ref.signs(d, 99)
        assert (orc.signs(d, 99) == sg).all()
        assert (orc.fwht(x, sg).view(np.uint32) == ref.fwht(x, sg).view(np.uint32)).all()
        assert (orc.fwht(x, sg, True).view(np.uint32) == ref.fwht(x, sg, True).view(np.uint32)).all()
    for bits in (2, 3, 4):
        for v in np.concatenate([rng.standard_normal(500) * 1.5, [0.0, -0.0, np.inf, -np.inf, np.nan]]):
            assert orc.quantize_fast(float(np.float32(v)), bits) == ref.quantize_fast(float(np.float32(v)), bits)
        # exactly on, just below and just above every threshold
        cb = ref.centroids(bits)
        for i in range(len(cb) - 1):
            t = np.float32((cb[i] + cb[i + 1]) * np.float32(0.5))
            for v in (t, np.nextafter(t, np.float32(-9)), np.nextafter(t, np.float32(9))):
                assert orc.quantize_fast(float(v), bits) == ref.quantize_fast(float(v), bits)
