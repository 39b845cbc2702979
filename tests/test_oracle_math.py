"""The CPU oracle against the invariants upstream's own unit tests assert for
the math layer (tests/unit/test_fwht.cpp, test_packing.cpp, test_codebook.cpp,
test_quantizer_229.cpp) and against known answers produced by the upstream
build (tests/golden/math_known_answers.npz)."""
import os

import numpy as np
import pytest

from oracle import loader

GOLD = os.path.join(os.path.dirname(__file__), "golden", "math_known_answers.npz")


@pytest.fixture(scope="module")
def ka():
    return np.load(GOLD)


def test_next_pow2_known_answers(orc, ka):
    got = [orc.next_pow2(int(x)) for x in ka["next_pow2_in"]]
    assert got == list(ka["next_pow2_out"])


def test_rademacher_known_answers(orc, ka):
    for s in (0, 1, 42, 0xDEADBEEF, 42 ^ 0xDEADBEEFCAFE):
        d = orc.signs(128, s)
        assert set(np.unique(d)) <= {-1, 1}
        assert (d == ka[f"signs_{s}"]).all()
    # seed 42 starts  - + - - - + + - - + + - + + + +   (upstream generator)
    first = "".join("+" if v > 0 else "-" for v in orc.signs(32, 42))
    assert first == "-+---++--++-++++-++-+---+++---++"
    assert (orc.signs(64, 42) != orc.signs(64, 43)).any()
    assert (orc.signs(64, 0) == orc.signs(64, 0xdeadbeefcafe1234)).all()  # seed 0 falls back


def test_fwht_known_answers_bitexact(orc, ka):
    x = ka["fwht_x"]
    sg = orc.signs(128, 42)
    assert (orc.fwht(x, sg).view(np.uint32) == ka["fwht_fwd_128"].view(np.uint32)).all()
    assert (orc.fwht(x, sg, inverse=True).view(np.uint32) == ka["fwht_inv_128"].view(np.uint32)).all()
    assert (orc.fwht(x[:96], orc.signs(96, 42)).view(np.uint32) == ka["fwht_fwd_96"].view(np.uint32)).all()


@pytest.mark.parametrize("d", [32, 64, 128, 256, 512, 1024])
def test_fwht_round_trip_and_linearity(orc, d):
    rng = np.random.default_rng(d)
    sg = orc.signs(d, 7)
    x = rng.standard_normal(d).astype(np.float32)
    y = rng.standard_normal(d).astype(np.float32)
    back = orc.fwht(orc.fwht(x, sg), sg, inverse=True)
    assert np.mean((back - x) ** 2) < 1e-10
    lin = orc.fwht((2 * x + 3 * y).astype(np.float32), sg)
    assert np.allclose(lin, 2 * orc.fwht(x, sg) + 3 * orc.fwht(y, sg), atol=1e-4)
    # orthonormal: preserves the L2 norm
    assert abs(np.linalg.norm(orc.fwht(x, sg)) - np.linalg.norm(x)) < 1e-3


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_codebook_and_quantizer_decisions(orc, ka, bits):
    cb = orc.centroids(bits)
    assert (cb == ka[f"cb_{bits}"]).all()
    assert len(cb) == 1 << bits and (np.diff(cb) > 0).all()
    assert np.allclose(cb, -cb[::-1])  # symmetric
    got = np.array([orc.quantize_fast(float(v), bits) for v in ka["q_grid"]], dtype=np.uint8)
    assert (got == ka[f"q_idx_{bits}"]).all()
    for i, c in enumerate(cb):  # a centroid quantises to itself
        assert orc.quantize_fast(float(c), bits) == i
    assert orc.quantize_fast(float("inf"), bits) == (1 << bits) - 1
    assert orc.quantize_fast(float("-inf"), bits) == 0
    assert orc.quantize_fast(float("nan"), bits) == (1 << (bits - 1)) - 1
    assert orc.quantize_fast(0.0, bits) == 1 << (bits - 1)
    assert orc.quantize_fast(-0.0, bits) == 1 << (bits - 1)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("d", [8, 32, 64, 128, 256])
def test_pack_round_trip(orc, ka, bits, d):
    rng = np.random.default_rng(bits * 1000 + d)
    idx = rng.integers(0, 1 << bits, d).astype(np.uint8)
    packed = orc.pack(idx, bits)
    assert len(packed) == d * bits // 8
    assert (orc.unpack(packed, d, bits) == idx).all()
    if d == 128:
        assert (orc.pack(ka[f"pack_idx_{bits}"], bits) == ka[f"pack_bytes_{bits}"]).all()


def test_pack_rejects_other_widths(orc):
    with pytest.raises(ValueError):
        orc.pack(np.zeros(8, dtype=np.uint8), 5)


@pytest.mark.parametrize("dim,bits,max_rel", [(64, 4, 0.15), (128, 4, 0.15), (128, 3, 0.25), (128, 2, 0.45)])
def test_quantise_dequantise_error_bounds(orc, dim, bits, max_rel):
    """Reconstruction stays within the distortion the bit width allows and the
    stored scale is the L2 norm of the input (upstream test_quantizer_229.cpp)."""
    rng = np.random.default_rng(3)
    h = loader.Head(orc, dim, bits, bits, 8, 42)
    x = rng.standard_normal(dim).astype(np.float32)
    h.append(x, x)
    assert abs(h.k_scale()[0] - np.linalg.norm(x)) < 1e-3 * np.linalg.norm(x)
    idx = orc.unpack(h.k_data()[0], h.padded, bits)
    assert idx.max() < (1 << bits) and len(np.unique(idx)) >= min(4, 1 << bits) - 1
    cb = orc.centroids(bits)
    rec = orc.fwht((cb[idx] / np.sqrt(h.padded)).astype(np.float32), h.signs(), inverse=True)[:dim] * h.k_scale()[0]
    assert np.linalg.norm(rec - x) / np.linalg.norm(x) < max_rel


def test_head_argument_checks(orc):
    for bad in [dict(dim=0), dict(k_bits=5), dict(v_bits=1), dict(capacity=-1), dict(hybrid_thresh=-1), dict(dim=1025)]:
        kw = dict(dim=64, k_bits=4, v_bits=2, capacity=8, seed=1, v_mass=0.0, hybrid_thresh=0)
        kw.update(bad)
        with pytest.raises(ValueError):
            loader.Head(orc, **kw)


def test_ring_eviction_reset_and_mirror(orc):
    """FIFO ring, kv_bytes, reset, and the hybrid mirror being dropped at the
    first eviction (upstream tests/unit/test_api.cpp:423-451)."""
    rng = np.random.default_rng(5)
    h = loader.Head(orc, 64, 4, 2, 10, 42, 0.0, 16)
    k = rng.standard_normal((25, 64)).astype(np.float32)
    h.append_many(k[:10], k[:10])
    assert (h.size, h.ring_head, h.mirror_tokens) == (10, 0, 10)
    assert h.kv_bytes == 10 * (32 + 16)
    first_rows = h.k_data().copy()
    h.append(k[10], k[10])
    assert (h.size, h.ring_head, h.mirror_tokens) == (10, 1, 0)  # evicted: mirror gone
    assert (h.k_data()[1:] == first_rows[1:]).all() and (h.k_data()[0] != first_rows[0]).any()
    out, n = h.compute(k[0])
    assert n == 10 and np.isfinite(out).all()
    h.reset()
    assert (h.size, h.ring_head, h.kv_bytes) == (0, 0, 0)
    out, n = h.compute(k[0])
    assert n == 0 and (out == 0).all()
    h.append(k[0], k[0])
    assert h.mirror_tokens == 1  # mirror builds again after a reset


def test_attention_matches_float_reference(orc):
    """K16/V16 passthrough equals plain softmax attention; 4-bit stays close
    (cosine bound as in upstream tests/test_la_policy.py:193-232)."""
    rng = np.random.default_rng(9)
    T, d = 200, 64
    K = rng.standard_normal((T, d)).astype(np.float32)
    V = rng.standard_normal((T, d)).astype(np.float32)
    q = rng.standard_normal(d).astype(np.float32)
    w = np.exp((K @ q) / np.sqrt(d) - ((K @ q) / np.sqrt(d)).max())
    want = (w / w.sum()) @ V
    h16 = loader.Head(orc, d, 16, 16, 256, 1)
    h16.append_many(K, V)
    assert np.allclose(h16.compute(q)[0], want, atol=1e-5)
    h4 = loader.Head(orc, d, 4, 4, 256, 1)
    h4.append_many(K, V)
    got = h4.compute(q)[0]
    assert np.dot(got, want) / (np.linalg.norm(got) * np.linalg.norm(want)) > 0.90
