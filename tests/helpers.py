"""Shared helpers for the parity tests: seeded inputs, CPU-checker runs, tolerances."""
from __future__ import annotations

import numpy as np

from oracle import loader

# Tolerance for attention outputs and scales (fp32): |a-b| <= ATOL + RTOL*|b|
RTOL = 1e-5
ATOL = 1e-4


def make_kv(rng, n_tokens, heads, dim, dist="normal"):
    """[n_tokens, heads, dim] float32 keys and values."""
    shape = (n_tokens, heads, dim)
    if dist == "normal":
        k, v = rng.standard_normal(shape), rng.standard_normal(shape)
    elif dist == "student3":
        k, v = rng.standard_t(3, shape), rng.standard_t(3, shape)
    elif dist == "student4_outlier":  # heavy tails + 3 fixed channels per head scaled x10
        k, v = rng.standard_t(4, shape), rng.standard_t(4, shape)
        ch = np.random.default_rng(1).choice(dim, size=(heads, 3))
        for h in range(heads):
            k[:, h, ch[h]] *= 10.0
            v[:, h, ch[h]] *= 10.0
    elif dist == "normal_outlier":  # 1% of entries replaced by N(0,20)
        k, v = rng.standard_normal(shape), rng.standard_normal(shape)
        for a in (k, v):
            m = rng.random(shape) < 0.01
            a[m] = rng.standard_normal(int(m.sum())) * 20.0
    elif dist == "lognormal_channel":  # N(0,1) x per-channel log-normal(0, 0.5) scale
        s = np.exp(0.5 * rng.standard_normal((1, heads, dim)))
        k, v = rng.standard_normal(shape) * s, rng.standard_normal(shape) * s
    elif dist == "tiny":
        k, v = rng.standard_normal(shape) * 1e-7, rng.standard_normal(shape) * 3e-7
    else:
        raise ValueError(dist)
    return k.astype(np.float32), v.astype(np.float32)


class CpuHeads:
    """`heads` independent CPU-checker heads seeded like a multi-head handle."""

    def __init__(self, lib, heads, dim, k_bits, v_bits, capacity, base_seed, v_mass=0.0, hybrid_thresh=0, seeds=None):
        self.heads = [loader.Head(lib, dim, k_bits, v_bits, capacity,
                                  seeds[h] if seeds is not None else loader.mha_head_seed(base_seed, h),
                                  v_mass, hybrid_thresh) for h in range(heads)]
        self.dim = dim

    def append_many(self, keys, vals):  # [T, H, dim]
        for h, hd in enumerate(self.heads):
            hd.append_many(keys[:, h, :], vals[:, h, :])

    def compute(self, q):  # [H, dim] -> [H, dim]
        return np.stack([hd.compute(q[h])[0] for h, hd in enumerate(self.heads)])

    def compute_batch(self, q):  # [H, nq, dim]
        return np.stack([hd.compute_batch(q[h])[0] for h, hd in enumerate(self.heads)])

    def reset(self):
        for hd in self.heads:
            hd.reset()


def assert_close(got, want, what="", rtol=RTOL, atol=ATOL):
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bound = atol + rtol * np.abs(want.astype(np.float64))
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.size} outside tolerance; worst at {i}: "
                             f"got {got[i]!r} want {want[i]!r} (|err| {err[i]:.3e}, bound {bound[i]:.3e})")


def assert_cache_equal(exported, head: loader.Head, what=""):
    """Packed rows bit-exact, scales bit-exact, ring state equal (live slots only)."""
    n, cap = head.size, head.capacity
    assert exported["ring_size"] == n, f"{what}: ring size {exported['ring_size']} vs {n}"
    assert exported["ring_head"] == head.ring_head, f"{what}: ring head"
    assert exported["mirror_tokens"] == head.mirror_tokens, f"{what}: mirror tokens"
    live = np.arange(cap) if n == cap else np.arange(n)
    kd, vd = head.k_data(), head.v_data()
    ke, ve = exported["k_rows"], exported["v_rows"]
    assert ke.shape == kd.shape and ve.shape == vd.shape, f"{what}: row geometry"
    bad_k = np.nonzero((ke[live] != kd[live]).any(axis=1))[0]
    bad_v = np.nonzero((ve[live] != vd[live]).any(axis=1))[0]
    assert bad_k.size == 0, f"{what}: {bad_k.size} K rows differ, first slot {live[bad_k[0]]}"
    assert bad_v.size == 0, f"{what}: {bad_v.size} V rows differ, first slot {live[bad_v[0]]}"
    ks, vs = head.k_scale(), head.v_scale()
    assert (exported["k_scale"][live].view(np.uint32) == ks[live].view(np.uint32)).all(), f"{what}: K scales differ"
    assert (exported["v_scale"][live].view(np.uint32) == vs[live].view(np.uint32)).all(), f"{what}: V scales differ"
    assert (exported["signs"] == head.signs()).all(), f"{what}: signs differ"


def unpack_rows(lib, rows, P, bits):
    """[n, row_bytes] packed rows -> [n, P] indices (MSB-first layouts of
    core/quantizer.cpp:156-194); vectorised for 2 and 4 bits, row by row otherwise."""
    rows = np.asarray(rows, dtype=np.uint8)
    if bits == 4:
        return np.stack([rows >> 4, rows & 15], axis=-1).reshape(rows.shape[0], -1)[:, :P]
    if bits == 2:
        return np.stack([rows >> 6, (rows >> 4) & 3, (rows >> 2) & 3, rows & 3], axis=-1).reshape(rows.shape[0], -1)[:, :P]
    return np.stack([lib.unpack(r, P, bits) for r in rows])


# How close to v_mass the running mass must be at a block boundary for a sparse-V
# cut to count as borderline.  The CUDA weights differ from the CPU's in their last
# bits (other exp routine, other summation order of the normaliser), so a mass that
# the CPU sees a hair below v_mass the GPU may see a hair above, and the walk stops
# one step earlier or later.  1e-5 is ~170 float ulps of a mass near 1.
SPARSE_MASS_SLACK = 1e-5


def assert_sparse_close(got, head: "loader.Head", q, v_mass, what="", block=4):
    """Sparse-V output of the CUDA path against the oracle head `head` (which must be the
    C restatement).  Inside tolerance: fine.  Outside: accepted only if (a) the oracle's
    running mass at the neighbouring step boundary is within SPARSE_MASS_SLACK of v_mass
    and (b) the output matches the oracle re-run with the cut moved to that boundary,
    within the normal tolerance.  Returns True if the plain comparison passed."""
    want, mass, count = head.sparse_trace(q)
    try:
        assert_close(got, want, what)
        return True
    except AssertionError as first:
        alts = []
        if len(mass) >= 2 and v_mass - float(mass[-2]) <= SPARSE_MASS_SLACK:
            alts.append(int(count[-2]))                      # the GPU stopped one step earlier
        if len(mass) >= 1 and float(mass[-1]) - v_mass <= SPARSE_MASS_SLACK and int(count[-1]) < head.size:
            c = int(count[-1])
            alts.append(c + 4 if (block == 4 and c + 3 < head.size) else c + 1)  # ... or one step later
        for c in alts:
            try:
                assert_close(got, head.compute_cut(q, c), what)
                return False
            except AssertionError:
                pass
        raise AssertionError(f"{what}: sparse-V output differs and the cut is not borderline "
                             f"(mass trail {mass[-3:]}, rows {count[-3:]}, v_mass {v_mass}); {first}") from None


def exact_attention_f64(lib, head: loader.Head, q):
    """Dense attention over a CPU head's packed cache evaluated in float64: the
    yardstick for inputs whose logits are so large that the FP32 reference itself
    carries visible rounding noise."""
    P, dim = head.padded, head.dim
    n = head.size
    H = np.array([[1.0]])
    while H.shape[0] < P:
        H = np.block([[H, H], [H, -H]])
    sg = head.signs().astype(np.float64)
    x = np.zeros(P)
    x[:dim] = np.asarray(q, dtype=np.float64)
    qn = np.sqrt(np.sum(x * x) + 1e-12)
    qr = H @ (x / qn * sg) * qn  # (1/sqrt p) and sqrt p cancel
    from_rows = lambda rows, bits: lib.centroids(bits).astype(np.float64)[unpack_rows(lib, rows, P, bits)]
    kb = head.k_row_bytes * 8 // P
    vb = head.v_row_bytes * 8 // P
    K = from_rows(head.k_data()[:n], kb)
    V = from_rows(head.v_data()[:n], vb)
    logits = (K @ qr) / (np.sqrt(dim) * P) * head.k_scale()[:n].astype(np.float64)
    e = np.exp(logits - logits.max())
    acc = (e / e.sum() * head.v_scale()[:n].astype(np.float64) / np.sqrt(P)) @ V
    return ((H @ acc) / np.sqrt(P) * sg)[:dim]


def assert_close_conditioned(got, want, exact, what=""):
    """Within the FP32 tolerance of the reference, or -- where the reference itself
    sits further than that from the float64 value -- at least as close to the
    float64 value as the reference is (with 50 % slack)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    exact = np.asarray(exact, dtype=np.float64)
    bound = ATOL + RTOL * np.abs(want)
    ok = (np.abs(got - want) <= bound) | (np.abs(got - exact) <= 1.5 * np.abs(want - exact) + bound)
    if not ok.all():
        i = np.unravel_index(np.argmin(ok), ok.shape)
        raise AssertionError(f"{what}: {int((~ok).sum())} of {ok.size} outside tolerance; first at {i}: got {got[i]!r} "
                             f"reference {want[i]!r} float64 {exact[i]!r}")
