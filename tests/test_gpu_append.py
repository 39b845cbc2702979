"""CUDA append path against the CPU oracle: packed K/V rows and scales must be
BIT-EXACT, ring state and hybrid-mirror bookkeeping equal.  Calls go through
the C ABI (adaptq_b200.MHAContext is a thin ctypes layer over it)."""
import numpy as np
import pytest

from helpers import CpuHeads, assert_cache_equal, make_kv

pytestmark = pytest.mark.gpu

# dim, k_bits, v_bits, capacity, token batches, v_mass, hybrid, dist
CASES = [
    (64, 4, 2, 256, [200], 0.0, 0, "normal"),
    (64, 4, 2, 64, [50, 1, 1, 30, 100], 0.0, 0, "student4_outlier"),      # wraps; batch larger than capacity
    (128, 4, 2, 300, [1, 2, 3, 250], 0.0, 0, "normal_outlier"),
    (128, 2, 2, 128, [128, 5], 0.0, 0, "student3"),
    (128, 4, 4, 96, [96], 0.0, 0, "student3"),
    (128, 3, 3, 80, [33, 47, 10], 0.0, 0, "lognormal_channel"),
    (64, 3, 2, 96, [96, 96], 0.0, 0, "lognormal_channel"),
    (64, 2, 4, 50, [49], 0.0, 0, "normal"),
    (64, 16, 2, 80, [40, 50], 0.0, 0, "student4_outlier"),
    (128, 16, 16, 40, [41], 0.0, 0, "normal"),
    (64, 4, 2, 700, [300, 300], 0.95, 512, "normal"),                      # mirror fills to 512 then stops
    (64, 4, 2, 100, [60, 60], 0.95, 512, "normal"),                        # mirror dropped by eviction
    (96, 4, 3, 64, [40], 0.0, 16, "normal"),                               # non power of two: padded to 128
    (40, 2, 4, 64, [37], 0.0, 0, "tiny"),                                  # tiny norms: the clip changes indices
    (256, 4, 2, 32, [20], 0.0, 0, "normal"),                               # general kernel (padded 256)
    (20, 3, 2, 16, [20], 0.0, 0, "normal"),                                # padded 32
    (1000, 4, 4, 8, [5], 0.0, 0, "normal"),                                # padded 1024
]


@pytest.mark.parametrize("dim,kb,vb,cap,batches,vm,hyb,dist", CASES)
@pytest.mark.parametrize("device_inputs", [False, True])
def test_append_bit_exact(gpu_lib, orc, dim, kb, vb, cap, batches, vm, hyb, dist, device_inputs):
    import torch
    from adaptq_b200 import MHAContext
    heads = 3
    rng = np.random.default_rng(dim + kb * 11 + vb * 7 + cap)
    ctx = MHAContext(heads, dim, kb, vb, cap, seed=42, v_mass=vm, hybrid_thresh=hyb)
    cpu = CpuHeads(orc, heads, dim, kb, vb, cap, 42, vm, hyb)
    for T in batches:
        k, v = make_kv(rng, T, heads, dim, dist)
        cpu.append_many(k, v)
        if device_inputs:
            ctx.append_all(torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
        else:
            ctx.append_all(k, v)
        ctx.synchronize()
        for h in range(heads):
            assert_cache_equal(ctx.export_head(h), cpu.heads[h], f"head {h} after batch of {T}")
    assert ctx.kv_bytes() == sum(h.kv_bytes for h in cpu.heads)


def test_per_head_calls_equal_batched_calls(gpu_lib, orc):
    """adaptq_mha_append head by head (upstream's calling pattern) lands the same
    bytes as the all-heads call, including heads that run ahead of others."""
    from adaptq_b200 import MHAContext
    heads, dim, cap = 4, 64, 24
    rng = np.random.default_rng(0)
    k, v = make_kv(rng, 40, heads, dim)
    a = MHAContext(heads, dim, 4, 2, cap, seed=7, v_mass=0.0, hybrid_thresh=8)
    cpu = CpuHeads(orc, heads, dim, 4, 2, cap, 7, 0.0, 8)
    for t in range(10):           # ragged: head h receives t tokens only while t % (h+1) == 0
        for h in range(heads):
            if t % (h + 1) == 0:
                a.append(h, k[t, h], v[t, h], t)
                cpu.heads[h].append(k[t, h], v[t, h], t)
    for h in range(heads):
        assert_cache_equal(a.export_head(h), cpu.heads[h], f"ragged head {h}")
    a.append_all(k[10:40], v[10:40])   # all-heads call on non-uniform ring state
    cpu.append_many(k[10:40], v[10:40])
    for h in range(heads):
        assert_cache_equal(a.export_head(h), cpu.heads[h], f"head {h} after batched call")
    # a long batch on the still non-uniform state: per-head launches over strided rows
    k2, v2 = make_kv(rng, 150, heads, dim)
    a.append_all(k2, v2)
    cpu.append_many(k2, v2)
    for h in range(heads):
        assert_cache_equal(a.export_head(h), cpu.heads[h], f"head {h} after the long strided batch")


def test_special_values(gpu_lib, orc):
    """Zero, huge, NaN, Inf and alternating-sign vectors (upstream tests/unit/test_api.cpp:334-358)."""
    from adaptq_b200 import MHAContext
    dim = 64
    rows = np.zeros((6, 1, dim), dtype=np.float32)
    rows[1] = 1e38
    rows[2, 0, 3] = np.nan
    rows[3, 0, 5] = np.inf
    rows[4, 0] = np.where(np.arange(dim) % 2 == 0, 1.0, -1.0)
    rows[5] = 1e-30
    for bits in (2, 3, 4):
        ctx = MHAContext(1, dim, bits, bits, 8, seed=3, v_mass=0.0, hybrid_thresh=0)
        cpu = CpuHeads(orc, 1, dim, bits, bits, 8, 3)
        ctx.append_all(rows, rows)
        cpu.append_many(rows, rows)
        e = ctx.export_head(0)
        assert (e["k_rows"][:6] == cpu.heads[0].k_data()[:6]).all()
        ks, want = e["k_scale"][:6], cpu.heads[0].k_scale()[:6]
        same = (ks.view(np.uint32) == want.view(np.uint32)) | (np.isnan(ks) & np.isnan(want))
        assert same.all()


def test_special_rows_inside_a_bulk_batch(gpu_lib, orc):
    """NaN / Inf / huge / tiny / zero vectors scattered through a 700-token batch:
    they take the general routine while their warp neighbours take the table
    quantiser; every row must still equal the oracle's."""
    from adaptq_b200 import MHAContext
    heads, dim, T = 2, 128, 700
    rng = np.random.default_rng(77)
    k, v = make_kv(rng, T, heads, dim, "normal_outlier")
    for a in (k, v):
        for t in rng.choice(T, 60, replace=False):
            kind = rng.integers(0, 6)
            h = rng.integers(0, heads)
            if kind == 0: a[t, h] = 0.0
            elif kind == 1: a[t, h, rng.integers(0, dim)] = np.nan
            elif kind == 2: a[t, h, rng.integers(0, dim)] = np.inf
            elif kind == 3: a[t, h] = 3e37
            elif kind == 4: a[t, h] *= 1e-9
            else: a[t, h] = 1e-30
    for bits in (2, 3, 4):
        ctx = MHAContext(heads, dim, bits, bits, T, seed=5, v_mass=0.0, hybrid_thresh=0)
        cpu = CpuHeads(orc, heads, dim, bits, bits, T, 5)
        ctx.append_all(k, v)
        cpu.append_many(k, v)
        ctx.synchronize()
        for h in range(heads):
            e = ctx.export_head(h)
            assert (e["k_rows"] == cpu.heads[h].k_data()).all() and (e["v_rows"] == cpu.heads[h].v_data()).all()
            for got, want in ((e["k_scale"], cpu.heads[h].k_scale()), (e["v_scale"], cpu.heads[h].v_scale())):
                assert ((got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))).all()


def test_general_and_specialised_append_agree(gpu_lib, orc):
    """Policy 1 forces the general (warp-per-vector) kernel; bytes must not change."""
    from adaptq_b200 import MHAContext
    rng = np.random.default_rng(4)
    k, v = make_kv(rng, 70, 2, 128, "normal_outlier")
    outs = []
    for policy in (0, 1):
        gpu_lib.adaptq_set_kernel_policy(policy)
        try:
            ctx = MHAContext(2, 128, 4, 2, 64, seed=1, v_mass=0.0, hybrid_thresh=0)
            ctx.append_all(k, v)
            outs.append([ctx.export_head(h) for h in range(2)])
        finally:
            gpu_lib.adaptq_set_kernel_policy(0)
    for h in range(2):
        for key in ("k_rows", "v_rows"):
            assert (outs[0][h][key] == outs[1][h][key]).all()
        assert (outs[0][h]["k_scale"].view(np.uint32) == outs[1][h]["k_scale"].view(np.uint32)).all()
