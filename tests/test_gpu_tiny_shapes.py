"""The smallest and most awkward shapes: empty caches, capacity 1, appends of 0, 1, 3,
4 and 5 tokens, rings that wrap in the middle of a 64-vector tile, batches longer than
the capacity, every bit-width pair class -- rows bit-exact against the CPU oracle,
outputs within tolerance, and adaptq_mha_synchronize() clean at the end (in the checked
build of the library that also verifies the guard bytes behind every device buffer and
the device-side index checks; tests/test_gpu_checked_build.py runs this file under it)."""
import numpy as np
import pytest

from helpers import CpuHeads, assert_cache_equal, assert_close, assert_sparse_close, make_kv

pytestmark = pytest.mark.gpu

BITS = [(4, 2), (2, 2), (4, 4), (3, 2), (16, 2), (4, 16), (16, 16), (3, 3)]


@pytest.mark.parametrize("kb,vb", BITS)
@pytest.mark.parametrize("dim,cap", [(64, 1), (64, 4), (128, 4), (128, 70), (96, 5)])
def test_tiny_and_wrapping(gpu_lib, orc, kb, vb, dim, cap):
    from adaptq_b200 import MHAContext
    heads = 3
    rng = np.random.default_rng(dim + cap + kb + vb)
    ctx = MHAContext(heads, dim, kb, vb, cap, seed=3, v_mass=0.0, hybrid_thresh=0)
    cpu = CpuHeads(orc, heads, dim, kb, vb, cap, 3)
    q = rng.standard_normal((heads, dim)).astype(np.float32)
    assert not np.any(ctx.compute_all(q))                        # empty cache: zeros
    for n in (0, 1, 3, 4, 5, 64, 13, 1, cap + 7):                # 64 + 13 straddles a tile and (cap 70) the ring end
        if n == 0:
            ctx.append_all(np.zeros((0, heads, dim), np.float32), np.zeros((0, heads, dim), np.float32))
        else:
            k, v = make_kv(rng, n, heads, dim)
            ctx.append_all(k, v)
            cpu.append_many(k, v)
        for h in range(heads):
            assert_cache_equal(ctx.export_head(h), cpu.heads[h], f"after {n} tokens, head {h}")
        if cpu.heads[0].size:
            assert_close(ctx.compute_all(q), cpu.compute(q), f"after {n} tokens")
    # one head at a time (per-head ring states diverge), then all together again
    k, v = make_kv(rng, 3, heads, dim)
    for t in range(3):
        ctx.append(1, k[t, 1], v[t, 1], t)
        cpu.heads[1].append(k[t, 1], v[t, 1])
    for h in range(heads):
        assert_cache_equal(ctx.export_head(h), cpu.heads[h], f"single-head appends, head {h}")
        assert_close(ctx.compute(h, q[h]), cpu.heads[h].compute(q[h])[0], f"single-head compute {h}")
    ctx.synchronize()
    ctx.reset()
    assert ctx.kv_bytes() == 0
    ctx.synchronize()


@pytest.mark.parametrize("cap,hyb", [(4, 2), (6, 512), (1, 1)])
def test_tiny_with_engine_defaults(gpu_lib, orc, cap, hyb):
    """Sparse V and the FP32 window on rings of a few tokens."""
    from adaptq_b200 import MHAContext
    heads, dim = 2, 64
    rng = np.random.default_rng(cap)
    ctx = MHAContext(heads, dim, 4, 2, cap, seed=3, v_mass=0.95, hybrid_thresh=hyb)
    cpu = CpuHeads(orc, heads, dim, 4, 2, cap, 3, 0.95, hyb)
    for step in range(cap + 3):
        k, v = make_kv(rng, 1, heads, dim)
        q = rng.standard_normal((heads, dim)).astype(np.float32)
        out = ctx.decode_step(k[0], v[0], q, pos=step)
        cpu.append_many(k, v)
        for h in range(heads):
            hd = cpu.heads[h]
            if hd.mirror_tokens == hd.size and hd.size <= hyb:
                assert_close(out[h], hd.compute(q[h])[0], f"step {step} head {h} (FP32 window)")
            else:
                assert_sparse_close(out[h], hd, q[h], 0.95, f"step {step} head {h}")
    ctx.synchronize()
