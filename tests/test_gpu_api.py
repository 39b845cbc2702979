"""C-ABI behaviour on a device: error strings, empty cache, reset, kv_bytes and
the Python mirrors (Engine, AdaptQAttention) -- restating upstream's
tests/unit/test_api.cpp, tests/test_la_policy.py and tests/test_torch_adapter.py."""
import ctypes as C

import numpy as np
import pytest

from helpers import CpuHeads, assert_close, make_kv

pytestmark = pytest.mark.gpu


def test_single_head_handle(gpu_lib, orc):
    L = gpu_lib
    err = lambda: L.adaptq_last_error().decode()
    h = C.c_void_p(L.adaptq_create(64, 4, 2, 32, 42, C.c_float(0.0), 0))
    assert h
    q = np.ones(64, dtype=np.float32)
    out = np.full(64, 7.0, dtype=np.float32)
    assert L.adaptq_compute(h, q.ctypes.data, out.ctypes.data) == 0 and (out == 0).all()  # empty: zeros
    assert L.adaptq_compute(h, None, out.ctypes.data) == -1 and err() == "adaptq_compute: null query"
    assert L.adaptq_compute(h, q.ctypes.data, None) == -1 and err() == "adaptq_compute: null out"
    L.adaptq_append(h, None, q.ctypes.data, 0)
    assert err() == "adaptq_append: null key"
    assert L.adaptq_compute_batch(h, q.ctypes.data, -1, out.ctypes.data) == -1
    assert err() == "adaptq_compute_batch: negative num_queries"
    assert L.adaptq_compute_batch(h, None, 0, None) == 0
    rng = np.random.default_rng(0)
    k, v = make_kv(rng, 40, 1, 64)
    cpu = CpuHeads(orc, 1, 64, 4, 2, 32, 0, seeds=[42])
    for t in range(40):
        L.adaptq_append(h, k[t, 0].ctypes.data, v[t, 0].ctypes.data, t)
    cpu.append_many(k, v)
    assert L.adaptq_kv_bytes(h) == 32 * (32 + 16)
    assert L.adaptq_compute(h, q.ctypes.data, out.ctypes.data) == 32
    assert_close(out, cpu.compute(q[None])[0], "single-head handle")
    L.adaptq_reset(h)
    assert L.adaptq_kv_bytes(h) == 0 and err() == ""
    assert L.adaptq_compute(h, q.ctypes.data, out.ctypes.data) == 0 and (out == 0).all()
    L.adaptq_destroy(h)


def test_mha_errors(gpu_lib):
    L = gpu_lib
    err = lambda: L.adaptq_last_error().decode()
    m = C.c_void_p(L.adaptq_mha_create(2, 64, 4, 4, 16, 1, C.c_float(0.0), 0))
    x = np.ones(64, dtype=np.float32)
    L.adaptq_mha_append(m, 2, x.ctypes.data, x.ctypes.data, 0)
    assert err() == "adaptq_mha_append: head_idx out of range"
    assert L.adaptq_mha_compute(m, -1, x.ctypes.data, x.ctypes.data) == -1
    assert err() == "adaptq_mha_compute: head_idx out of range"
    assert L.adaptq_mha_compute_batch(m, 0, x.ctypes.data, -2, x.ctypes.data) == -1
    assert err() == "adaptq_mha_compute_batch: negative num_queries"
    L.adaptq_mha_append(m, 0, x.ctypes.data, x.ctypes.data, 0)
    assert err() == ""  # success clears the string on the multi-head calls
    assert L.adaptq_mha_total_kv_bytes(m) == 64
    L.adaptq_mha_destroy(m)


def test_long_context_returns_exact_count(gpu_lib):
    """A 70 000-token ring returns exactly n (upstream test_api.cpp:303-330)."""
    from adaptq_b200 import MHAContext
    import torch
    ctx = MHAContext(1, 64, 2, 2, 70000, seed=1, v_mass=0.0, hybrid_thresh=0)
    g = torch.Generator(device="cuda").manual_seed(0)
    kv = torch.randn((65600, 1, 64), device="cuda", generator=g)
    ctx.append_all(kv, kv)
    q = np.ones(64, dtype=np.float32)
    out = np.zeros(64, dtype=np.float32)
    n = gpu_lib.adaptq_mha_compute(ctx._h, 0, q.ctypes.data, out.ctypes.data)
    assert n == 65600 and np.isfinite(out).all()


def test_engine_surface(gpu_lib, orc):
    from adaptq_b200 import Engine
    e = Engine(dim=64, heads=4, k_bits=4, v_bits=2, capacity=256, seed=42)
    assert (e.dim, e.heads, e.k_bits, e.v_bits, e.capacity, e.pos) == (64, 4, 4, 2, 256, 0)
    with pytest.raises(ValueError, match=r"k and v must be shape \(4, 64\)"):
        e.append(np.zeros((3, 64), np.float32), np.zeros((3, 64), np.float32))
    with pytest.raises(ValueError, match=r"q must be shape \(4, 64\)"):
        e.compute(np.zeros((4, 63), np.float32))
    rng = np.random.default_rng(0)
    cpu = CpuHeads(orc, 4, 64, 4, 2, 256, 42, 0.95, 512)
    for t in range(20):
        k, v = make_kv(rng, 1, 4, 64)
        e.append(k[0], v[0])
        cpu.append_many(k, v)
    assert e.pos == 20 and e.kv_bytes == 20 * 4 * (32 + 16)
    q = rng.standard_normal((4, 64)).astype(np.float32)
    out = e.compute(q)
    assert out.dtype == np.float32 and out.shape == (4, 64)
    assert_close(out, cpu.compute(q), "Engine defaults (hybrid window)")
    e.reset()
    assert e.pos == 0 and e.kv_bytes == 0 and (e.compute(q) == 0).all()
    # memory ordering of the bit widths (upstream tests/test_la_policy.py:77-120)
    def bytes_for(kb, vb):
        x = Engine(dim=64, heads=2, k_bits=kb, v_bits=vb, capacity=64)
        x.append(q[:2], q[:2])
        return x.kv_bytes
    assert bytes_for(4, 2) < bytes_for(4, 4) and bytes_for(3, 2) < bytes_for(4, 2) < bytes_for(16, 2)


def test_torch_adapter(gpu_lib):
    import torch
    from adaptq_b200 import AdaptQAttention
    m = AdaptQAttention(dim=64, heads=4, k_bits=4, v_bits=2, capacity=128)
    with pytest.raises(ValueError, match="expects 3D tensors"):
        m(torch.zeros(4, 64), torch.zeros(4, 64), torch.zeros(4, 64))
    with pytest.raises(ValueError, match="does not support batch_size > 1"):
        m(torch.zeros(2, 4, 64), torch.zeros(2, 4, 64), torch.zeros(2, 4, 64))
    with pytest.raises(ValueError, match=r"Expected q shape \(1, 4, 64\)"):
        m(torch.zeros(1, 3, 64), torch.zeros(1, 3, 64), torch.zeros(1, 3, 64))
    x = torch.randn(1, 4, 64, dtype=torch.float16, device="cuda")
    y = m(x, x, x)
    assert y.shape == (1, 4, 64) and y.dtype == torch.float16 and y.is_cuda
    # one token attends to itself: softmax weight 1 -> output is (hybrid, exact) v
    assert torch.allclose(y.float(), x.float(), atol=2e-3)
    yc = m(x.cpu().float(), x.cpu().float(), x.cpu().float())
    assert not yc.is_cuda and yc.dtype == torch.float32
    m.reset_cache()
    assert m.engine.kv_bytes == 0


@pytest.mark.parametrize("hybrid_thresh,v_mass", [(512, 0.95), (0, 0.0)])
@pytest.mark.parametrize("k_bits,v_bits,min_cos", [(4, 4, 0.90), (4, 2, 0.85), (3, 2, 0.75), (16, 2, 0.85), (16, 16, 0.999)])
def test_output_quality_against_dense(gpu_lib, k_bits, v_bits, min_cos, hybrid_thresh, v_mass):
    """Mean cosine similarity of the attention output against the K16/V16 run, with
    upstream's bounds (tests/test_la_policy.py:193-232: dim 64, 4 heads, 32 tokens,
    Engine defaults).  Upstream's defaults keep those 32 tokens inside the FP32
    hybrid window; the second parametrisation switches the window off so that the
    quantised kernels themselves are held to the same bounds."""
    from adaptq_b200 import Engine
    dim, heads, seq = 64, 4, 32
    rng = np.random.default_rng(7)
    ks = rng.standard_normal((seq, heads, dim)).astype(np.float32)
    vs = rng.standard_normal((seq, heads, dim)).astype(np.float32)
    q = rng.standard_normal((heads, dim)).astype(np.float32)

    def run(kb, vb):
        e = Engine(dim=dim, heads=heads, k_bits=kb, v_bits=vb, capacity=256, seed=42, v_mass=v_mass,
                   hybrid_thresh=hybrid_thresh)
        for t in range(seq):
            e.append(ks[t], vs[t])
        return e.compute(q)

    dense, out = run(16, 16), run(k_bits, v_bits)
    sims = [float(np.dot(dense[h], out[h]) / (np.linalg.norm(dense[h]) * np.linalg.norm(out[h]))) for h in range(heads)]
    assert np.mean(sims) >= min_cos, f"K{k_bits}-V{v_bits}: mean cosine {np.mean(sims):.4f} < {min_cos}"


def test_long_run_through_the_adapter_stays_close_to_exact_attention(gpu_lib):
    """512 decode steps through AdaptQAttention against float64 softmax attention
    over the same keys and values: MSE < 5e-3 and cosine > 0.90 on the steps past
    256 (the criteria of upstream tests/test_accuracy.py:28-29, 110-123).  As
    upstream notes nowhere but implies, the default hybrid window (512) keeps this
    whole run on the FP32 path; a second run with a 64-token window exercises the
    quantised kernels (K4/V4) under the same criteria."""
    import torch
    from adaptq_b200 import AdaptQAttention
    dim, heads, steps = 128, 4, 512
    g = torch.Generator().manual_seed(0)
    q = torch.randn((steps, 1, heads, dim), generator=g)
    k = torch.randn((steps, 1, heads, dim), generator=g)
    v = torch.randn((steps, 1, heads, dim), generator=g)
    for hyb in (512, 64):
        m = AdaptQAttention(dim=dim, heads=heads, k_bits=4, v_bits=4, capacity=1024)
        if hyb != 512:
            from adaptq_b200 import Engine
            m.engine = Engine(dim=dim, heads=heads, k_bits=4, v_bits=4, capacity=1024, seed=42, v_mass=0.0, hybrid_thresh=hyb)
        mses, coss = [], []
        for t in range(steps):
            out = m(q[t].cuda(), k[t].cuda(), v[t].cuda())[0].double().cpu()
            if t >= 256:
                kk, vv = k[: t + 1, 0].double(), v[: t + 1, 0].double()         # [t+1, heads, dim]
                logits = torch.einsum("hd,thd->ht", q[t, 0].double(), kk) / dim ** 0.5
                ref = torch.einsum("ht,thd->hd", torch.softmax(logits, dim=1), vv)
                mses.append(float(((out - ref) ** 2).mean()))
                coss.append(float(torch.nn.functional.cosine_similarity(out.flatten(), ref.flatten(), dim=0)))
        assert max(mses) < 5e-3 and min(coss) > 0.90, (hyb, max(mses), min(coss))
