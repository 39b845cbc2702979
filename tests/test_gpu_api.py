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
