"""adaptq_mha_compute_all_static: the allocation-free decode entry point.

Some users of this library are not allowed to let it allocate GPU memory while
they are serving: their own memory pool already holds all free HBM, or they
cannot accept the stall a cudaMalloc/cudaFree may cause in a decode loop.  For
them the split-KV partials go to a fixed 4 MiB array inside the library instead
of a lazily grown buffer.  This file checks, through the C ABI, that the entry
point returns the same numbers as adaptq_mha_compute_all on two calls in a row
(the array is shared and keeps old contents, so the second call runs on dirty
scratch), that it refuses what it cannot serve, and that it does not allocate.

The file name sorts last on purpose: if it fails, every other test has run.
"""
import ctypes as C

import numpy as np
import pytest

from helpers import ATOL, RTOL

pytestmark = pytest.mark.gpu


def _ctx(heads, dim, kb, vb, T, seed, torch, cpu=None):
    """A filled cache; `cpu` (CPU-checker heads) receives the same tokens."""
    from adaptq_b200 import MHAContext
    ctx = MHAContext(heads, dim, kb, vb, T, seed=seed, v_mass=0.0, hybrid_thresh=0)
    g = torch.Generator(device="cuda").manual_seed(seed)
    done = 0
    while done < T:
        t = min(4096, T - done)
        k = torch.randn((t, heads, dim), device="cuda", generator=g)
        v = torch.randn((t, heads, dim), device="cuda", generator=g)
        ctx.append_all(k, v)
        if cpu is not None:
            cpu.append_many(k.cpu().numpy(), v.cpu().numpy())
        done += t
    return ctx, g


def test_static_scratch_matches_regular_entry_point_twice(gpu_lib, orc):
    import torch
    from helpers import CpuHeads, assert_close
    from adaptq_b200 import _lib
    L = gpu_lib
    heads, dim, T = 3, 128, 20000          # 20 000 tokens -> several spans -> the scratch is really used
    cpu = CpuHeads(orc, heads, dim, 4, 2, T, 11)
    ctx, g = _ctx(heads, dim, 4, 2, T, 11, torch, cpu)
    other, _ = _ctx(2, 128, 2, 2, 9000, 12, torch)   # a second handle sharing the same static array
    for round_ in range(2):
        q = torch.randn((heads, 2, dim), device="cuda", generator=g)
        want = torch.empty_like(q)
        got = torch.full_like(q, float("nan"))
        assert L.adaptq_mha_compute_all(ctx._h, C.c_void_p(q.data_ptr()), 2, C.c_void_p(want.data_ptr())) == T
        mem_before = torch.cuda.mem_get_info()[0]
        info = _lib.MhaInfo()
        L.adaptq_mha_info(ctx._h, C.byref(info))
        bytes_before = info.device_bytes     # everything the handle has allocated, staging included
        n = L.adaptq_mha_compute_all_static(ctx._h, C.c_void_p(q.data_ptr()), 2, C.c_void_p(got.data_ptr()))
        assert n == T, L.adaptq_last_error().decode()
        torch.cuda.synchronize()
        L.adaptq_mha_info(ctx._h, C.byref(info))
        assert info.device_bytes == bytes_before, "the allocation-free entry point grew one of the handle's buffers"
        if round_ == 1:  # the address lookup of the very first call is behind us: nothing may be allocated
            assert torch.cuda.mem_get_info()[0] >= mem_before
        a, b = got.cpu().numpy(), want.cpu().numpy()
        assert np.isfinite(a).all()
        assert (np.abs(a - b) <= ATOL + RTOL * np.abs(b)).all(), f"round {round_}: max |diff| {np.abs(a - b).max()}"
        # ... and both are what the CPU oracle computes from the same tokens
        assert_close(a, cpu.compute_batch(q.cpu().numpy()), f"round {round_} against the oracle")
        # dirty the shared array through another handle before the next round
        q2 = torch.randn((2, 1, 128), device="cuda", generator=g)
        o2, w2 = torch.empty_like(q2), torch.empty_like(q2)
        assert L.adaptq_mha_compute_all_static(other._h, C.c_void_p(q2.data_ptr()), 1, C.c_void_p(o2.data_ptr())) == 9000
        assert L.adaptq_mha_compute_all(other._h, C.c_void_p(q2.data_ptr()), 1, C.c_void_p(w2.data_ptr())) == 9000
        torch.cuda.synchronize()
        assert torch.allclose(o2, w2, rtol=RTOL, atol=ATOL)


def test_static_scratch_refusals(gpu_lib):
    import torch
    from adaptq_b200 import MHAContext
    L = gpu_lib
    err = lambda: L.adaptq_last_error().decode()
    ctx, g = _ctx(2, 128, 4, 2, 600, 3, torch)
    q = torch.randn((2, 1, 128), device="cuda", generator=g)
    o = torch.empty_like(q)
    qh = np.zeros((2, 1, 128), dtype=np.float32)
    assert L.adaptq_mha_compute_all_static(ctx._h, qh.ctypes.data, 1, C.c_void_p(o.data_ptr())) == -1
    assert "device memory" in err()
    assert L.adaptq_mha_compute_all_static(None, C.c_void_p(q.data_ptr()), 1, C.c_void_p(o.data_ptr())) == -1
    assert err() == "adaptq_mha_compute_all_static: null handle"
    assert L.adaptq_mha_compute_all_static(ctx._h, C.c_void_p(q.data_ptr()), 0, C.c_void_p(o.data_ptr())) == -1
    k16 = MHAContext(2, 128, 16, 2, 64, seed=1, v_mass=0.0, hybrid_thresh=0)   # FP32 keys: not a streaming shape
    assert L.adaptq_mha_compute_all_static(k16._h, C.c_void_p(q.data_ptr()), 1, C.c_void_p(o.data_ptr())) == -1
    assert "needs 2/3/4-bit K and V" in err()
    # too many (span, head, query) partials for the fixed array: refused, not truncated
    big, _ = _ctx(8, 128, 2, 2, 70000, 5, torch)
    nq = 128
    qb = torch.randn((8, nq, 128), device="cuda", generator=g)
    ob = torch.empty_like(qb)
    assert L.adaptq_mha_compute_all_static(big._h, C.c_void_p(qb.data_ptr()), nq, C.c_void_p(ob.data_ptr())) == -1
    assert "exceed" in err() and "static scratch" in err()
    # an empty cache answers zeros
    empty = MHAContext(2, 128, 4, 2, 64, seed=1, v_mass=0.0, hybrid_thresh=0)
    o.fill_(5.0)
    assert L.adaptq_mha_compute_all_static(empty._h, C.c_void_p(q.data_ptr()), 1, C.c_void_p(o.data_ptr())) == 0
    torch.cuda.synchronize()
    assert (o == 0).all()
