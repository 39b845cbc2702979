"""Host-side failure paths, exercised on a healthy GPU through the library's test hook
adaptq_inject_failure (no GPU is faulted, trapped or hung): the nth device allocation,
page-locked host allocation or kernel-launch check reports failure.  Every entry point
must then return NULL / -1 with an error text, leak nothing, leave the ring state where
it was, and keep the handle usable -- upstream instead lets std::bad_alloc fly through
its C ABI (cache/ring_buffer.cpp:71-76, core/adaptq_c_api.cpp:69-72)."""
import ctypes as C

import numpy as np
import pytest

from helpers import CpuHeads, assert_cache_equal, assert_close, make_kv

pytestmark = pytest.mark.gpu

DEVICE_ALLOC, PINNED_ALLOC, LAUNCH = 1, 2, 3


@pytest.fixture()
def hook(gpu_lib):
    yield gpu_lib.adaptq_inject_failure
    for kind in (DEVICE_ALLOC, PINNED_ALLOC, LAUNCH):
        gpu_lib.adaptq_inject_failure(kind, 0)


def _free_bytes(torch):
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_every_allocation_of_a_constructor_may_fail(gpu_lib, hook):
    import torch
    L = gpu_lib
    err = lambda: L.adaptq_last_error().decode()
    warm = L.adaptq_mha_create(2, 64, 4, 2, 64, 1, C.c_float(0.95), 8)   # loads kernels, settles the allocator
    L.adaptq_mha_destroy(C.c_void_p(warm))
    free0 = _free_bytes(torch)
    n_allocs = 7                                                         # K, V, two scale arrays, signs, status, FP32 window
    for nth in range(1, n_allocs + 1):
        hook(DEVICE_ALLOC, nth)
        assert L.adaptq_mha_create(2, 64, 4, 2, 64, 1, C.c_float(0.95), 8) is None, nth
        assert "device allocation" in err() and "failed" in err()
        assert _free_bytes(torch) == free0, f"allocation {nth} failed and something leaked"
    hook(DEVICE_ALLOC, n_allocs + 1)                                     # beyond the last one: the constructor succeeds
    h = L.adaptq_mha_create(2, 64, 4, 2, 64, 1, C.c_float(0.95), 8)
    assert h
    L.adaptq_mha_destroy(C.c_void_p(h))
    hook(DEVICE_ALLOC, 0)
    for ctor in (lambda: L.adaptq_create(64, 4, 2, 64, 1, C.c_float(0.0), 0),
                 lambda: L.adaptq_stack_create(3, 2, 64, (C.c_int * 3)(16, 4, 4), (C.c_int * 3)(2, 2, 2), 32, 42, C.c_float(0.0), 0),
                 lambda: L.adaptq_runtime_create(2, 2, 64, 4, 32, C.c_float(0.0))):
        hook(DEVICE_ALLOC, 9)                                            # inside the second part of the stack
        hook(DEVICE_ALLOC, 3)
        assert ctor() is None and "failed" in err()
        hook(DEVICE_ALLOC, 0)
    assert _free_bytes(torch) == free0


def test_staging_scratch_and_launch_failures_leave_the_handle_usable(gpu_lib, orc, hook):
    import torch
    from adaptq_b200 import MHAContext, _lib
    L = gpu_lib
    heads, dim, cap = 2, 128, 20000
    rng = np.random.default_rng(1)
    k, v = make_kv(rng, 9000, heads, dim)
    ctx = MHAContext(heads, dim, 4, 2, cap, seed=5, v_mass=0.0, hybrid_thresh=0)
    cpu = CpuHeads(orc, heads, dim, 4, 2, cap, 5)
    info = _lib.MhaInfo()

    def device_bytes():
        L.adaptq_mha_info(ctx._h, C.byref(info))
        return info.device_bytes

    base = device_bytes()
    # 1. staging buffers for host inputs: device part, then the page-locked part
    hook(DEVICE_ALLOC, 1)
    with pytest.raises(RuntimeError, match="device allocation"):
        ctx.append_all(k[:100], v[:100])
    assert device_bytes() == base and ctx.export_head(0)["ring_size"] == 0
    hook(DEVICE_ALLOC, 0)
    seen = []
    for _ in range(2):                       # the device part succeeds and is kept (and accounted) for the next call
        hook(PINNED_ALLOC, 1)
        with pytest.raises(RuntimeError, match="CUDA error"):
            ctx.append_all(k[:100], v[:100])
        seen.append(device_bytes())
        assert ctx.export_head(0)["ring_size"] == 0
    assert seen[0] == seen[1] > base, "a failed page-locked allocation must not grow the handle again"
    hook(PINNED_ALLOC, 0)
    # 2. a launch check that reports failure: -1, ring state not advanced, a retry stores the same rows
    kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    hook(LAUNCH, 1)
    with pytest.raises(RuntimeError, match="CUDA error"):
        ctx.append_all(kd, vd)
    assert ctx.export_head(0)["ring_size"] == 0 and ctx.kv_bytes() == 0
    ctx.append_all(kd, vd)
    cpu.append_many(k, v)
    for h in range(heads):
        assert_cache_equal(ctx.export_head(h), cpu.heads[h], f"head {h}")
    # 3. the split-KV scratch (9000 tokens -> several spans per head)
    q = rng.standard_normal((heads, dim)).astype(np.float32)
    qd = torch.from_numpy(q).cuda()
    before = device_bytes()
    hook(DEVICE_ALLOC, 1)
    with pytest.raises(RuntimeError, match="device allocation"):
        ctx.compute_all(qd)
    assert device_bytes() == before
    hook(DEVICE_ALLOC, 0)
    hook(LAUNCH, 1)
    with pytest.raises(RuntimeError, match="CUDA error"):
        ctx.compute_all(qd)
    assert_close(ctx.compute_all(qd).cpu().numpy(), cpu.compute(q), "after the injected failures")
    # 4. one-head calls report through the error string (void functions upstream)
    hook(LAUNCH, 1)
    L.adaptq_mha_append(ctx._h, 0, k[0, 0].ctypes.data, v[0, 0].ctypes.data, 0)
    assert "CUDA error" in L.adaptq_last_error().decode()
    assert ctx.export_head(0)["ring_size"] == 9000
    ctx.synchronize()
    ctx.close()
    assert L.adaptq_inject_failure(7, 1) == -1 and L.adaptq_inject_failure(1, -1) == -1
