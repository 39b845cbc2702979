"""adaptq_mha_decode_step: one call = append of one token per head + attention.

It must give exactly what adaptq_mha_append_batch followed by
adaptq_mha_compute_all gives (same kernels, same order per head), both on the
plain path (few heads, pageable host memory) and on the pipelined path
(>= 4096 heads, page-locked host buffers, chunks overlapped on three streams),
and leave the cache in the same state.  The small case is also checked
against the CPU oracle.
"""
import numpy as np
import pytest

from helpers import CpuHeads, assert_cache_equal, assert_close, make_kv

pytestmark = pytest.mark.gpu


def test_decode_step_small_against_oracle(gpu_lib, orc):
    import adaptq_b200
    heads, dim, cap = 6, 64, 48
    rng = np.random.default_rng(3)
    k, v = make_kv(rng, 60, heads, dim)
    q = rng.standard_normal((60, heads, dim)).astype(np.float32)
    ctx = adaptq_b200.MHAContext(heads, dim, 4, 2, cap, seed=9, v_mass=0.0, hybrid_thresh=0)
    cpu = CpuHeads(orc, heads, dim, 4, 2, cap, 9)
    for t in range(60):  # wraps the ring
        out = ctx.decode_step(k[t], v[t], q[t], pos=t)
        cpu.append_many(k[t:t + 1], v[t:t + 1])
        if t % 7 == 0 or t == 59:
            assert_close(out, cpu.compute(q[t]), f"decode_step t={t}")
    for h in (0, heads - 1):
        assert_cache_equal(ctx.export_head(h), cpu.heads[h], f"head {h}")
    ctx.close()


@pytest.mark.parametrize("dim,kb,vb,vm,heads,cap", [
    (128, 4, 2, 0.0, 5, 700),      # streaming kernel, one span
    (128, 3, 3, 0.0, 3, 9000),     # streaming kernel, two spans merged in the launch
    (64, 2, 2, 0.0, 4, 300),       # general kernel
    (64, 16, 2, 0.0, 4, 300),      # FP32 keys: two append launches in front of the attention kernel
    (64, 4, 2, 0.95, 4, 500),      # sparse V: logits formed in the sorting block
])
def test_device_decode_steps_see_the_token_just_appended(gpu_lib, orc, dim, kb, vb, vm, heads, cap):
    """Decode steps on device tensors: the attention kernel is launched so that it may start
    while the append kernel of the same step still runs (it waits inside before reading the
    cache).  Every step's output must contain the token appended in that step -- checked
    against the CPU oracle over steps that fill the ring's tail and then evict every time,
    with a query that points at the new key so that the new token carries most of the weight."""
    import torch
    import adaptq_b200
    from helpers import assert_sparse_close
    rng = np.random.default_rng(cap + kb)
    steps = 24
    k, v = make_kv(rng, cap - steps // 2 + steps, heads, dim)
    pre = cap - steps // 2
    ctx = adaptq_b200.MHAContext(heads, dim, kb, vb, cap, seed=11, v_mass=vm, hybrid_thresh=0)
    cpu = CpuHeads(orc, heads, dim, kb, vb, cap, 11, vm, 0)
    ctx.append_all(torch.from_numpy(k[:pre]).cuda(), torch.from_numpy(v[:pre]).cuda())
    cpu.append_many(k[:pre], v[:pre])
    dk, dv, dq = (torch.empty((heads, dim), device="cuda") for _ in range(3))
    do = torch.empty((heads, dim), device="cuda")
    for s in range(steps):
        t = pre + s
        q = (k[t] * 0.5 + 0.1 * rng.standard_normal((heads, dim))).astype(np.float32)
        dk.copy_(torch.from_numpy(k[t])); dv.copy_(torch.from_numpy(v[t])); dq.copy_(torch.from_numpy(q))
        ctx.decode_step(dk, dv, dq, out=do, pos=t)
        cpu.append_many(k[t:t + 1], v[t:t + 1])
        got = do.cpu().numpy()
        if vm > 0:
            for h in range(heads):
                assert_sparse_close(got[h], cpu.heads[h], q[h], vm, f"step {s} head {h}")
        else:
            assert_close(got, cpu.compute(q), f"step {s}")
    ctx.synchronize()
    ctx.close()


@pytest.mark.parametrize("bits", [(4, 2), (2, 4), (3, 4)])
def test_decode_step_pipelined_equals_two_calls(gpu_lib, orc, bits):
    import torch
    import adaptq_b200
    from oracle import loader
    heads, dim, cap = 6000 + 40, 128, 96  # not a multiple of the chunk count; enough for the small first and last chunk
    kb, vb = bits
    sample = (0, 517, heads - 1)          # these heads are also run on the CPU oracle
    cpu = {h: loader.Head(orc, dim, kb, vb, cap, loader.mha_head_seed(5, h)) for h in sample}
    g = torch.Generator(device="cuda").manual_seed(11)
    a = adaptq_b200.MHAContext(heads, dim, kb, vb, cap, seed=5, v_mass=0.0, hybrid_thresh=0)
    b = adaptq_b200.MHAContext(heads, dim, kb, vb, cap, seed=5, v_mass=0.0, hybrid_thresh=0)
    pre_k = torch.randn((cap - 2, heads, dim), device="cuda", generator=g)
    pre_v = torch.randn((cap - 2, heads, dim), device="cuda", generator=g)
    a.append_all(pre_k, pre_v)
    b.append_all(pre_k, pre_v)
    for h, hd in cpu.items():
        hd.append_many(pre_k[:, h].cpu().numpy(), pre_v[:, h].cpu().numpy())
    launches0 = gpu_lib.adaptq_kernel_launches()
    for step in range(4):  # the last two steps evict
        k = torch.randn((heads, dim), device="cuda", generator=g)
        v = torch.randn((heads, dim), device="cuda", generator=g)
        q = torch.randn((heads, dim), device="cuda", generator=g)
        hk, hv, hq = (t.cpu().pin_memory() for t in (k, v, q))
        ho = torch.empty((heads, dim)).pin_memory()
        got = a.decode_step(hk, hv, hq, out=ho, pos=cap - 2 + step)
        b.append_all(k, v)
        want = b.compute_all(q)
        assert torch.equal(got, want.cpu()), f"step {step}: pipelined decode step differs from append + compute"
        for h, hd in cpu.items():
            hd.append(k[h].cpu().numpy(), v[h].cpu().numpy())
            assert_close(got[h].numpy(), hd.compute(q[h].cpu().numpy())[0], f"step {step} head {h} against the oracle")
    assert gpu_lib.adaptq_kernel_launches() > launches0
    for h in sample:
        assert_cache_equal(a.export_head(h), cpu[h], f"head {h} against the oracle")
        ea, eb = a.export_head(h), b.export_head(h)
        for key in ("k_rows", "v_rows", "k_scale", "v_scale"):
            assert np.array_equal(ea[key], eb[key]), (h, key)
        assert (ea["ring_head"], ea["ring_size"]) == (eb["ring_head"], eb["ring_size"])
    a.close()
    b.close()


def test_decode_step_argument_errors(gpu_lib):
    import ctypes as C
    L = gpu_lib
    m = C.c_void_p(L.adaptq_mha_create(2, 64, 4, 4, 16, 1, C.c_float(0.0), 0))
    x = np.ones((2, 64), dtype=np.float32)
    assert L.adaptq_mha_decode_step(m, None, x.ctypes.data, x.ctypes.data, x.ctypes.data, 0) == -1
    assert L.adaptq_last_error().decode() == "adaptq_mha_decode_step: null keys"
    assert L.adaptq_mha_decode_step(m, x.ctypes.data, x.ctypes.data, x.ctypes.data, None, 0) == -1
    assert L.adaptq_last_error().decode() == "adaptq_mha_decode_step: null outs"
    assert L.adaptq_mha_decode_step(None, x.ctypes.data, x.ctypes.data, x.ctypes.data, x.ctypes.data, 0) == -1
    assert L.adaptq_mha_decode_step(m, x.ctypes.data, x.ctypes.data, x.ctypes.data, x.ctypes.data, 0) == 1
    L.adaptq_mha_destroy(m)
