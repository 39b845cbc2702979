"""The second-stack surface of the CUDA library (include/adaptq_runtime.h) on the GPU:
RuntimeContext append/compute against the CPU oracle and -- where oracle/_ref holds
the upstream build -- against upstream's own RuntimeContext; AQSS v2 snapshots written
by either side read by the other (byte-identical for a full cache) and restored into a
device cache; the IKernelBackend primitives against upstream's backend and the oracle.
Outputs within 1e-5 relative / 1e-4 absolute (helpers.RTOL / ATOL), rows bit-exact."""
import ctypes as C
import struct

import numpy as np
import pytest

from helpers import assert_cache_equal, assert_close, assert_sparse_close
from oracle import loader

pytestmark = pytest.mark.gpu


def _refv2():
    return loader.RefV2() if loader.RefV2.available() else None


def _fill(rng, rt, cpu, up, L, H, D, T):
    for t in range(T):
        k = rng.standard_normal((L, H, D)).astype(np.float32)
        v = rng.standard_normal((L, H, D)).astype(np.float32)
        if t % 3 == 0:                      # one call for the whole token ...
            rt.append_token(k, v)
        else:                               # ... or upstream's per-(layer, head) calls
            for l in range(L):
                for h in range(H):
                    rt.append(l, h, k[l, h], v[l, h])
        for l in range(L):
            for h in range(H):
                cpu[(l, h)].append(k[l, h], v[l, h])
                if up is not None:
                    up.append(l, h, k[l, h], v[l, h])


@pytest.mark.parametrize("D,bits,cap,T,v_mass", [(64, 4, 48, 70, 0.0), (128, 2, 300, 300, 0.0), (128, 4, 9000, 8500, 0.0),
                                                 (64, 3, 64, 40, 0.0), (64, 4, 200, 260, 0.9), (96, 4, 32, 32, 0.0)])
def test_runtime_matches_oracle_and_upstream(gpu_lib, orc, D, bits, cap, T, v_mass):
    from adaptq_b200.runtime import RuntimeContext, RuntimeContextConfig
    L, H = 2, 3
    rng = np.random.default_rng(D + bits + T)
    rt = RuntimeContext(RuntimeContextConfig(n_layers=L, n_heads=H, dim=D, bits=bits, capacity=cap, v_mass=v_mass))
    R = _refv2()
    up = R.runtime(L, H, D, bits, cap, v_mass) if (R and T <= 400) else None   # upstream's per-call loop is slow in Python
    cpu = {}
    for l in range(L):
        for h in range(H):
            cpu[(l, h)] = loader.Head(orc, D, bits, bits, cap, loader.v2_head_seed(l, h), v_mass, 0)
            cpu[(l, h)].set_sparse_block(1)
    _fill(rng, rt, cpu, up, L, H, D, T)
    assert rt.token_pos() == T
    for (l, h), hd in cpu.items():
        assert_cache_equal(rt.export_head(l, h, H), hd, f"head {(l, h)}")
    for i in range(3):
        q = rng.standard_normal((L, H, D)).astype(np.float32)
        all_out = rt.compute_token(q)
        for (l, h), hd in cpu.items():
            got, n = rt.compute(l, h, q[l, h])
            assert n == min(T, cap)
            assert np.array_equal(got, all_out[l, h])
            if v_mass > 0:
                assert_sparse_close(got, hd, q[l, h], v_mass, f"query {i} head {(l, h)}", block=1)
            else:
                assert_close(got, hd.compute(q[l, h])[0], f"query {i} head {(l, h)}")
                if up is not None:
                    assert_close(got, up.compute(l, h, q[l, h])[0], f"query {i} head {(l, h)} against upstream's RuntimeContext")
    with pytest.raises(IndexError):
        rt.compute(L, 0, q[0, 0])
    rt.reset()
    assert rt.token_pos() == 0 and rt.compute(0, 0, q[0, 0])[1] == 0


def test_snapshots_cross_upstream(gpu_lib, orc, tmp_path):
    from adaptq_b200.runtime import RuntimeContext, RuntimeContextConfig
    R = _refv2()
    L, H, D, bits, cap = 2, 2, 64, 4, 40
    rng = np.random.default_rng(11)
    for T in (cap + 13, 25):                # a full, wrapped cache and a partly filled one
        rt = RuntimeContext(RuntimeContextConfig(n_layers=L, n_heads=H, dim=D, bits=bits, capacity=cap))
        up = R.runtime(L, H, D, bits, cap, 0.0) if R else None
        cpu = {(l, h): loader.Head(orc, D, bits, bits, cap, loader.v2_head_seed(l, h)) for l in range(L) for h in range(H)}
        _fill(rng, rt, cpu, up, L, H, D, T)
        mine = tmp_path / f"mine_{T}.aqss"
        rt.save_snapshot(mine)
        raw = mine.read_bytes()
        magic, version, nl, nh, dim, b, ntok, total, flags = struct.unpack_from("<IIiiiiiiQ", raw, 0)
        assert (magic, version, nl, nh, dim, b, ntok, total, flags) == (0x41515353, 2, L, H, D, bits, T, L * H, 2)
        if R:
            info = R.load_snapshot(mine)     # upstream's reader accepts the file
            assert info["n_tokens"] == T and info["cache_sizes"] == [min(T, cap)] * (L * H) and info["flags"] == 2
            theirs = tmp_path / f"theirs_{T}.aqss"
            up.save(theirs)
            if T >= cap:                     # full cache: the two files are the same bytes
                assert theirs.read_bytes() == raw
        # restore (from upstream's file when there is one and it holds the V rows, i.e. the cache was full)
        src = tmp_path / f"theirs_{T}.aqss" if (R and T >= cap) else mine
        back = RuntimeContext.load_snapshot(src, capacity=cap)
        assert back.token_pos() == T
        for (l, h), hd in cpu.items():
            assert_cache_equal(back.export_head(l, h, H), hd, f"restored head {(l, h)}")
        q = rng.standard_normal((L, H, D)).astype(np.float32)
        assert np.array_equal(back.compute_token(q), rt.compute_token(q))
        # the restored cache keeps evicting in the right place
        k, v = rng.standard_normal((L, H, D)).astype(np.float32), rng.standard_normal((L, H, D)).astype(np.float32)
        back.append_token(k, v)
        for (l, h), hd in cpu.items():
            hd.append(k[l, h], v[l, h])
            assert_cache_equal(back.export_head(l, h, H), hd, f"restored head {(l, h)} after one more token")
            assert_close(back.compute(l, h, q[l, h])[0], hd.compute(q[l, h])[0], f"restored head {(l, h)}")
    with pytest.raises(RuntimeError, match="more than the requested capacity"):
        RuntimeContext.load_snapshot(mine, capacity=8)


def test_import_head_is_the_inverse_of_export_head(gpu_lib, orc):
    from adaptq_b200 import MHAContext
    heads, dim, cap = 3, 128, 50
    rng = np.random.default_rng(3)
    a = MHAContext(heads, dim, 4, 2, cap, seed=42, v_mass=0.0, hybrid_thresh=0)
    b = MHAContext(heads, dim, 4, 2, cap, seed=42, v_mass=0.0, hybrid_thresh=0)
    k = rng.standard_normal((70, heads, dim)).astype(np.float32)
    v = rng.standard_normal((70, heads, dim)).astype(np.float32)
    a.append_all(k, v)
    for h in range(heads):
        e = a.export_head(h)
        rc = gpu_lib.adaptq_mha_import_head(b._h, h, e["k_rows"].ctypes.data, e["v_rows"].ctypes.data, e["k_scale"].ctypes.data,
                                            e["v_scale"].ctypes.data, cap, e["ring_head"], e["ring_size"])
        assert rc == 0, gpu_lib.adaptq_last_error().decode()
    q = rng.standard_normal((heads, dim)).astype(np.float32)
    assert np.array_equal(a.compute_all(q), b.compute_all(q))
    assert gpu_lib.adaptq_mha_import_head(b._h, 9, None, None, None, None, 0, 0, 0) == -1
    assert gpu_lib.adaptq_last_error().decode() == "adaptq_mha_import_head: head_idx out of range"


@pytest.mark.parametrize("padded,bits,n", [(64, 4, 100), (128, 2, 1000), (128, 3, 37), (256, 4, 5), (64, 2, 1)])
def test_kernel_backend_primitives(gpu_lib, orc, padded, bits, n):
    from adaptq_b200.runtime import KernelBackend
    kb = KernelBackend()
    assert kb.name() == "cuda_sm100a" and kb.is_available()
    R = _refv2()
    rng = np.random.default_rng(padded + bits + n)
    D = orc.signs(padded, 77)
    x = rng.standard_normal((3, padded)).astype(np.float32)
    fwd, inv = kb.fwht_forward(x, D), kb.fwht_inverse(x, D)
    for i in range(3):
        assert_close(fwd[i], orc.fwht(x[i], D), "fwht_forward", atol=1e-5)
        assert_close(inv[i], orc.fwht(x[i], D, inverse=True), "fwht_inverse", atol=1e-5)
        if R:
            assert_close(fwd[i], R.fwht(x[i], D), "fwht_forward against upstream's backend", atol=1e-5)
    assert_close(kb.fwht_inverse(fwd, D), x, "inverse(forward(x))", atol=1e-5)
    # rows at a stride larger than the packed row, as in upstream's slab (slot_bytes = max(packed, dim*4))
    rb = (padded * bits + 7) // 8
    slab = np.zeros((n, padded * 4), dtype=np.uint8)
    idx = rng.integers(0, 1 << bits, size=(n, padded)).astype(np.uint8)
    for i in range(n):
        slab[i, :rb] = orc.pack(idx[i], bits)
    scales = (rng.random(n).astype(np.float32) + 0.5)
    q = rng.standard_normal(padded).astype(np.float32)
    cb = orc.centroids(bits).astype(np.float64)
    want_logits = (cb[idx] @ q.astype(np.float64)) * scales / padded
    got = kb.kdot_batch(q, slab, scales, padded, bits)
    assert_close(got, want_logits.astype(np.float32), "kdot_batch", atol=1e-5)
    w = rng.random(n).astype(np.float32)
    w[::7] = 0.0
    want_acc = ((w * scales).astype(np.float64)[:, None] * cb[idx]).sum(0)
    acc = kb.vaccum_batch(slab, scales, w, padded, bits)
    assert_close(acc, want_acc.astype(np.float32), "vaccum_batch", atol=1e-4)
    if R:
        assert_close(got, R.kdot_batch(q, slab, scales, padded, bits), "kdot_batch against upstream's backend", atol=1e-5)
        assert_close(acc, R.vaccum_batch(slab, scales, w, padded, bits), "vaccum_batch against upstream's backend", atol=1e-4)
    assert gpu_lib.adaptq_kernel_kdot_batch(None, None, 0, None, 3, 64, 4, None) == -1
    assert gpu_lib.adaptq_last_error().decode() == "adaptq_kernel_kdot_batch: null q_rot"
    assert gpu_lib.adaptq_kernel_fwht_forward(x.ctypes.data, D.ctypes.data, 48, 1) == -1
