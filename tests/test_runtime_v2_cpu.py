"""CPU-side checks for the second-stack surface (include/adaptq_runtime.h):
the oracle restates upstream's HARFixedStrategy::compute_full once it is given
that stack's seeds and its one-row-at-a-time sparse-V rule (checked against
upstream's own RuntimeContext where oracle/_ref holds it), and the snapshot
reader of the CUDA library rejects malformed AQSS files with upstream's
messages before it ever touches a device."""
import struct

import numpy as np
import pytest

from helpers import assert_close
from oracle import loader


@pytest.mark.parametrize("bits,v_mass", [(4, 0.0), (2, 0.0), (3, 0.0), (4, 0.9)])
def test_oracle_restates_upstream_second_stack(orc, bits, v_mass):
    if not loader.RefV2.available():
        pytest.skip("oracle/_ref/libadaptq_ref_v2.so not built (upstream sources not on this machine)")
    R = loader.RefV2()
    L, H, D, cap, T = 2, 2, 64, 48, 70
    rng = np.random.default_rng(bits)
    rt = R.runtime(L, H, D, bits, cap, v_mass)
    heads = {}
    for l in range(L):
        for h in range(H):
            hd = loader.Head(orc, D, bits, bits, cap, loader.v2_head_seed(l, h), v_mass, 0)
            hd.set_sparse_block(1)
            heads[(l, h)] = hd
    for t in range(T):
        for (l, h), hd in heads.items():
            k, v = rng.standard_normal(D).astype(np.float32), rng.standard_normal(D).astype(np.float32)
            rt.append(l, h, k, v)
            hd.append(k, v)
    assert rt.token_pos() == T
    for i in range(4):
        q = rng.standard_normal(D).astype(np.float32)
        for key, hd in heads.items():
            got, n = rt.compute(*key, q)
            want, n2 = hd.compute(q)
            assert n == n2 == cap
            if v_mass > 0:   # borderline cuts aside, the two walks pick the same rows
                _, mass, count = hd.sparse_trace(q)
                if min(abs(float(mass[-1]) - v_mass), abs(v_mass - float(mass[-2])) if len(mass) > 1 else 1.0) < 1e-5:
                    continue
            assert_close(got, want, f"query {i} head {key}")


def _header(magic=0x41515353, version=2, layers=1, heads=1, dim=64, bits=4, tokens=0, total=1, flags=0):
    return struct.pack("<IIiiiiiiQ", magic, version, layers, heads, dim, bits, tokens, total, flags)


@pytest.mark.parametrize("blob,msg", [
    (b"short", "file too small"),
    (_header(magic=0x12345678) + b"\0" * 32, "invalid magic"),
    (_header(version=3) + b"\0" * 32, "snapshot version 3 > current version 2"),
    (_header(bits=5) + b"\0" * 32, "invalid bits"),
    (_header(total=7) + b"\0" * 32, "inconsistent head count"),
    (_header(layers=0) + b"\0" * 32, "invalid layer/head dimensions"),
    (_header() + struct.pack("<iiii", 0, 0, 4, 256) + struct.pack("<Q", 999) + b"\0" * 64, "inconsistent storage data size"),
    (_header() + struct.pack("<iiii", 0, 3, 0, 256) + b"\0" * 64, "invalid head coordinates"),
    (_header() + struct.pack("<iiii", 0, 0, 0, 256) + struct.pack("<Q", 0) + struct.pack("<i", 5) + b"\0" * 64, "scale count does not match"),
    (_header() + struct.pack("<iiii", 0, 0, 1, 256) + struct.pack("<Q", 512) + b"\0" * 100, "storage data exceeds remaining"),
])
def test_snapshot_reader_rejects_malformed_files(tmp_path, blob, msg):
    """The same checks, in the same order, as SessionSnapshot::load (replay/session_snapshot.cpp:271-400)."""
    import ctypes as C
    import adaptq_b200
    L = adaptq_b200.load()
    p = tmp_path / "bad.aqss"
    p.write_bytes(blob)
    assert L.adaptq_runtime_snapshot_load(str(p).encode(), 0, C.c_float(0.0)) is None
    assert msg in L.adaptq_last_error().decode(), L.adaptq_last_error().decode()
    assert L.adaptq_runtime_snapshot_load(str(tmp_path / "absent.aqss").encode(), 0, C.c_float(0.0)) is None
    assert "cannot open" in L.adaptq_last_error().decode()
