"""Upstream's own consumers of the C ABI, compiled from upstream's files against
this library by oracle/build_ref_binding.sh (into the git-ignored oracle/_ref/):

* the pybind11 module ``adaptq_py`` (adapters/adapter_python.cpp +
  core/adaptq_backend_vtable.cpp, unchanged) -- what upstream's Python package
  imports (adaptq/core.py:2-3);
* the plain-C example program (adapters/adapter_standalone.c);
* the llama.cpp adapter class (adapters/adapter_llamacpp.cpp) behind a driver.

Each is run on the GPU and its numbers are compared with the CPU oracle.  Where
the upstream checkout itself is on the machine, upstream's own pytest files for
this path are run as well, through upstream's unmodified Python package.
The tests skip where oracle/_ref/ does not hold the binaries.
"""
import os
import struct
import subprocess
import sys

import numpy as np
import pytest

from helpers import CpuHeads, assert_close, assert_sparse_close, make_kv

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_OUT = os.path.join(ROOT, "oracle", "_ref")


def _adaptq_py():
    if not any(f.startswith("adaptq_py") for f in (os.listdir(REF_OUT) if os.path.isdir(REF_OUT) else [])):
        pytest.skip("oracle/_ref/adaptq_py*.so not built (oracle/build_ref_binding.sh needs the upstream checkout)")
    if REF_OUT not in sys.path:
        sys.path.insert(0, REF_OUT)
    import adaptq_py
    return adaptq_py


@pytest.mark.parametrize("kb,vb,vm,hyb", [(4, 2, 0.0, 0), (4, 2, 0.95, 512), (16, 2, 0.95, 512), (3, 4, 0.0, 0)])
def test_upstream_pybind_module_on_this_library(gpu_lib, orc, kb, vb, vm, hyb):
    aq = _adaptq_py()
    heads, dim, cap, T = 3, 64, 700, 800          # wraps; longer than the FP32 window
    rng = np.random.default_rng(7)
    k, v = make_kv(rng, T, heads, dim)
    ctx = aq.MHAContext(n_heads=heads, head_dim=dim, k_bits=kb, v_bits=vb, capacity=cap, seed=42, v_mass=vm, hybrid_thresh=hyb)
    cpu = CpuHeads(orc, heads, dim, kb, vb, cap, 42, vm, hyb)
    assert (ctx.n_heads, ctx.head_dim) == (heads, dim)
    for t in range(T):
        for h in range(heads):
            ctx.append(h, k[t, h], v[t, h], t)
    cpu.append_many(k, v)
    assert ctx.kv_bytes() == sum(h.kv_bytes for h in cpu.heads)
    sparse = vm > 0 and kb != 16
    q = rng.standard_normal((heads, 4, dim)).astype(np.float32)
    for h in range(heads):
        single = ctx.compute(h, q[h, 0])
        batch = ctx.compute_batch(h, q[h])
        assert single.shape == (dim,) and batch.shape == (4, dim) and batch.dtype == np.float32
        for i in range(4):
            if sparse:
                assert_sparse_close(batch[i], cpu.heads[h], q[h, i], vm, f"head {h} query {i}")
            else:
                assert_close(batch[i], cpu.heads[h].compute(q[h, i])[0], f"head {h} query {i}")
        assert np.array_equal(single, batch[0])
    with pytest.raises(Exception, match="dim mismatch"):
        ctx.append(0, k[0, 0, :10], v[0, 0], 0)
    ctx.reset()
    assert ctx.kv_bytes() == 0
    assert np.array_equal(ctx.compute(0, q[0, 0]), np.zeros(dim, np.float32))


def test_upstream_standalone_c_program(gpu_lib):
    exe = os.path.join(REF_OUT, "adapter_standalone")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/adapter_standalone not built")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.strip().splitlines()
    assert lines[-1] == "OK" and len(lines) == 5
    # 4 heads x 1024 tokens x (64 + 64) packed bytes at 4/4 bits, dim 128 (include/ring_buffer.h:93)
    assert all("kv_bytes=524288" in ln for ln in lines[:4])


def test_upstream_llamacpp_adapter_class(gpu_lib, orc, tmp_path):
    exe = os.path.join(REF_OUT, "llamacpp_driver")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/llamacpp_driver not built")
    H, D, bits, cap, T, NQ, hyb, vm, seed = 4, 128, 4, 1024, 600, 3, 0, 0.0, 1234
    rng = np.random.default_rng(5)
    k, v = make_kv(rng, T, H, D)
    q = rng.standard_normal((H, NQ, D)).astype(np.float32)
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(fin, "wb") as f:
        f.write(struct.pack("<7ifQ", H, D, bits, cap, T, NQ, hyb, vm, seed))
        f.write(k.tobytes()); f.write(v.tobytes()); f.write(q.tobytes())
    r = subprocess.run([exe, str(fin), str(fout)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = open(fout, "rb").read()
    single = np.frombuffer(raw, np.float32, H * D).reshape(H, D)
    batch = np.frombuffer(raw, np.float32, H * NQ * D, offset=4 * H * D).reshape(H, NQ, D)
    kv_bytes, kv_after, used = struct.unpack_from("<QQi", raw, 4 * (H * D + H * NQ * D))
    cpu = CpuHeads(orc, H, D, bits, bits, cap, seed, vm, hyb)
    cpu.append_many(k, v)
    assert_close(batch, cpu.compute_batch(q), "attention_batch")
    assert_close(single, cpu.compute(q[:, 0]), "attention")
    assert (kv_bytes, kv_after, used) == (sum(h.kv_bytes for h in cpu.heads), 0, T)
    assert "KV:" in r.stderr


UPSTREAM_TESTS = ["tests/test_la_policy.py", "tests/test_asymmetric_engine.py", "tests/test_torch_adapter.py",
                  "tests/test_accuracy.py"]


def test_upstream_pytest_files_through_upstream_python_package(gpu_lib):
    """Upstream's own test files for this path, run unmodified: they import upstream's
    `adaptq` package, which imports `adaptq_py` -- here the module built above, i.e. every
    number comes from this library.  Needs the upstream checkout on the machine."""
    _adaptq_py()
    ref = os.environ.get("ADAPTQ_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    files = [os.path.join(ref, f) for f in UPSTREAM_TESTS]
    if not all(os.path.exists(f) for f in files):
        pytest.skip("the upstream checkout is not on this machine")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([REF_OUT, ref]))
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider", *files],
                       capture_output=True, text=True, timeout=1800, env=env, cwd=ref)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
