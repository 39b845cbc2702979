"""The shared library loads (no GPU needed) and exports every function that
the headers under include/ declare; argument errors that need
no device behave as upstream's C API does."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = set()
    for hdr in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", hdr)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(adaptq_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


@pytest.fixture(scope="module")
def lib():
    from adaptq_b200 import build
    build.build_library()
    import adaptq_b200
    return adaptq_b200.load()


def test_every_declared_symbol_is_exported(lib):
    from adaptq_b200 import _lib
    names = declared_functions()
    assert len(names) >= 45
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes prototype"
    assert set(_lib.SYMBOLS) <= set(names)


def test_identity(lib):
    assert lib.adaptq_version().decode().endswith("-sm100a")
    f = lib.adaptq_features()
    assert f & (1 << 1) and f & (1 << 2) and f & (1 << 8) and not (f & 1)


def test_null_and_range_errors_without_a_device(lib):
    err = lambda: lib.adaptq_last_error().decode()
    assert lib.adaptq_compute(None, None, None) == -1 and err() == "adaptq_compute: null handle"
    lib.adaptq_append(None, None, None, 0)
    assert err() == "adaptq_append: null handle"
    assert lib.adaptq_compute_batch(None, None, 0, None) == -1 and err() == "adaptq_compute_batch: null handle"
    assert lib.adaptq_kv_bytes(None) == 0 and err() == "adaptq_kv_bytes: null handle"
    lib.adaptq_reset(None)
    assert err() == "adaptq_reset: null handle"
    assert lib.adaptq_mha_compute(None, 0, None, None) == -1 and err() == "adaptq_mha_compute: null handle"
    assert lib.adaptq_mha_total_kv_bytes(None) == 0 and err() == "adaptq_mha_total_kv_bytes: null handle"
    lib.adaptq_destroy(None)
    lib.adaptq_mha_destroy(None)
    for args in [(0, 4, 4, 16), (64, 5, 4, 16), (64, 4, 1, 16), (64, 4, 4, -1)]:
        assert lib.adaptq_create(*args, 1, C.c_float(0.0), 0) is None
        assert err() == "adaptq_create: invalid dimensions or capacity"
    assert lib.adaptq_create(64, 4, 4, 16, 1, C.c_float(0.0), -1) is None
    assert lib.adaptq_mha_create(0, 64, 4, 4, 16, 1, C.c_float(0.0), 0) is None
    assert err() == "adaptq_mha_create: invalid parameters"
    assert lib.adaptq_create(2000, 4, 4, 16, 1, C.c_float(0.0), 0) is None  # pads above 1024: upstream throws
    assert "1024" in err()


def test_no_silent_cpu_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    assert lib.adaptq_create(64, 4, 2, 16, 1, C.c_float(0.0), 0) is None
    assert "no usable CUDA device" in lib.adaptq_last_error().decode()
    from adaptq_b200 import Engine
    with pytest.raises(RuntimeError):
        Engine(dim=64, heads=2)
