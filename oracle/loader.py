"""ctypes bindings for the CPU checkers -- TEST INFRASTRUCTURE.

Two libraries expose the same head-level interface under different prefixes:

* ``liboracle.so``  (prefix ``orc_``): the plain-C restatement in
  ``adaptq_oracle.c``; always buildable (``make -C oracle``).
* ``_ref/libadaptq_ref.so`` (prefix ``ref_``): the upstream C++ sources
  compiled by ``build_ref.sh``; present only where that script could run (or
  where its output was carried along).

Only tests, the smoke check and the CPU-baseline leg of the benchmark import
this module.  The product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)


def _ptr(a, t):
    return a.ctypes.data_as(t)


def build_oracle() -> str:
    """Compile liboracle.so if missing or stale; return its path."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "adaptq_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-w", "-o", so, src, "-lm"])
    return so


def ref_path(fast: bool = False) -> str:
    return os.path.join(_HERE, "_ref", "libadaptq_ref_fast.so" if fast else "libadaptq_ref.so")


def ref_available(fast: bool = False) -> bool:
    return os.path.exists(ref_path(fast))


class _Lib:
    """Head-level interface shared by both libraries."""

    def __init__(self, path: str, prefix: str):
        self.lib = C.CDLL(path)
        self.prefix = prefix
        L = self.lib
        g = lambda name: getattr(L, prefix + name)
        self.head_create = g("head_create")
        self.head_create.restype = C.c_void_p
        self.head_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_float, C.c_int]
        self.head_destroy = g("head_destroy"); self.head_destroy.argtypes = [C.c_void_p]; self.head_destroy.restype = None
        self.head_append = g("head_append"); self.head_append.argtypes = [C.c_void_p, _f32p, _f32p, C.c_int]; self.head_append.restype = None
        self.head_append_many = g("head_append_many"); self.head_append_many.argtypes = [C.c_void_p, _f32p, _f32p, C.c_int, C.c_int]; self.head_append_many.restype = None
        self.head_compute = g("head_compute"); self.head_compute.argtypes = [C.c_void_p, _f32p, _f32p]; self.head_compute.restype = C.c_int
        self.head_compute_batch = g("head_compute_batch"); self.head_compute_batch.argtypes = [C.c_void_p, _f32p, C.c_int, _f32p]; self.head_compute_batch.restype = C.c_int
        self.head_reset = g("head_reset"); self.head_reset.argtypes = [C.c_void_p]; self.head_reset.restype = None
        for name, rt in [("head_k_data", _u8p), ("head_v_data", _u8p), ("head_k_scale", _f32p),
                         ("head_v_scale", _f32p), ("head_signs", _i8p)]:
            f = g(name); f.argtypes = [C.c_void_p]; f.restype = rt; setattr(self, name, f)
        for name in ["head_ring_head", "head_size", "head_padded", "head_k_row_bytes",
                     "head_v_row_bytes", "head_mirror_tokens"]:
            f = g(name); f.argtypes = [C.c_void_p]; f.restype = C.c_int; setattr(self, name, f)
        self.head_kv_bytes = g("head_kv_bytes"); self.head_kv_bytes.argtypes = [C.c_void_p]; self.head_kv_bytes.restype = C.c_size_t
        self.next_pow2 = g("next_pow2"); self.next_pow2.argtypes = [C.c_int]; self.next_pow2.restype = C.c_int
        self.gen_rademacher = g("gen_rademacher"); self.gen_rademacher.argtypes = [_i8p, C.c_int, C.c_uint64]; self.gen_rademacher.restype = None
        self.fwht_forward = g("fwht_forward"); self.fwht_forward.argtypes = [_f32p, _i8p, C.c_int]
        self.fwht_inverse = g("fwht_inverse"); self.fwht_inverse.argtypes = [_f32p, _i8p, C.c_int]
        self.quantize_fast = g("quantize_fast"); self.quantize_fast.argtypes = [C.c_float, C.c_int]; self.quantize_fast.restype = C.c_int
        self.pack_indices = g("pack_indices"); self.pack_indices.argtypes = [_u8p, C.c_int, C.c_int, _u8p]; self.pack_indices.restype = C.c_int
        self.unpack_indices = g("unpack_indices"); self.unpack_indices.argtypes = [_u8p, C.c_int, C.c_int, _u8p]; self.unpack_indices.restype = C.c_int
        self.codebook = g("codebook"); self.codebook.argtypes = [C.c_int]; self.codebook.restype = _f32p
        self.codebook_size = g("codebook_size"); self.codebook_size.argtypes = [C.c_int]; self.codebook_size.restype = C.c_int
        if prefix == "orc_":  # test hooks that only the restatement has
            self.head_compute_cut = g("head_compute_cut")
            self.head_compute_cut.argtypes = [C.c_void_p, _f32p, _f32p, C.c_int]; self.head_compute_cut.restype = C.c_int
            self.head_sparse_trace = g("head_sparse_trace")
            self.head_sparse_trace.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, C.POINTER(C.c_int), C.c_int]
            self.head_sparse_trace.restype = C.c_int
            self.head_set_sparse_block = g("head_set_sparse_block")
            self.head_set_sparse_block.argtypes = [C.c_void_p, C.c_int]; self.head_set_sparse_block.restype = None

    # -- numpy conveniences -------------------------------------------------
    def signs(self, n: int, seed: int) -> np.ndarray:
        d = np.zeros(n, dtype=np.int8)
        self.gen_rademacher(_ptr(d, _i8p), n, C.c_uint64(seed & (2**64 - 1)))
        return d

    def fwht(self, x: np.ndarray, signs: np.ndarray, inverse: bool = False) -> np.ndarray:
        y = np.ascontiguousarray(x, dtype=np.float32).copy()
        s = np.ascontiguousarray(signs, dtype=np.int8)
        (self.fwht_inverse if inverse else self.fwht_forward)(_ptr(y, _f32p), _ptr(s, _i8p), len(y))
        return y

    def pack(self, idx: np.ndarray, bits: int) -> np.ndarray:
        idx = np.ascontiguousarray(idx, dtype=np.uint8)
        out = np.zeros((len(idx) * bits + 7) // 8, dtype=np.uint8)
        rc = self.pack_indices(_ptr(idx, _u8p), len(idx), bits, _ptr(out, _u8p))
        if rc != 0:
            raise ValueError("unsupported bit width")
        return out

    def unpack(self, packed: np.ndarray, d: int, bits: int) -> np.ndarray:
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        out = np.zeros(d, dtype=np.uint8)
        rc = self.unpack_indices(_ptr(packed, _u8p), d, bits, _ptr(out, _u8p))
        if rc != 0:
            raise ValueError("unsupported bit width")
        return out

    def centroids(self, bits: int) -> np.ndarray:
        n = self.codebook_size(bits)
        p = self.codebook(bits)
        return np.array([p[i] for i in range(n)], dtype=np.float32)


class Head:
    """One attention head on the CPU checker `lib` (an `_Lib`)."""

    def __init__(self, lib: _Lib, dim, k_bits, v_bits, capacity, seed, v_mass=0.0, hybrid_thresh=0):
        self.L = lib
        self.dim = dim
        self.h = lib.head_create(dim, k_bits, v_bits, capacity, C.c_uint64(seed & (2**64 - 1)),
                                 C.c_float(v_mass), hybrid_thresh)
        if not self.h:
            raise ValueError("head_create rejected the arguments")
        self.capacity = capacity

    def close(self):
        if self.h:
            self.L.head_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def append(self, k, v, pos=0):
        k = np.ascontiguousarray(k, dtype=np.float32); v = np.ascontiguousarray(v, dtype=np.float32)
        self.L.head_append(self.h, _ptr(k, _f32p), _ptr(v, _f32p), pos)

    def append_many(self, keys, vals, pos0=0):
        keys = np.ascontiguousarray(keys, dtype=np.float32); vals = np.ascontiguousarray(vals, dtype=np.float32)
        assert keys.shape == vals.shape and keys.shape[1] == self.dim
        self.L.head_append_many(self.h, _ptr(keys, _f32p), _ptr(vals, _f32p), keys.shape[0], pos0)

    def compute(self, q):
        q = np.ascontiguousarray(q, dtype=np.float32)
        out = np.zeros(self.dim, dtype=np.float32)
        n = self.L.head_compute(self.h, _ptr(q, _f32p), _ptr(out, _f32p))
        return out, n

    def set_sparse_block(self, rows):
        """1: sparse V adds single rows from the start (the V2 stack's rule); 4: blocks of four first."""
        self.L.head_set_sparse_block(self.h, rows)

    def compute_cut(self, q, count):
        """Sparse V with exactly `count` rows of the sorted order accumulated (oracle only)."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        out = np.zeros(self.dim, dtype=np.float32)
        self.L.head_compute_cut(self.h, _ptr(q, _f32p), _ptr(out, _f32p), int(count))
        return out

    def sparse_trace(self, q):
        """(output, running mass after every step, rows accumulated after every step) of the
        natural sparse-V walk (oracle only)."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        out = np.zeros(self.dim, dtype=np.float32)
        cap = self.size + 4
        mass = np.zeros(cap, dtype=np.float32)
        count = np.zeros(cap, dtype=np.int32)
        n = self.L.head_sparse_trace(self.h, _ptr(q, _f32p), _ptr(out, _f32p), _ptr(mass, _f32p),
                                     count.ctypes.data_as(C.POINTER(C.c_int)), cap)
        return out, mass[:n].copy(), count[:n].copy()

    def compute_batch(self, qs):
        qs = np.ascontiguousarray(qs, dtype=np.float32)
        out = np.zeros_like(qs)
        n = self.L.head_compute_batch(self.h, _ptr(qs, _f32p), qs.shape[0], _ptr(out, _f32p))
        return out, n

    def reset(self):
        self.L.head_reset(self.h)

    @property
    def size(self): return self.L.head_size(self.h)
    @property
    def ring_head(self): return self.L.head_ring_head(self.h)
    @property
    def padded(self): return self.L.head_padded(self.h)
    @property
    def k_row_bytes(self): return self.L.head_k_row_bytes(self.h)
    @property
    def v_row_bytes(self): return self.L.head_v_row_bytes(self.h)
    @property
    def mirror_tokens(self): return self.L.head_mirror_tokens(self.h)
    @property
    def kv_bytes(self): return self.L.head_kv_bytes(self.h)

    def _arr(self, p, n, dt):
        if n == 0:
            return np.zeros(0, dtype=dt)
        return np.ctypeslib.as_array(p, shape=(n,)).astype(dt, copy=True)

    def k_data(self): return self._arr(self.L.head_k_data(self.h), self.capacity * self.k_row_bytes, np.uint8).reshape(self.capacity, -1)
    def v_data(self): return self._arr(self.L.head_v_data(self.h), self.capacity * self.v_row_bytes, np.uint8).reshape(self.capacity, -1)
    def k_scale(self): return self._arr(self.L.head_k_scale(self.h), self.capacity, np.float32)
    def v_scale(self): return self._arr(self.L.head_v_scale(self.h), self.capacity, np.float32)
    def signs(self): return self._arr(self.L.head_signs(self.h), self.padded, np.int8)


_cache = {}


def oracle() -> _Lib:
    if "orc" not in _cache:
        _cache["orc"] = _Lib(build_oracle(), "orc_")
    return _cache["orc"]


def reference(fast: bool = False) -> _Lib:
    key = "ref_fast" if fast else "ref"
    if key not in _cache:
        if not ref_available(fast):
            raise FileNotFoundError(ref_path(fast) + " (run oracle/build_ref.sh where the upstream sources are)")
        _cache[key] = _Lib(ref_path(fast), "ref_")
    return _cache[key]


def mha_head_seed(base_seed: int, head_idx: int) -> int:
    """Per-head seed rule of the multi-head handle (upstream core/adaptq_c_api.cpp:160)."""
    return (base_seed ^ (head_idx * 0xDEADBEEFCAFE)) & (2**64 - 1)


def time_reference_heads(n_heads, dim, k_bits, v_bits, capacity, base_seed, keys, vals, queries,
                         n_steps, n_threads, v_mass=0.0, hybrid_thresh=0, fast=True):
    """Run the upstream build's timing harness. keys/vals: [n_heads, n_tokens, dim]."""
    L = reference(fast).lib
    f = L.ref_time_heads
    f.restype = C.c_int
    f.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_float, C.c_int,
                  _f32p, _f32p, C.c_int, _f32p, C.c_int, _f32p, C.c_int,
                  C.POINTER(C.c_double), C.POINTER(C.c_double)]
    keys = np.ascontiguousarray(keys, dtype=np.float32); vals = np.ascontiguousarray(vals, dtype=np.float32)
    queries = np.ascontiguousarray(queries, dtype=np.float32)
    outs = np.zeros((n_heads, dim), dtype=np.float32)
    ta, tc = C.c_double(0), C.c_double(0)
    rc = f(n_heads, dim, k_bits, v_bits, capacity, C.c_uint64(base_seed), C.c_float(v_mass), hybrid_thresh,
           _ptr(keys, _f32p), _ptr(vals, _f32p), keys.shape[1], _ptr(queries, _f32p), n_steps,
           _ptr(outs, _f32p), n_threads, C.byref(ta), C.byref(tc))
    if rc != 0:
        raise RuntimeError("ref_time_heads failed")
    return ta.value, tc.value, outs


def ref_max_threads() -> int:
    L = reference(True).lib
    L.ref_max_threads.restype = C.c_int
    return L.ref_max_threads()


class RefV2:
    """Upstream's second stack (RuntimeContext / SessionSnapshot / IKernelBackend) as
    compiled into _ref/libadaptq_ref_v2.so by build_ref.sh."""

    PATH = os.path.join(_HERE, "_ref", "libadaptq_ref_v2.so")

    @classmethod
    def available(cls) -> bool:
        return os.path.exists(cls.PATH)

    def __init__(self):
        L = self.lib = C.CDLL(self.PATH)
        L.refv2_last_error.restype = C.c_char_p
        L.refv2_create.restype = C.c_void_p
        L.refv2_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
        L.refv2_destroy.argtypes = [C.c_void_p]
        L.refv2_append.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p, _f32p]
        L.refv2_compute.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p, _f32p]
        L.refv2_token_pos.argtypes = [C.c_void_p]
        L.refv2_snapshot_save.argtypes = [C.c_void_p, C.c_char_p]
        L.refv2_snapshot_load.argtypes = [C.c_char_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int]
        L.refv2_kernel_name.restype = C.c_char_p
        L.refv2_kernel_fwht.argtypes = [_f32p, _i8p, C.c_int, C.c_int]
        L.refv2_kernel_kdot_batch.argtypes = [_f32p, _u8p, C.c_size_t, _f32p, C.c_int, C.c_int, C.c_int, _f32p]
        L.refv2_kernel_vaccum_batch.argtypes = [_f32p, _u8p, C.c_size_t, _f32p, _f32p, C.c_int, C.c_int, C.c_int]

    def error(self) -> str:
        return self.lib.refv2_last_error().decode()

    class Runtime:
        def __init__(self, owner, n_layers, n_heads, dim, bits, capacity, v_mass=0.0):
            self.o, self.dim = owner, dim
            self.h = owner.lib.refv2_create(n_layers, n_heads, dim, bits, capacity, C.c_float(v_mass))
            if not self.h:
                raise RuntimeError(owner.error())

        def append(self, layer, head, k, v):
            k = np.ascontiguousarray(k, dtype=np.float32); v = np.ascontiguousarray(v, dtype=np.float32)
            if self.o.lib.refv2_append(self.h, layer, head, _ptr(k, _f32p), _ptr(v, _f32p)) != 0:
                raise RuntimeError(self.o.error())

        def compute(self, layer, head, q):
            q = np.ascontiguousarray(q, dtype=np.float32)
            out = np.zeros(self.dim, dtype=np.float32)
            n = self.o.lib.refv2_compute(self.h, layer, head, _ptr(q, _f32p), _ptr(out, _f32p))
            if n < 0:
                raise RuntimeError(self.o.error())
            return out, n

        def token_pos(self):
            return self.o.lib.refv2_token_pos(self.h)

        def save(self, path):
            if self.o.lib.refv2_snapshot_save(self.h, str(path).encode()) != 0:
                raise RuntimeError(self.o.error())

        def close(self):
            if self.h:
                self.o.lib.refv2_destroy(self.h)
                self.h = None

        def __del__(self):
            try:
                self.close()
            except Exception:
                pass

    def runtime(self, *a, **kw):
        return RefV2.Runtime(self, *a, **kw)

    def load_snapshot(self, path, max_heads=4096):
        hdr = (C.c_int * 7)()
        sizes = (C.c_int * max_heads)()
        if self.lib.refv2_snapshot_load(str(path).encode(), hdr, sizes, max_heads) != 0:
            raise RuntimeError(self.error())
        keys = ("n_layers", "n_heads", "dim", "bits", "n_tokens", "n_head_blocks", "flags")
        d = dict(zip(keys, list(hdr)))
        d["cache_sizes"] = list(sizes)[:min(max_heads, d["n_head_blocks"])]
        return d

    def kernel_name(self):
        return self.lib.refv2_kernel_name().decode()

    def fwht(self, x, D, inverse=False):
        y = np.ascontiguousarray(x, dtype=np.float32).copy()
        D = np.ascontiguousarray(D, dtype=np.int8)
        self.lib.refv2_kernel_fwht(_ptr(y, _f32p), _ptr(D, _i8p), len(y), 1 if inverse else 0)
        return y

    def kdot_batch(self, q_rot, rows, scales, padded, bits):
        q = np.ascontiguousarray(q_rot, dtype=np.float32)
        rows = np.ascontiguousarray(rows, dtype=np.uint8); sc = np.ascontiguousarray(scales, dtype=np.float32)
        out = np.zeros(rows.shape[0], dtype=np.float32)
        self.lib.refv2_kernel_kdot_batch(_ptr(q, _f32p), _ptr(rows, _u8p), rows.strides[0], _ptr(sc, _f32p), rows.shape[0],
                                         padded, bits, _ptr(out, _f32p))
        return out

    def vaccum_batch(self, rows, scales, weights, padded, bits):
        rows = np.ascontiguousarray(rows, dtype=np.uint8); sc = np.ascontiguousarray(scales, dtype=np.float32)
        w = np.ascontiguousarray(weights, dtype=np.float32)
        acc = np.zeros(padded, dtype=np.float32)
        self.lib.refv2_kernel_vaccum_batch(_ptr(acc, _f32p), _ptr(rows, _u8p), rows.strides[0], _ptr(sc, _f32p), _ptr(w, _f32p),
                                           rows.shape[0], padded, bits)
        return acc


def v2_head_seed(layer: int, head: int) -> int:
    """Per-head seed of upstream's second stack (runtime/runtime_context.cpp:128)."""
    return layer * 65537 + head
