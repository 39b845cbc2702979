"""RuntimeContext: upstream's second stack (the "V2" plugin runtime,
runtime/runtime_context.h) with its default har_fixed strategy on contiguous
slab storage, over the CUDA library -- plus AQSS v2 session snapshots
(replay/session_snapshot.h) of the device cache and the IKernelBackend
primitives (include/adaptq/kernel.h).  Same names and argument meaning as the
C++ classes; see include/adaptq_runtime.h for what each call replaces.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .mha import _as_arg


class RuntimeContextConfig:
    """Fields of upstream's RuntimeContextConfig that the path uses (runtime_context.h:34-46)."""

    def __init__(self, n_layers=1, n_heads=1, dim=128, bits=4, capacity=4096, v_mass=0.0):
        self.n_layers, self.n_heads, self.dim, self.bits = n_layers, n_heads, dim, bits
        self.capacity, self.v_mass = capacity, v_mass


class RuntimeContext:
    def __init__(self, cfg: RuntimeContextConfig = None, _handle=None, **kw):
        self._L = _lib.load()
        self._h = None
        if _handle is None:
            cfg = cfg or RuntimeContextConfig(**kw)
            h = self._L.adaptq_runtime_create(cfg.n_layers, cfg.n_heads, cfg.dim, cfg.bits, cfg.capacity, C.c_float(cfg.v_mass))
            if not h:
                raise RuntimeError(_lib.last_error() or "adaptq_runtime_create failed")
            _handle = h
        self._h = C.c_void_p(_handle)
        info = _lib.MhaInfo()
        self._L.adaptq_mha_info(C.c_void_p(self._L.adaptq_runtime_handle(self._h)), C.byref(info))
        self._dim, self._bits, self._capacity, self._total = info.dim, info.k_bits, info.capacity, info.n_heads
        self._n_heads = cfg.n_heads if cfg is not None else None

    # -- upstream surface (runtime/runtime_context.h) ---------------------------------
    def append(self, layer, head, k_vec, v_vec):
        k = np.ascontiguousarray(k_vec, dtype=np.float32)
        v = np.ascontiguousarray(v_vec, dtype=np.float32)
        if k.shape != (self._dim,) or v.shape != (self._dim,):
            raise ValueError(f"k_vec and v_vec must be float[{self._dim}]")
        if self._L.adaptq_runtime_append(self._h, layer, head, k.ctypes.data, v.ctypes.data) != 0:
            raise IndexError(_lib.last_error()) if "out of range" in _lib.last_error() else RuntimeError(_lib.last_error())

    def compute(self, layer, head, q_vec):
        q = np.ascontiguousarray(q_vec, dtype=np.float32)
        if q.shape != (self._dim,):
            raise ValueError(f"q_vec must be float[{self._dim}]")
        out = np.empty(self._dim, dtype=np.float32)
        n = self._L.adaptq_runtime_compute(self._h, layer, head, q.ctypes.data, out.ctypes.data)
        if n < 0:
            raise IndexError(_lib.last_error()) if "out of range" in _lib.last_error() else RuntimeError(_lib.last_error())
        return out, n

    def reset(self):
        self._L.adaptq_runtime_reset(self._h)

    def token_pos(self):
        return self._L.adaptq_runtime_token_pos(self._h)

    def dim(self):
        return self._dim

    def bits(self):
        return self._bits

    # -- all (layer, head) pairs per call ----------------------------------------------
    def append_token(self, k, v):
        """k, v: [n_layers, n_heads, dim]; numpy or torch (host / CUDA)."""
        kp, kk, _ = _as_arg(k)
        vp, vk, _ = _as_arg(v)
        if int(np.prod(kk.shape)) != self._total * self._dim or tuple(vk.shape) != tuple(kk.shape):
            raise ValueError("k and v must be shape (n_layers, n_heads, dim)")
        if self._L.adaptq_runtime_append_token(self._h, kp, vp) != 0:
            raise RuntimeError(_lib.last_error())

    def compute_token(self, q):
        qp, qk, _ = _as_arg(q)
        if int(np.prod(qk.shape)) != self._total * self._dim:
            raise ValueError("q must be shape (n_layers, n_heads, dim)")
        try:
            import torch
            out = torch.empty_like(qk) if isinstance(qk, torch.Tensor) else np.empty_like(qk)
        except ImportError:  # pragma: no cover
            out = np.empty_like(qk)
        op, ok, _ = _as_arg(out)
        if self._L.adaptq_runtime_compute_token(self._h, qp, op) < 0:
            raise RuntimeError(_lib.last_error())
        return ok

    # -- SessionSnapshot (replay/session_snapshot.h) ----------------------------------------
    def save_snapshot(self, path: str):
        if self._L.adaptq_runtime_snapshot_save(self._h, str(path).encode()) != 0:
            raise RuntimeError(_lib.last_error())

    @classmethod
    def load_snapshot(cls, path: str, capacity: int = 0, v_mass: float = 0.0):
        L = _lib.load()
        h = L.adaptq_runtime_snapshot_load(str(path).encode(), capacity, C.c_float(v_mass))
        if not h:
            raise RuntimeError(_lib.last_error())
        return cls(_handle=h)

    def export_head(self, layer, head, n_heads):
        """Host copy of one head's device cache (rows, scales, ring state)."""
        from .mha import MHAContext
        view = MHAContext.__new__(MHAContext)
        view._L, view._h = self._L, C.c_void_p(self._L.adaptq_runtime_handle(self._h))
        view.info = _lib.MhaInfo()
        self._L.adaptq_mha_info(view._h, C.byref(view.info))
        try:
            return MHAContext.export_head(view, layer * n_heads + head)
        finally:
            view._h = None  # the runtime owns the handle

    def close(self):
        if getattr(self, "_h", None):
            self._L.adaptq_runtime_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KernelBackend:
    """adaptq::IKernelBackend (include/adaptq/kernel.h:24-94) on the device.  Compressed
    vectors are given as a [n, row_stride] uint8 array plus a scale array."""

    def __init__(self):
        self._L = _lib.load()

    def name(self):
        return self._L.adaptq_kernel_backend_name().decode()

    def is_available(self):
        try:
            import torch
            return bool(torch.cuda.is_available())
        except ImportError:  # pragma: no cover
            return False

    def _fwht(self, fn, x, D):
        x = np.ascontiguousarray(x, dtype=np.float32).copy()
        D = np.ascontiguousarray(D, dtype=np.int8)
        nvec = 1 if x.ndim == 1 else x.shape[0]
        if fn(x.ctypes.data, D.ctypes.data, x.shape[-1], nvec) != 0:
            raise RuntimeError(_lib.last_error())
        return x

    def fwht_forward(self, x, D):
        return self._fwht(self._L.adaptq_kernel_fwht_forward, x, D)

    def fwht_inverse(self, x, D):
        return self._fwht(self._L.adaptq_kernel_fwht_inverse, x, D)

    def kdot_batch(self, q_rot, k_rows, k_scales, padded, bits):
        q = np.ascontiguousarray(q_rot, dtype=np.float32)
        rows = np.ascontiguousarray(k_rows, dtype=np.uint8)
        sc = np.ascontiguousarray(k_scales, dtype=np.float32)
        out = np.empty(rows.shape[0], dtype=np.float32)
        if self._L.adaptq_kernel_kdot_batch(q.ctypes.data, rows.ctypes.data, rows.strides[0], sc.ctypes.data, rows.shape[0],
                                            padded, bits, out.ctypes.data) != 0:
            raise RuntimeError(_lib.last_error())
        return out

    def vaccum_batch(self, v_rows, v_scales, weights, padded, bits):
        rows = np.ascontiguousarray(v_rows, dtype=np.uint8)
        sc = np.ascontiguousarray(v_scales, dtype=np.float32)
        w = np.ascontiguousarray(weights, dtype=np.float32)
        acc = np.empty(padded, dtype=np.float32)
        if self._L.adaptq_kernel_vaccum_batch(acc.ctypes.data, rows.ctypes.data, rows.strides[0] if rows.shape[0] else 0,
                                              sc.ctypes.data, w.ctypes.data, rows.shape[0], padded, bits) != 0:
            raise RuntimeError(_lib.last_error())
        return acc
