"""LayerStack: the caches of all layers of a model behind one handle
(adaptq_stack_* in include/adaptq_b200.h).  Layer l is what upstream's
``Engine(dim, heads, k_bits[l], v_bits[l], capacity, seed ^ l, ...)`` holds
(adaptq/core.py:9-44; one Engine per layer with seed 42 ^ layer is how
upstream's README and benchmarks build a model), but a token moves through
every layer in ONE call instead of 2 x layers x heads calls.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .mha import MHAContext, _as_arg, _is_cuda_tensor

try:
    import torch
except Exception:  # pragma: no cover
    torch = None


class LayerStack:
    def __init__(self, n_layers: int, heads: int, dim: int, k_bits=4, v_bits=4, capacity: int = 4096, seed: int = 42,
                 v_mass: float = 0.95, hybrid_thresh: int = 512):
        """k_bits / v_bits: one int for every layer, or a list with one entry per layer
        (e.g. [16] + [4] * 23: FP32 keys in layer 0, the layer-aware policy)."""
        self._L = _lib.load()
        self._h = None
        kb = [k_bits] * n_layers if isinstance(k_bits, int) else list(k_bits)
        vb = [v_bits] * n_layers if isinstance(v_bits, int) else list(v_bits)
        if len(kb) != n_layers or len(vb) != n_layers:
            raise ValueError("k_bits and v_bits need one entry per layer")
        self.n_layers, self.heads, self.dim, self.capacity = n_layers, heads, dim, capacity
        self.k_bits, self.v_bits = kb, vb
        h = self._L.adaptq_stack_create(n_layers, heads, dim, (C.c_int * n_layers)(*kb), (C.c_int * n_layers)(*vb), capacity,
                                        C.c_uint64(int(seed) & (2**64 - 1)), C.c_float(v_mass), hybrid_thresh)
        if not h:
            raise RuntimeError(_lib.last_error() or "adaptq_stack_create failed")
        self._h = C.c_void_p(h)
        self.pos = 0
        self._stream = 0
        self._step_cache = None  # (k, v, q, out, their data pointers, the converted arguments) of the last step()

    def _adopt(self, *tensors):
        if torch is None or not any(_is_cuda_tensor(t) for t in tensors):
            return
        stream = int(torch.cuda.current_stream().cuda_stream)
        if stream != self._stream:
            self._L.adaptq_stack_set_stream(self._h, C.c_void_p(stream))
            self._stream = stream

    def _check(self, t, lead=()):
        want = tuple(lead) + (self.n_layers, self.heads, self.dim)
        if tuple(t.shape) != want:
            raise ValueError(f"expected shape {want}, got {tuple(t.shape)}")

    def append(self, k, v):
        """k, v: (layers, heads, dim) for one token or (tokens, layers, heads, dim)."""
        self._adopt(k, v)
        kp, kk, _ = _as_arg(k)
        vp, vk, _ = _as_arg(v)
        T = 1 if kk.ndim == 3 else kk.shape[0]
        self._check(kk, () if kk.ndim == 3 else (T,))
        self._check(vk, () if vk.ndim == 3 else (T,))
        if self._L.adaptq_stack_append(self._h, kp, vp, T, self.pos) != 0:
            raise RuntimeError(_lib.last_error())
        self.pos += T

    def compute(self, q, out=None):
        self._adopt(q, out)
        qp, qk, _ = _as_arg(q)
        self._check(qk)
        if out is None:
            out = torch.empty_like(qk) if (torch is not None and isinstance(qk, torch.Tensor)) else np.empty_like(qk)
        op, ok, _ = _as_arg(out)
        if self._L.adaptq_stack_compute(self._h, qp, op) < 0:
            raise RuntimeError(_lib.last_error())
        return ok

    def step(self, k, v, q, out=None):
        """append(k, v) then compute(q) for every layer, as one library call."""
        # A decode loop hands over the same four CUDA tensors (refilled in place) every token:
        # then the shape checks and pointer conversions of the previous call still hold.
        c = self._step_cache
        if (c is not None and c[0] is k and c[1] is v and c[2] is q and c[3] is out and
                (k.data_ptr(), v.data_ptr(), q.data_ptr(), out.data_ptr()) == c[4]):
            stream = torch.cuda.current_stream().cuda_stream
            if stream != self._stream:
                self._L.adaptq_stack_set_stream(self._h, C.c_void_p(int(stream)))
                self._stream = int(stream)
            if self._L.adaptq_stack_decode_step(self._h, *c[5], self.pos) < 0:
                raise RuntimeError(_lib.last_error())
            self.pos += 1
            return out
        self._adopt(k, v, q, out)
        kp, kk, _ = _as_arg(k)
        vp, vk, _ = _as_arg(v)
        qp, qk, _ = _as_arg(q)
        for t in (kk, vk, qk):
            self._check(t)
        if out is None:
            out = torch.empty_like(qk) if (torch is not None and isinstance(qk, torch.Tensor)) else np.empty_like(qk)
        op, ok, _ = _as_arg(out)
        if self._L.adaptq_stack_decode_step(self._h, kp, vp, qp, op, self.pos) < 0:
            raise RuntimeError(_lib.last_error())
        self.pos += 1
        if all(_is_cuda_tensor(t) for t in (k, v, q, out)) and kk is k and vk is v and qk is q and ok is out:
            self._step_cache = (k, v, q, out, (k.data_ptr(), v.data_ptr(), q.data_ptr(), out.data_ptr()), (kp, vp, qp, op))
        else:
            self._step_cache = None
        return ok

    def reset(self):
        self._L.adaptq_stack_reset(self._h)
        self.pos = 0

    @property
    def kv_bytes(self) -> int:
        return int(self._L.adaptq_stack_kv_bytes(self._h))

    @property
    def parts(self) -> int:
        return self._L.adaptq_stack_parts(self._h)

    def synchronize(self):
        if self._L.adaptq_stack_synchronize(self._h) != 0:
            raise RuntimeError(_lib.last_error())

    def export_head(self, layer, head):
        first = C.c_int(0)
        h = self._L.adaptq_stack_layer_handle(self._h, layer, C.byref(first))
        if not h:
            raise IndexError(_lib.last_error())
        view = MHAContext.__new__(MHAContext)
        view._L, view._h = self._L, C.c_void_p(h)
        view.info = _lib.MhaInfo()
        self._L.adaptq_mha_info(view._h, C.byref(view.info))
        try:
            return MHAContext.export_head(view, first.value + head)
        finally:
            view._h = None  # the stack owns the handle

    def close(self):
        if getattr(self, "_h", None):
            self._L.adaptq_stack_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
