"""MHAContext: the class upstream exposes from its pybind11 module ``adaptq_py``
(adapters/adapter_python.cpp:30-93), here over the CUDA library's C ABI, plus
the all-heads calls of include/adaptq_b200.h.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

try:  # torch is only needed for device-tensor arguments
    import torch
except Exception:  # pragma: no cover
    torch = None


def _as_arg(x, shape_check=None):
    """Return (pointer, keepalive, is_device).  Accepts numpy arrays (host) and
    torch tensors (host or CUDA); both must be float32 and contiguous."""
    if torch is not None and isinstance(x, torch.Tensor):
        if x.dtype != torch.float32 or not x.is_contiguous():
            x = x.detach().to(torch.float32).contiguous()
        return C.c_void_p(x.data_ptr()), x, x.is_cuda
    a = np.ascontiguousarray(x, dtype=np.float32)
    return C.c_void_p(a.ctypes.data), a, False


def _is_cuda_tensor(x) -> bool:
    return torch is not None and isinstance(x, torch.Tensor) and x.is_cuda


class MHAContext:
    """n_heads independent quantized KV caches on the current CUDA device.

    Same constructor keywords, methods and error behaviour as upstream's
    ``adaptq_py.MHAContext``; ``append_all`` / ``compute_all`` are additions.
    """

    def __init__(self, n_heads, head_dim, k_bits, v_bits, capacity, seed=0, v_mass=0.95,
                 hybrid_thresh=512, seeds=None):
        L = _lib.load()
        self._L = L
        self._h = None
        if seeds is not None:
            arr = (C.c_uint64 * len(seeds))(*[int(s) & (2**64 - 1) for s in seeds])
            if len(seeds) != n_heads:
                raise ValueError("len(seeds) must equal n_heads")
            h = L.adaptq_mha_create_seeded(n_heads, arr, head_dim, k_bits, v_bits, capacity,
                                           C.c_float(v_mass), hybrid_thresh)
        else:
            h = L.adaptq_mha_create(n_heads, head_dim, k_bits, v_bits, capacity,
                                    C.c_uint64(int(seed) & (2**64 - 1)), C.c_float(v_mass), hybrid_thresh)
        if not h:
            raise RuntimeError(_lib.last_error() or "adaptq_mha_create failed")
        self._h = C.c_void_p(h)
        self._n_heads = n_heads
        self._head_dim = head_dim
        info = _lib.MhaInfo()
        L.adaptq_mha_info(self._h, C.byref(info))
        self.info = info
        self._stream = 0  # the CUDA stream the library launches on (0: the legacy default stream)

    def _adopt(self, *tensors):
        """Before a call that takes CUDA tensors: they must live on the handle's
        device, and the library must launch on the stream PyTorch is currently
        using -- otherwise, under torch.cuda.stream(s), its kernels could read
        inputs that are not produced yet, the caller could read outputs that are
        not written yet, and temporaries made here could be recycled by the
        caching allocator while a kernel still reads them."""
        dev = None
        for t in tensors:
            if _is_cuda_tensor(t):
                idx = t.device.index if t.device.index is not None else torch.cuda.current_device()
                if idx != self.info.device:
                    raise ValueError(f"CUDA tensor on device {idx}, but this cache lives on device {self.info.device}")
                dev = idx
        if dev is None:
            return
        stream = int(torch.cuda.current_stream(dev).cuda_stream)
        if stream != self._stream:
            self.set_stream(stream)

    def close(self):
        if getattr(self, "_h", None):
            self._L.adaptq_mha_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- upstream surface -----------------------------------------------------
    def append(self, head, key, val, pos):
        k = np.ascontiguousarray(key, dtype=np.float32)
        v = np.ascontiguousarray(val, dtype=np.float32)
        if k.ndim != 1 or v.ndim != 1 or k.shape[0] != self._head_dim or v.shape[0] != self._head_dim:
            raise ValueError("key/val dim mismatch")
        self._L.adaptq_mha_append(self._h, head, k.ctypes.data, v.ctypes.data, pos)
        self._raise_if_error()

    def compute(self, head, query):
        q = np.ascontiguousarray(query, dtype=np.float32)
        if q.ndim != 1 or q.shape[0] != self._head_dim:
            raise ValueError("query dim mismatch")
        out = np.empty(self._head_dim, dtype=np.float32)
        n = self._L.adaptq_mha_compute(self._h, head, q.ctypes.data, out.ctypes.data)
        if n < 0:
            raise RuntimeError(_lib.last_error())
        return out

    def compute_batch(self, head, queries):
        q = np.ascontiguousarray(queries, dtype=np.float32)
        if q.ndim != 2 or q.shape[1] != self._head_dim:
            raise ValueError("queries dim mismatch")
        out = np.empty_like(q)
        n = self._L.adaptq_mha_compute_batch(self._h, head, q.ctypes.data, q.shape[0], out.ctypes.data)
        if n < 0:
            raise RuntimeError(_lib.last_error())
        return out

    def reset(self):
        self._L.adaptq_mha_reset(self._h)

    def kv_bytes(self):
        return int(self._L.adaptq_mha_total_kv_bytes(self._h))

    @property
    def n_heads(self):
        return self._n_heads

    @property
    def head_dim(self):
        return self._head_dim

    # -- all heads at once (include/adaptq_b200.h) -------------------------------
    def append_all(self, keys, vals, pos0=0):
        """keys, vals: [n_tokens, n_heads, dim] (or [n_heads, dim] for one token);
        numpy (host) or torch (host / CUDA) float32."""
        self._adopt(keys, vals)
        kp, kk, _ = _as_arg(keys)
        vp, vk, _ = _as_arg(vals)
        shape = tuple(kk.shape)
        vshape = tuple(vk.shape)
        if len(shape) == 2:
            shape = (1,) + shape
        if len(vshape) == 2:
            vshape = (1,) + vshape
        if len(shape) != 3 or shape[1] != self._n_heads or shape[2] != self._head_dim or vshape != shape:
            raise ValueError(f"keys and vals must both be shape (T, {self._n_heads}, {self._head_dim})")
        rc = self._L.adaptq_mha_append_batch(self._h, kp, vp, shape[0], pos0)
        if rc != 0:
            raise RuntimeError(_lib.last_error())

    def compute_all(self, queries, out=None):
        """queries: [n_heads, dim] or [n_heads, nq, dim].  Returns an array/tensor of
        the same shape, on the same device as `queries`."""
        self._adopt(queries, out)
        qp, qk, is_dev = _as_arg(queries)
        shape = tuple(qk.shape)
        nq = 1 if len(shape) == 2 else shape[1]
        if shape[0] != self._n_heads or shape[-1] != self._head_dim or len(shape) not in (2, 3):
            raise ValueError(f"queries must be shape ({self._n_heads}, [nq,] {self._head_dim})")
        if out is None:
            out = torch.empty_like(qk) if (torch is not None and isinstance(qk, torch.Tensor)) else np.empty_like(qk)
        op, ok, _ = _as_arg(out)
        n = self._L.adaptq_mha_compute_all(self._h, qp, nq, op)
        if n < 0:
            raise RuntimeError(_lib.last_error())
        return ok

    def decode_step(self, keys, vals, queries, out=None, pos=0):
        """One decode step for all heads: append keys/vals [n_heads, dim], then attend
        with queries [n_heads, dim].  Same result as append_all + compute_all; with
        page-locked host arrays the transfers overlap the kernels."""
        self._adopt(keys, vals, queries, out)
        kp, kk, _ = _as_arg(keys)
        vp, vk, _ = _as_arg(vals)
        qp, qk, _ = _as_arg(queries)
        want = (self._n_heads, self._head_dim)
        if tuple(kk.shape) != want or tuple(vk.shape) != want or tuple(qk.shape) != want:
            raise ValueError(f"keys, vals and queries must be shape ({self._n_heads}, {self._head_dim})")
        if out is None:
            out = torch.empty_like(qk) if (torch is not None and isinstance(qk, torch.Tensor)) else np.empty_like(qk)
        op, ok, _ = _as_arg(out)
        if self._L.adaptq_mha_decode_step(self._h, kp, vp, qp, op, pos) < 0:
            raise RuntimeError(_lib.last_error())
        return ok

    def compute_partial(self, queries, out=None):
        """Un-normalised split-KV partials [n_heads, nq, 2+padded] for sequence sharding."""
        self._adopt(queries, out)
        qp, qk, _ = _as_arg(queries)
        shape = tuple(qk.shape)
        nq = 1 if len(shape) == 2 else shape[1]
        pf = self._L.adaptq_mha_partial_floats(self._h)
        if out is None:
            if torch is not None and isinstance(qk, torch.Tensor):
                out = torch.empty((self._n_heads, nq, pf), dtype=torch.float32, device=qk.device)
            else:
                out = np.empty((self._n_heads, nq, pf), dtype=np.float32)
        op, ok, _ = _as_arg(out)
        if self._L.adaptq_mha_compute_partial(self._h, qp, nq, op) < 0:
            raise RuntimeError(_lib.last_error())
        return ok

    def compute_partial_to_peers(self, queries, peer_buf_ptrs, peer_flag_ptrs, rank):
        """Split-KV partials stored straight into every rank's gather buffer (device
        addresses as mapped in this process) -- see adaptq_mha_compute_partial_to_peers."""
        self._adopt(queries)
        qp, qk, _ = _as_arg(queries)
        shape = tuple(qk.shape)
        nq = 1 if len(shape) == 2 else shape[1]
        world = len(peer_buf_ptrs)
        bufs = (C.c_void_p * world)(*[int(p) for p in peer_buf_ptrs])
        flags = (C.c_void_p * world)(*[int(p) for p in peer_flag_ptrs])
        if self._L.adaptq_mha_compute_partial_to_peers(self._h, qp, nq, bufs, flags, world, rank) < 0:
            raise RuntimeError(_lib.last_error())

    def merge_from_peers(self, gather_buf_ptr, flags_ptr, world, expected, nq=1, out=None):
        """Wait for every rank's arrival count to reach `expected`, merge, write [n_heads, nq, dim]."""
        if out is None:
            out = torch.empty((self._n_heads, nq, self._head_dim), dtype=torch.float32,
                              device=torch.device("cuda", self.info.device))
        self._adopt(out)
        op, ok, _ = _as_arg(out)
        rc = self._L.adaptq_mha_merge_from_peers(self._h, C.c_void_p(int(gather_buf_ptr)), C.c_void_p(int(flags_ptr)), world,
                                                 C.c_uint(expected & 0xFFFFFFFF), nq, op)
        if rc < 0:
            raise RuntimeError(_lib.last_error())
        return ok

    def merge_partials(self, partials, nq=1, out=None):
        """partials: [n_parts, n_heads, nq, 2+padded] -> [n_heads, nq, dim]."""
        self._adopt(partials, out)
        pp, pk, _ = _as_arg(partials)
        n_parts = pk.shape[0]
        if out is None:
            if torch is not None and isinstance(pk, torch.Tensor):
                out = torch.empty((self._n_heads, nq, self._head_dim), dtype=torch.float32, device=pk.device)
            else:
                out = np.empty((self._n_heads, nq, self._head_dim), dtype=np.float32)
        op, ok, _ = _as_arg(out)
        if self._L.adaptq_mha_merge_partials(self._h, pp, n_parts, nq, op) < 0:
            raise RuntimeError(_lib.last_error())
        return ok

    def set_stream(self, cuda_stream_ptr):
        """Launch this handle's work on the given CUDA stream from now on (the library
        first waits for what it queued on the previous one)."""
        self._L.adaptq_mha_set_stream(self._h, C.c_void_p(cuda_stream_ptr))
        self._stream = int(cuda_stream_ptr or 0)

    def synchronize(self):
        if self._L.adaptq_mha_synchronize(self._h) != 0:
            raise RuntimeError(_lib.last_error())

    def export_head(self, head):
        """Host copy of one head's cache in upstream's layout (for parity checks)."""
        i = self.info
        k = np.zeros((i.capacity, i.k_row_bytes), dtype=np.uint8)
        v = np.zeros((i.capacity, i.v_row_bytes), dtype=np.uint8)
        ks = np.zeros(i.capacity, dtype=np.float32)
        vs = np.zeros(i.capacity, dtype=np.float32)
        sg = np.zeros(i.padded, dtype=np.int8)
        rh, rs, mt = C.c_int(0), C.c_int(0), C.c_int(0)
        rc = self._L.adaptq_mha_export_head(self._h, head, k.ctypes.data, v.ctypes.data, ks.ctypes.data,
                                            vs.ctypes.data, sg.ctypes.data, C.byref(rh), C.byref(rs), C.byref(mt))
        if rc != 0:
            raise RuntimeError(_lib.last_error())
        return {"k_rows": k, "v_rows": v, "k_scale": ks, "v_scale": vs, "signs": sg,
                "ring_head": rh.value, "ring_size": rs.value, "mirror_tokens": mt.value}

    def _raise_if_error(self):
        e = _lib.last_error()
        if e:
            raise RuntimeError(e)
