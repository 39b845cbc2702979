"""Engine: upstream's Python entry point (adaptq/core.py:9-83) over the CUDA library.

Same constructor keywords, attributes, shape checks and messages.  One call
moves all heads (upstream loops over heads in Python and makes one C call per
head); results are what that loop would produce.
"""
from __future__ import annotations

import numpy as np

from .mha import MHAContext


class Engine:
    def __init__(self, dim: int, heads: int, k_bits: int = 4, v_bits: int = 4, capacity: int = 4096,
                 seed: int = 42, v_mass: float = 0.95, hybrid_thresh: int = 512):
        self.dim = dim
        self.heads = heads
        self.k_bits = k_bits
        self.v_bits = v_bits
        self.capacity = capacity
        self._ctx = MHAContext(n_heads=heads, head_dim=dim, k_bits=k_bits, v_bits=v_bits, capacity=capacity,
                               seed=seed, v_mass=v_mass, hybrid_thresh=hybrid_thresh)
        self.pos = 0

    def append(self, k, v):
        """k, v: (heads, dim); numpy, or torch tensors on any device."""
        if tuple(k.shape) != (self.heads, self.dim) or tuple(v.shape) != (self.heads, self.dim):
            raise ValueError(f"k and v must be shape ({self.heads}, {self.dim})")
        self._ctx.append_all(k, v, self.pos)
        self.pos += 1

    def append_many(self, k, v):
        """k, v: (tokens, heads, dim) -- a whole prefill in one call."""
        if k.ndim != 3 or tuple(k.shape[1:]) != (self.heads, self.dim) or tuple(v.shape) != tuple(k.shape):
            raise ValueError(f"k and v must be shape (T, {self.heads}, {self.dim})")
        self._ctx.append_all(k, v, self.pos)
        self.pos += int(k.shape[0])

    def step(self, k, v, q):
        """append(k, v) followed by compute(q) as one library call (what upstream's
        AdaptQAttention.forward does per token, adaptq/torch_adapter.py:100-108)."""
        want = (self.heads, self.dim)
        if tuple(k.shape) != want or tuple(v.shape) != want:
            raise ValueError(f"k and v must be shape ({self.heads}, {self.dim})")
        if tuple(q.shape) != want:
            raise ValueError(f"q must be shape ({self.heads}, {self.dim})")
        out = self._ctx.decode_step(k, v, q, pos=self.pos)
        self.pos += 1
        return out

    def compute(self, q):
        """q: (heads, dim) -> float32 (heads, dim), numpy in / numpy out, tensor in / tensor out."""
        if tuple(q.shape) != (self.heads, self.dim):
            raise ValueError(f"q must be shape ({self.heads}, {self.dim})")
        return self._ctx.compute_all(q)

    def reset(self):
        self._ctx.reset()
        self.pos = 0

    @property
    def kv_bytes(self) -> int:
        return self._ctx.kv_bytes()
