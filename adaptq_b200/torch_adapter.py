"""AdaptQAttention: upstream's nn.Module wrapper (adaptq/torch_adapter.py:20-112).

Same constructor, same (1, heads, dim) one-token-per-call contract, same error
messages.  CUDA tensors are consumed in place (no .cpu().numpy() round trip);
CPU tensors are staged by the library.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .core import Engine


class AdaptQAttention(nn.Module):
    def __init__(self, dim: int, heads: int, k_bits: int = 4, v_bits: int = 4, capacity: int = 4096, seed: int = 42):
        super().__init__()
        self.dim = dim
        self.heads = heads
        self.k_bits = k_bits
        self.v_bits = v_bits
        self.engine = Engine(dim=dim, heads=heads, k_bits=k_bits, v_bits=v_bits, capacity=capacity, seed=seed)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
            raise ValueError(
                f"AdaptQAttention.forward() expects 3D tensors (batch, heads, dim). "
                f"Got shapes q={tuple(q.shape)}, k={tuple(k.shape)}, v={tuple(v.shape)}.")
        batch_size = q.size(0)
        if batch_size != 1:
            raise ValueError(
                f"AdaptQAttention does not support batch_size > 1 (got {batch_size}). "
                "AdapTQ maintains a single KV cache per Engine instance. "
                "For multi-sequence batches, create one AdaptQAttention per sequence "
                "and process each independently.")
        if q.size(1) != self.heads or q.size(2) != self.dim:
            raise ValueError(f"Expected q shape (1, {self.heads}, {self.dim}), got {tuple(q.shape)}.")
        if k.shape != q.shape:
            raise ValueError(f"Expected k shape {tuple(q.shape)}, got {tuple(k.shape)}.")
        if v.shape != q.shape:
            raise ValueError(f"Expected v shape {tuple(q.shape)}, got {tuple(v.shape)}.")
        k32 = k.detach()[0].to(torch.float32).contiguous()
        v32 = v.detach()[0].to(torch.float32).contiguous()
        q32 = q.detach()[0].to(torch.float32).contiguous()
        out = self.engine.step(k32, v32, q32)
        return out.unsqueeze(0).to(device=q.device, dtype=q.dtype)

    def reset_cache(self) -> None:
        self.engine.reset()


class BatchedAdaptQAttention(nn.Module):
    """`batch` independent sequences behind one handle: what a Python loop over
    `batch` AdaptQAttention modules (one Engine each, same `seed`, as upstream's
    batch_size > 1 message prescribes, adaptq/torch_adapter.py:78-85) computes,
    but every step is one library call over batch*heads caches, and the tensors
    stay on the GPU.

    forward(q, k, v): k, v (batch, heads, dim); q (batch, heads*q_per_kv, dim),
    query head j reading KV head j // q_per_kv (grouped-query attention; the
    cache of a KV head comes from HBM once for its q_per_kv queries).
    prefill(k, v): (batch, tokens, heads, dim), appended in token order.
    """

    def __init__(self, dim: int, heads: int, batch: int, k_bits: int = 4, v_bits: int = 4, capacity: int = 4096,
                 seed: int = 42, q_per_kv: int = 1, v_mass: float = 0.95, hybrid_thresh: int = 512):
        super().__init__()
        from .mha import MHAContext
        if batch <= 0 or q_per_kv <= 0:
            raise ValueError("batch and q_per_kv must be positive")
        self.dim, self.heads, self.batch, self.q_per_kv = dim, heads, batch, q_per_kv
        self.k_bits, self.v_bits = k_bits, v_bits
        # head i of every sequence is seeded like head i of upstream's handle (core/adaptq_c_api.cpp:160)
        head_seeds = [(seed ^ (i * 0xDEADBEEFCAFE)) & 0xFFFFFFFFFFFFFFFF for i in range(heads)]
        self._ctx = MHAContext(batch * heads, dim, k_bits, v_bits, capacity, seeds=head_seeds * batch,
                               v_mass=v_mass, hybrid_thresh=hybrid_thresh)
        self.pos = 0

    def _flat(self, t: torch.Tensor, shape) -> torch.Tensor:
        return t.detach().to(torch.float32).contiguous().view(shape)

    def prefill(self, k: torch.Tensor, v: torch.Tensor) -> None:
        want = (self.batch, self.heads, self.dim)
        if k.dim() != 4 or (k.size(0), k.size(2), k.size(3)) != want or v.shape != k.shape:
            raise ValueError(f"Expected k and v of shape ({self.batch}, T, {self.heads}, {self.dim}), "
                             f"got {tuple(k.shape)} and {tuple(v.shape)}.")
        T = k.size(1)
        # library layout: [tokens][head-instances][dim]
        kk = k.detach().to(torch.float32).permute(1, 0, 2, 3).contiguous().view(T, self.batch * self.heads, self.dim)
        vv = v.detach().to(torch.float32).permute(1, 0, 2, 3).contiguous().view(T, self.batch * self.heads, self.dim)
        self._ctx.append_all(kk, vv, self.pos)
        self.pos += T

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        kv_shape = (self.batch, self.heads, self.dim)
        q_shape = (self.batch, self.heads * self.q_per_kv, self.dim)
        if tuple(k.shape) != kv_shape or tuple(v.shape) != kv_shape:
            raise ValueError(f"Expected k and v of shape {kv_shape}, got {tuple(k.shape)} and {tuple(v.shape)}.")
        if tuple(q.shape) != q_shape:
            raise ValueError(f"Expected q of shape {q_shape}, got {tuple(q.shape)}.")
        n = self.batch * self.heads
        k32, v32 = self._flat(k, (n, self.dim)), self._flat(v, (n, self.dim))
        if self.q_per_kv == 1:
            out = self._ctx.decode_step(k32, v32, self._flat(q, (n, self.dim)), pos=self.pos)
        else:
            self._ctx.append_all(k32, v32, self.pos)
            out = self._ctx.compute_all(self._flat(q, (n, self.q_per_kv, self.dim)))
        self.pos += 1
        if not isinstance(out, torch.Tensor):
            out = torch.from_numpy(out)
        return out.view(q_shape).to(device=q.device, dtype=q.dtype)

    def reset_cache(self) -> None:
        self._ctx.reset()
        self.pos = 0
