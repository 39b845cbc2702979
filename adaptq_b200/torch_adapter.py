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
