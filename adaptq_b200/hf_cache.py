"""Hugging Face Transformers integration: upstream's ``AdapTQCache``
(adaptq/runtime_py/backends/transformers_hf.py:56-171) over the CUDA library.

Upstream subclasses ``DynamicCache``: ``update()`` quantises the new K/V in
Python and returns the *dequantised full history* of the layer, which the
model's own attention then reads -- O(context) Python and host work per layer
per token.  Here the cache keeps the packed rows on the GPU and the attention
itself runs on the fused decode kernel, so nothing is ever dequantised:

* ``AdapTQCache`` -- same constructor keywords as upstream's class (plus
  ``k_bits`` / ``v_bits`` / ``seed``); ``update()`` hands the new tokens to the
  layer's device cache;
* ``adaptq_fused_attention`` -- an attention function for Transformers'
  ``AttentionInterface``; register it with ``register_attention()`` and load the
  model with ``attn_implementation="adaptq_fused"``.  For every new token it
  appends the token's K/V and then attends with the token's queries (grouped
  queries share their KV head's cache), i.e. exactly the per-token
  append-then-compute that upstream's ``AdaptQAttention.forward`` performs
  (adaptq/torch_adapter.py:100-108).  A prompt of S tokens is S such steps
  (causal by construction).

With any other attention implementation the cache behaves like upstream's:
``update()`` returns the dequantised history (core/quantizer.cpp:139-151), built
on the host with numpy as upstream builds it -- the compatibility path, and the
yardstick the fused path is tested against.

Limits, as upstream's: batch size 1; a plain causal mask (no padding, no sliding
window); one bit width pair for all layers unless ``layer_bits`` is given.
"""
from __future__ import annotations

import weakref

import numpy as np
import torch
from transformers import DynamicCache

from .mha import MHAContext

ATTN_NAME = "adaptq_fused"
_active = None  # weakref to the cache whose update() ran last (the attention function finds it here)

_CB = {
    2: np.array([-1.5104, -0.4528, 0.4528, 1.5104], np.float32),
    3: np.array([-2.1529, -1.3439, -0.7560, -0.2451, 0.2451, 0.7560, 1.3439, 2.1529], np.float32),
    4: np.array([-2.4008, -1.8944, -1.5105, -1.2016, -0.9138, -0.6402, -0.3795, -0.1258,
                 0.1258, 0.3795, 0.6402, 0.9138, 1.2016, 1.5105, 1.8944, 2.4008], np.float32),
}  # core/codebook.cpp:32-62


def _unpack(rows: np.ndarray, padded: int, bits: int) -> np.ndarray:
    """[n, row_bytes] packed rows -> [n, padded] indices (core/quantizer.cpp:156-194, MSB first)."""
    if bits == 4:
        return np.stack([rows >> 4, rows & 15], axis=-1).reshape(rows.shape[0], -1)[:, :padded]
    if bits == 2:
        return np.stack([rows >> 6, (rows >> 4) & 3, (rows >> 2) & 3, rows & 3], axis=-1).reshape(rows.shape[0], -1)[:, :padded]
    r = rows.reshape(rows.shape[0], -1, 3).astype(np.uint32)
    v24 = (r[..., 0] << 16) | (r[..., 1] << 8) | r[..., 2]
    return np.stack([(v24 >> (21 - 3 * k)) & 7 for k in range(8)], axis=-1).reshape(rows.shape[0], -1)[:, :padded].astype(np.uint8)


def _hadamard(p: int) -> np.ndarray:
    h = np.array([[1.0]], np.float32)
    while h.shape[0] < p:
        h = np.block([[h, h], [h, -h]])
    return h


class AdapTQCache(DynamicCache):
    def __init__(self, n_layers: int, n_heads: int, head_dim: int, n_kv_heads: int = 0, adaptq_bits: int = 4,
                 adaptq_capacity: int = 4096, dense_mode: bool = False, use_pt_cache: bool = False,
                 device="cuda", k_bits: int = None, v_bits: int = None, seed: int = 42, layer_bits=None):
        super().__init__()
        self.n_layers, self.n_heads, self.head_dim = n_layers, n_heads, head_dim
        self.n_kv_heads = n_kv_heads if n_kv_heads > 0 else n_heads
        self.adaptq_bits, self.dense_mode = adaptq_bits, dense_mode
        self.capacity = adaptq_capacity
        self._adaptq_error = ""
        self._device = torch.device(device)
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        kb, vb = k_bits or adaptq_bits, v_bits or adaptq_bits
        self._bits = list(layer_bits) if layer_bits is not None else [(kb, vb)] * n_layers
        self._ctx, self._pending, self._tokens = [], {}, [0] * n_layers
        if not dense_mode:
            with torch.cuda.device(self._device):
                for l in range(n_layers):  # one engine per layer, seeded 42 ^ layer as upstream's examples do
                    self._ctx.append(MHAContext(self.n_kv_heads, head_dim, self._bits[l][0], self._bits[l][1], adaptq_capacity,
                                                seed=seed ^ l, v_mass=0.0, hybrid_thresh=0))

    # -- DynamicCache surface -----------------------------------------------------------
    def get_seq_length(self, layer_idx: int = 0) -> int:
        if self.dense_mode:
            return super().get_seq_length(layer_idx)
        return self._tokens[layer_idx] if layer_idx < self.n_layers else 0

    def get_mask_sizes(self, query_length, layer_idx: int = 0):
        if self.dense_mode:
            return super().get_mask_sizes(query_length, layer_idx)
        past = self._tokens[layer_idx] if layer_idx < self.n_layers else 0
        return min(past, self.capacity) + int(query_length), 0

    def update(self, key_states, value_states, layer_idx: int, *args, **kwargs):
        global _active
        if self.dense_mode:
            return super().update(key_states, value_states, layer_idx, *args, **kwargs)
        if key_states.dim() != 4 or key_states.shape[0] != 1:
            self._adaptq_error = "AdapTQ currently requires batch_size=1"
            raise ValueError(self._adaptq_error)
        # [1, kv_heads, S, D] -> [S, kv_heads, D] float32 on the cache's device
        k = key_states[0].transpose(0, 1).to(device=self._device, dtype=torch.float32).contiguous()
        v = value_states[0].transpose(0, 1).to(device=self._device, dtype=torch.float32).contiguous()
        _active = weakref.ref(self)
        self._tokens[layer_idx] += k.shape[0]
        if self._fused_for(kwargs):
            # the attention function appends token by token (each query sees the tokens up to its own)
            self._pending[layer_idx] = (k, v)
            return key_states, value_states
        self._ctx[layer_idx].append_all(k, v)
        k_all, v_all = self.dequantized(layer_idx)
        to = dict(device=key_states.device, dtype=key_states.dtype)
        return (torch.from_numpy(k_all).to(**to).transpose(0, 1).unsqueeze(0),
                torch.from_numpy(v_all).to(**to).transpose(0, 1).unsqueeze(0))

    fused = True  # set False to force the dequantise-everything behaviour of upstream's class

    def _fused_for(self, kwargs) -> bool:
        return bool(self.fused)

    # -- what upstream's class also offers ---------------------------------------------------
    def adaptq_error(self) -> str:
        return self._adaptq_error

    def kv_bytes(self) -> int:
        return sum(c.kv_bytes() for c in self._ctx)

    def dequantized(self, layer_idx: int):
        """(K, V) float32 [tokens, kv_heads, head_dim], oldest token first: every cached row through
        upstream's dequantize_raw arithmetic (core/quantizer.cpp:139-151)."""
        ctx = self._ctx[layer_idx]
        info = ctx.info
        P = info.padded
        H = _hadamard(P)
        outs = []
        for side, bits in (("k", info.k_bits), ("v", info.v_bits)):
            per_head = []
            for h in range(self.n_kv_heads):
                e = ctx.export_head(h)
                n, cap, head = e["ring_size"], info.capacity, e["ring_head"]
                order = (np.arange(n) + (head - n)) % cap if n else np.arange(0)
                rows = e[f"{side}_rows"][order]
                if bits == 16:
                    per_head.append(rows.view(np.float32).reshape(n, P)[:, :self.head_dim])
                    continue
                buf = _CB[bits][_unpack(rows, P, bits)] * np.float32(1.0 / np.sqrt(np.float32(P)))
                sg = e["signs"].astype(np.float32)
                y = (buf @ H) * np.float32(1.0 / np.sqrt(np.float32(P))) * sg      # fwht_inverse, core/fwht.cpp:106-134
                per_head.append((y[:, :self.head_dim] * e[f"{side}_scale"][order][:, None]).astype(np.float32))
            outs.append(np.stack(per_head, axis=1) if per_head else np.zeros((0, self.n_kv_heads, self.head_dim), np.float32))
        return outs[0], outs[1]

    # -- used by adaptq_fused_attention ------------------------------------------------------
    def _attend(self, layer_idx: int, query: torch.Tensor, scaling: float) -> torch.Tensor:
        """query [1, n_heads, S, D] -> [1, S, n_heads, D]; consumes the layer's pending K/V."""
        k, v = self._pending.pop(layer_idx)
        S, G, D = k.shape[0], self.n_heads // self.n_kv_heads, self.head_dim
        if query.shape[0] != 1 or query.shape[1] != self.n_heads or query.shape[2] != S or query.shape[3] != D:
            raise ValueError(f"query shape {tuple(query.shape)} does not match the {S} pending tokens of layer {layer_idx}")
        q = query[0].to(device=self._device, dtype=torch.float32)
        ref = 1.0 / float(D) ** 0.5                      # the kernel's own 1/sqrt(dim) (attention/attention.cpp:535)
        if scaling is not None and abs(float(scaling) - ref) > 1e-12 * ref:
            q = q * (float(scaling) / ref)
        q = q.transpose(0, 1).reshape(S, self.n_kv_heads, G, D).contiguous()   # query head j reads KV head j // G
        ctx = self._ctx[layer_idx]
        out = torch.empty((S, self.n_kv_heads, G, D), dtype=torch.float32, device=self._device)
        for t in range(S):
            if G == 1:
                ctx.decode_step(k[t], v[t], q[t, :, 0], out=out[t, :, 0])
            else:
                ctx.append_all(k[t], v[t])
                ctx.compute_all(q[t], out=out[t])
        return out.view(1, S, self.n_heads, D)


def adaptq_fused_attention(module, query, key, value, attention_mask, scaling=None, dropout=0.0, **kwargs):
    """Attention function for transformers.AttentionInterface: fused AdapTQ decode attention over
    the packed device cache of the AdapTQCache that this forward pass is updating."""
    cache = _active() if _active is not None else None
    if cache is None or module.layer_idx not in cache._pending:
        raise RuntimeError("adaptq_fused attention needs an adaptq_b200.hf_cache.AdapTQCache as past_key_values "
                           "(use_cache=True) whose update() ran for this layer")
    out = cache._attend(module.layer_idx, query, scaling)
    return out.to(dtype=query.dtype, device=query.device), None


def register_attention() -> str:
    """Make `attn_implementation="adaptq_fused"` available; returns that name."""
    from transformers import AttentionInterface
    AttentionInterface.register(ATTN_NAME, adaptq_fused_attention)
    try:  # the mask the model builds is not used (causality is in the append order): ask for the cheapest one
        from transformers import AttentionMaskInterface
        from transformers.masking_utils import sdpa_mask
        AttentionMaskInterface.register(ATTN_NAME, sdpa_mask)
    except Exception:
        pass
    return ATTN_NAME
