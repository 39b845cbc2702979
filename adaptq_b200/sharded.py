"""Multi-GPU use of the path: one process per GPU, torch.distributed for plumbing.

Two shardings, as the path offers them:

* ``shard_units``: independent head-instances (sequences x layers x heads)
  are split across ranks; nothing is exchanged.
* ``ShardedSequence``: ONE long sequence is spread over the ranks by token
  (token t lives on rank t mod G, local ring capacity = capacity / G, which
  keeps the global FIFO eviction order exact when G divides the capacity).
  Each rank runs the split-KV kernel over its shard and produces, per head
  and query, the softmax partial (max, sum, acc[padded]) in the rotated
  domain; the partials -- (2+padded)*4 bytes per head per rank -- are
  all-gathered, merged with the usual exp(m_i - m) rescale, and one inverse
  Walsh-Hadamard transform finishes the output.  Dense V only.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple


def shard_units(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) slice of `n_units` independent units for `rank`."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(n_units, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def local_token_slice(first_token: int, n_tokens: int, world: int, rank: int) -> slice:
    """Which of the tokens first_token .. first_token+n_tokens-1 live on `rank`
    (token t -> rank t mod world), as a slice into the batch."""
    start = (rank - first_token) % world
    return slice(start, n_tokens, world)


class PeerGather:
    """Gather buffers that every rank can store into directly (torch symmetric
    memory over NVLink), for ShardedSequence(..., exchange="peer"): per rank two
    buffers [world][items][partial_floats] used in turn, and `world` arrival
    counts that only ever grow.  The streaming kernel of rank r stores each
    head's combined partial into slice [r] of every rank's buffer and bumps
    that rank's count; the merge kernel waits for the counts (bounded) -- no
    collective call on the data path."""

    def __init__(self, items: int, partial_floats: int, world: int, rank: int, group=None):
        import torch
        import torch.distributed as dist
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only, no multicast binding
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        self.items, self.world, self.rank = items, world, rank
        n_buf = world * items * partial_floats
        self._t = symm.empty(2 * n_buf + 64, dtype=torch.float32, device="cuda")
        self._t.zero_()
        try:
            symm.enable_symm_mem_for_group(group.group_name)
        except Exception:
            pass  # newer torch enables every group
        hdl = symm.rendezvous(self._t, group)
        base = [int(p) for p in hdl.buffer_ptrs]
        self.buf_ptrs = [[b + 4 * par * n_buf for b in base] for par in (0, 1)]
        self.flag_ptrs = [b + 8 * n_buf for b in base]
        torch.cuda.synchronize()
        dist.barrier(group)  # every rank's counts are zero before anybody delivers
        self.step = 0


class ShardedSequence:
    """One logical KV cache of `capacity` tokens per head, spread over the ranks
    of `group` by token.  `make_context(local_capacity)` must return an object
    with append_all / compute_partial / merge_partials (adaptq_b200.MHAContext
    on a GPU; tests substitute a CPU stand-in).  `all_gather(tensor) -> stacked
    tensor [world, ...]` defaults to torch.distributed.all_gather_into_tensor."""

    def __init__(self, make_context, capacity: int, world: int, rank: int, all_gather=None, exchange: str = "nccl"):
        if capacity % world != 0:
            raise ValueError("capacity must be a multiple of the number of ranks to keep FIFO eviction exact")
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        self.world, self.rank = world, rank
        self.ctx = make_context(capacity // world)
        self.pos = 0
        self._gather = all_gather or self._dist_all_gather
        self._exchange = exchange
        self._peer = None  # PeerGather, made on the first compute (it needs the query count)

    @staticmethod
    def _dist_all_gather(t):
        import torch
        import torch.distributed as dist
        out = torch.empty((dist.get_world_size(),) + tuple(t.shape), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous())
        return out

    def append(self, keys, vals):
        """keys, vals: [n_tokens, heads, dim], the SAME on every rank (each rank keeps its tokens)."""
        n = keys.shape[0]
        sl = local_token_slice(self.pos, n, self.world, self.rank)
        k, v = keys[sl], vals[sl]
        if k.shape[0]:
            self.ctx.append_all(k.contiguous() if hasattr(k, "contiguous") else k,
                                v.contiguous() if hasattr(v, "contiguous") else v, self.pos)
        self.pos += n

    def compute(self, queries):
        """queries: [heads, dim] or [heads, nq, dim], the same on every rank -> outputs on every rank."""
        nq = 1 if len(queries.shape) == 2 else queries.shape[1]
        if self._exchange == "peer":
            if self._peer is None or self._peer.items != self.ctx.n_heads * nq:
                pf = self.ctx._L.adaptq_mha_partial_floats(self.ctx._h)
                self._peer = PeerGather(self.ctx.n_heads * nq, pf, self.world, self.rank)
            pg = self._peer
            par = pg.step & 1
            self.ctx.compute_partial_to_peers(queries, pg.buf_ptrs[par], pg.flag_ptrs, self.rank)
            pg.step += 1
            out = self.ctx.merge_from_peers(pg.buf_ptrs[par][self.rank], pg.flag_ptrs[self.rank], self.world,
                                            pg.step * pg.items, nq)
            return out[:, 0] if len(queries.shape) == 2 else out
        part = self.ctx.compute_partial(queries)     # [heads, nq, 2+padded]
        parts = self._gather(part)                   # [world, heads, nq, 2+padded]
        out = self.ctx.merge_partials(parts, nq=nq)  # [heads, nq, dim]
        return out[:, 0] if len(queries.shape) == 2 else out
