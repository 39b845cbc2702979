"""Multi-rank host logic on CPU: two gloo ranks run ShardedSequence with a CPU
stand-in for the device context (partials computed from the oracle's packed
rows), and the merged result must equal single-cache attention.  Also the
unit-sharding arithmetic."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_units_partition():
    from adaptq_b200.sharded import shard_units
    for n in (0, 1, 7, 256, 65536):
        for w in (1, 2, 3, 8):
            spans = [shard_units(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_units(10, 2, 2)


def test_local_token_slice_round_robin():
    from adaptq_b200.sharded import local_token_slice
    world = 4
    owner = {}
    pos = 0
    for batch in (1, 3, 8, 2, 5):
        for r in range(world):
            for i in range(batch)[local_token_slice(pos, batch, world, r)]:
                assert (pos + i) not in owner
                owner[pos + i] = r
        pos += batch
    assert all(owner[t] == t % world for t in range(pos))


class CpuShard:
    """Stand-in for MHAContext built on the CPU oracle: same three calls."""

    def __init__(self, heads, dim, bits, capacity, seeds):
        from oracle import loader
        self.L = loader.oracle()
        self.heads = [loader.Head(self.L, dim, bits, bits, capacity, s) for s in seeds]
        self.dim, self.bits = dim, bits
        self.P = self.heads[0].padded

    def append_all(self, k, v, pos0=0):
        for h, hd in enumerate(self.heads):
            hd.append_many(np.ascontiguousarray(k[:, h]), np.ascontiguousarray(v[:, h]))

    def compute_partial(self, q):
        P, cb = self.P, self.L.centroids(self.bits)
        out = np.zeros((len(self.heads), 1, 2 + P), dtype=np.float32)
        for h, hd in enumerate(self.heads):
            n = hd.size
            if n == 0:
                out[h, 0, 0] = -np.inf
                continue
            sg = hd.signs()
            qn = np.sqrt(np.sum(q[h].astype(np.float64) ** 2) + 1e-12)
            qr = self.L.fwht((q[h] / qn).astype(np.float32), sg) * np.float32(np.sqrt(P) * qn)
            kd, vd, ks, vs = hd.k_data()[:n], hd.v_data()[:n], hd.k_scale()[:n], hd.v_scale()[:n]
            K = np.stack([cb[self.L.unpack(r, P, self.bits)] for r in kd])
            V = np.stack([cb[self.L.unpack(r, P, self.bits)] for r in vd])
            logits = (K @ qr) * (1.0 / (np.sqrt(self.dim) * P)) * ks
            m = logits.max()
            e = np.exp(logits - m)
            out[h, 0, 0], out[h, 0, 1] = m, e.sum()
            out[h, 0, 2:] = (e * vs / np.sqrt(P)) @ V
        return out

    def merge_partials(self, parts, nq=1):
        parts = np.asarray(parts)
        H = parts.shape[1]
        out = np.zeros((H, nq, self.dim), dtype=np.float32)
        for h in range(H):
            p = parts[:, h, 0]
            live = p[:, 1] > 0
            M = p[live, 0].max()
            w = np.where(live, np.exp(p[:, 0] - M), 0.0)
            acc = (w[:, None] * p[:, 2:]).sum(0) / (w * p[:, 1]).sum()
            out[h, 0] = self.L.fwht(acc.astype(np.float32), self.heads[h].signs(), inverse=True)[: self.dim]
        return out


def _rank_main(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch
    import torch.distributed as dist
    from adaptq_b200.sharded import ShardedSequence
    from oracle import loader
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        heads, dim, cap, T, bits = 2, 64, 64, 90, 4
        seeds = [loader.mha_head_seed(11, h) for h in range(heads)]
        rng = np.random.default_rng(0)  # same stream on every rank
        k = rng.standard_normal((T, heads, dim)).astype(np.float32)
        v = rng.standard_normal((T, heads, dim)).astype(np.float32)
        qs = rng.standard_normal((heads, dim)).astype(np.float32)

        def gather(t):
            tt = torch.from_numpy(np.ascontiguousarray(t))
            out = [torch.empty_like(tt) for _ in range(world)]
            dist.all_gather(out, tt)
            return torch.stack(out).numpy()

        seq = ShardedSequence(lambda c: CpuShard(heads, dim, bits, c, seeds), cap, world, rank, all_gather=gather)
        for a, b in ((0, 1), (1, 40), (40, 90)):   # ragged batches; the last ones wrap the global ring
            seq.append(k[a:b], v[a:b])
        got = seq.compute(qs)
        whole = CpuShard(heads, dim, bits, cap, seeds)
        whole.append_all(k, v)
        want = np.stack([whole.heads[h].compute(qs[h])[0] for h in range(heads)])
        ok = bool(np.allclose(got, want, rtol=1e-5, atol=1e-4))
        local_sizes = [hd.size for hd in seq.ctx.heads]
        q.put((rank, ok, float(np.abs(got - want).max()), local_sizes))
    finally:
        dist.destroy_process_group()


def test_sequence_sharding_two_ranks_gloo():
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 2
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, err, sizes in res:
        assert ok, f"rank {rank}: max err {err}"
        assert sizes == [32, 32]   # global capacity 64 split over 2 ranks, both rings full
