"""One long sequence spread over 2 GPUs by token (token t on rank t mod 2): each
rank runs the split-KV kernel on its shard, the (max, sum, acc) partials are
all-gathered with NCCL and merged -- or, second case, stored by the kernels
straight into every rank's gather buffer over NVLink (torch symmetric memory)
and merged after a bounded wait on arrival counts; the result must equal
single-cache attention computed by the CPU oracle.  Needs two CUDA devices.
Ranks leave only after a final barrier, with nothing in flight."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank(rank, world, port, q, exchange):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")  # plain peer loads/stores only
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok, err = True, ""
    try:
        from adaptq_b200 import MHAContext
        from adaptq_b200.sharded import ShardedSequence
        from helpers import CpuHeads, assert_close_conditioned, exact_attention_f64, make_kv
        from oracle import loader
        heads, dim, cap, T = 4, 128, 12288, 12000
        seeds = [loader.mha_head_seed(7, h) for h in range(heads)]
        rng = np.random.default_rng(3)  # same stream on every rank
        k, v = make_kv(rng, T, heads, dim, "student3")
        qs = rng.standard_normal((heads, dim)).astype(np.float32)
        seq = ShardedSequence(lambda c: MHAContext(heads, dim, 2, 2, c, seeds=seeds, v_mass=0.0, hybrid_thresh=0),
                              cap, world, rank, exchange=exchange)
        kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
        for a, b in ((0, 1), (1, 5000), (5000, T)):
            seq.append(kd[a:b], vd[a:b])
        qd = torch.from_numpy(qs).cuda()
        got = seq.compute(qd).cpu().numpy()
        for _ in range(3):  # later steps reuse the buffers in turn and must give the same answer
            again = seq.compute(qd).cpu().numpy()
            assert np.array_equal(got, again)
        seq.ctx.synchronize()
        if rank == 0:
            cpu = CpuHeads(loader.oracle(), heads, dim, 2, 2, cap, 0, seeds=seeds)
            cpu.append_many(k, v)
            want = cpu.compute(qs)
            exact = np.stack([exact_attention_f64(loader.oracle(), cpu.heads[h], qs[h]) for h in range(heads)])
            assert_close_conditioned(got, want, exact, "sharded sequence")
    except Exception as e:  # reported through the queue; the rank still leaves in step with the other
        ok, err = False, repr(e)
    finally:
        # nothing of this rank may be in flight, and no peer may still be storing into
        # this rank's buffers, when the process goes away
        try:
            torch.cuda.synchronize()
            q.put((rank, ok, err))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["nccl", "peer"])
def test_sequence_sharded_over_two_gpus(exchange):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q, exchange)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok, err in res:
        assert ok, f"rank {rank}: {err}"
