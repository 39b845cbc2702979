"""BatchedAdaptQAttention against a loop over per-sequence AdaptQAttention
modules (upstream's prescription for batch_size > 1,
adaptq/torch_adapter.py:78-85): same outputs, tensors stay on the GPU."""
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cfg", [dict(k_bits=4, v_bits=2, v_mass=0.0, hybrid_thresh=0),
                                 dict(k_bits=4, v_bits=4, v_mass=0.95, hybrid_thresh=8),
                                 dict(k_bits=16, v_bits=2, v_mass=0.0, hybrid_thresh=0)])
def test_batched_equals_loop_of_single_sequence_modules(gpu_lib, orc, cfg):
    import torch
    from adaptq_b200 import BatchedAdaptQAttention, Engine
    from helpers import CpuHeads, assert_close, assert_sparse_close
    batch, heads, dim, cap = 3, 4, 64, 24
    # CPU oracle for the first and the last sequence (every sequence is seeded alike)
    cpus = {b: CpuHeads(orc, heads, dim, cfg["k_bits"], cfg["v_bits"], cap, 42, cfg["v_mass"], cfg["hybrid_thresh"])
            for b in (0, batch - 1)}
    g = torch.Generator(device="cuda").manual_seed(2)
    bat = BatchedAdaptQAttention(dim, heads, batch, capacity=cap, seed=42, **cfg)
    singles = [Engine(dim=dim, heads=heads, capacity=cap, seed=42, **cfg) for _ in range(batch)]
    pk = torch.randn((batch, 10, heads, dim), device="cuda", generator=g)
    pv = torch.randn((batch, 10, heads, dim), device="cuda", generator=g)
    bat.prefill(pk, pv)
    for b, e in enumerate(singles):
        e.append_many(pk[b].contiguous(), pv[b].contiguous())
    for b, c in cpus.items():
        c.append_many(pk[b].cpu().numpy(), pv[b].cpu().numpy())
    for step in range(20):  # wraps the ring
        q = torch.randn((batch, heads, dim), device="cuda", generator=g)
        k = torch.randn((batch, heads, dim), device="cuda", generator=g)
        v = torch.randn((batch, heads, dim), device="cuda", generator=g)
        out = bat(q, k, v)
        assert out.shape == q.shape and out.device == q.device
        for b, e in enumerate(singles):
            want = e.step(k[b].contiguous(), v[b].contiguous(), q[b].contiguous())
            # 1e-5 relative / 1e-4 absolute; identical kernels, so in practice bit-equal
            torch.testing.assert_close(out[b], want, rtol=1e-5, atol=1e-4, msg=f"step {step} sequence {b}")
        for b, c in cpus.items():
            c.append_many(k[b].cpu().numpy()[None], v[b].cpu().numpy()[None])
            qb, ob = q[b].cpu().numpy(), out[b].cpu().numpy()
            sparse = cfg["v_mass"] > 0 and cfg["k_bits"] != 16 and c.heads[0].mirror_tokens != c.heads[0].size
            for h in range(heads):
                if sparse:
                    assert_sparse_close(ob[h], c.heads[h], qb[h], cfg["v_mass"], f"step {step} sequence {b} head {h} vs oracle")
                else:
                    assert_close(ob[h], c.heads[h].compute(qb[h])[0], f"step {step} sequence {b} head {h} vs oracle")
    bat.reset_cache()
    assert bat.pos == 0


def test_grouped_queries(gpu_lib, orc):
    import torch
    from adaptq_b200 import BatchedAdaptQAttention, MHAContext
    from helpers import CpuHeads, assert_close
    batch, heads, dim, G = 2, 3, 128, 4
    cpu = CpuHeads(orc, heads, dim, 4, 2, 64, 7)   # sequence 0 on the CPU oracle
    g = torch.Generator(device="cuda").manual_seed(3)
    bat = BatchedAdaptQAttention(dim, heads, batch, k_bits=4, v_bits=2, capacity=64, seed=7, q_per_kv=G,
                                 v_mass=0.0, hybrid_thresh=0)
    ref = [MHAContext(heads, dim, 4, 2, 64, seed=7, v_mass=0.0, hybrid_thresh=0) for _ in range(batch)]
    for step in range(12):
        q = torch.randn((batch, heads * G, dim), device="cuda", generator=g)
        k = torch.randn((batch, heads, dim), device="cuda", generator=g)
        v = torch.randn((batch, heads, dim), device="cuda", generator=g)
        out = bat(q, k, v)
        for b in range(batch):
            ref[b].append_all(k[b].contiguous(), v[b].contiguous())
            for h in range(heads):
                want = ref[b].compute_batch(h, q[b, h * G:(h + 1) * G].contiguous().cpu().numpy())
                torch.testing.assert_close(out[b, h * G:(h + 1) * G].cpu(), torch.from_numpy(want), rtol=1e-5, atol=1e-4)
        cpu.append_many(k[0].cpu().numpy()[None], v[0].cpu().numpy()[None])
        want0 = cpu.compute_batch(q[0].cpu().numpy().reshape(heads, G, dim))
        assert_close(out[0].cpu().numpy().reshape(heads, G, dim), want0, f"step {step} against the oracle")


def test_shape_errors(gpu_lib):
    import torch
    from adaptq_b200 import BatchedAdaptQAttention
    m = BatchedAdaptQAttention(64, 2, 2, capacity=8)
    x = torch.zeros((2, 2, 64), device="cuda")
    with pytest.raises(ValueError):
        m(x, x[:1], x)
    with pytest.raises(ValueError):
        m(torch.zeros((2, 4, 64), device="cuda"), x, x)
    with pytest.raises(ValueError):
        m.prefill(torch.zeros((2, 3, 2, 32), device="cuda"), torch.zeros((2, 3, 2, 32), device="cuda"))
