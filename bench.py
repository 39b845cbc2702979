#!/usr/bin/env python
"""Benchmark of the AdapTQ decode hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (configuration 4 of the benchmark contract, the one the metric is quoted on):
batched decode at Llama-3-8B KV shape -- 256 independent sequences x 32 layers
x 8 KV heads = 65 536 head-instances per GPU, head dim 128, context 8192,
K 4-bit / V 2-bit, dense V, no hybrid window.  K/V are N(0,1) with 1 % of the
entries replaced by N(0,20) outliers (synthetic; no dataset is involved).

One step = one decode step of every sequence: append the new token's K and V
to every head (the ring is full, so the oldest token is evicted) and run
decode attention for one query per head.  value = sequences * steps / time
(tokens/s, all ranks).  Under torchrun every rank holds its own 256 sequences
(weak scaling, no collective on the data path).

The line also carries:
  e2e          the same step driven from pinned HOST buffers through the C ABI
               (adaptq_mha_decode_step: H2D of K, V, q and D2H of the outputs
               inside the timed region)
  roofline     streaming decode kernel: algorithmic KV bytes / measured kernel time
               against the measured HBM copy bandwidth (MEASURED_PEAKS.json)
  append       bulk-append kernel throughput (vectors/s) and its roofline
  longctx      the long-context configuration (one 131072-token sequence, 32 KV heads, K2/V2
               and K4/V4) with its KV range split over the N ranks (strong scaling): us per
               decode step, the local kernels' share, the exchange's share, one head checked
               against the CPU oracle ("sharded_check")
  parity_sample  four head-instances of the timed cache re-run on the CPU oracle outside the
               timed region: packed rows bit-exact, one step's outputs within tolerance
  cpu_baseline the upstream CPU implementation on this host's cores (bounded sample)
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SEQS, LAYERS, KV_HEADS, DIM, CONTEXT = 256, 32, 8, 128, 8192
K_BITS, V_BITS = 4, 2
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes (read + write) per algorithmic byte of the streaming decode kernel, from the ncu
# capture summarised in profiles/compute_stream_kernel_k4v2_dim128_ctx8192.md (1024 heads:
# 877.1 MB moved for 873.5 MB algorithmic); traffic grows in proportion to the heads processed.
STREAM_TRAFFIC_PER_ALG_BYTE = 1.004


# The contract is ONE JSON line on stdout.  Libraries print there too (NCCL writes its
# version banner to stdout when NCCL_DEBUG is set in the environment), so the process
# keeps a private copy of the real stdout for the JSON line and points file
# descriptor 1 at stderr for everybody else.
_REAL_STDOUT = None


def claim_stdout():
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(obj):
    data = (json.dumps(obj) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqs", type=int, default=SEQS, help="sequences per GPU (default: the contract's 256)")
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--k-bits", type=int, default=K_BITS, choices=[2, 3, 4], help="decode mode: key width (the contract's is 4)")
    ap.add_argument("--v-bits", type=int, default=V_BITS, choices=[2, 3, 4],
                    help="decode mode: value width (the contract's is 2)")
    ap.add_argument("--mode", default="decode", choices=["decode", "append", "latency", "longctx"],
                    help="append: only the bulk-append kernel benchmark; latency: per-token decode latency of the "
                         "small per-layer configurations (contract configurations 1-3); longctx: one 131072-token "
                         "sequence with its KV range split over the ranks (contract configuration 5)")
    ap.add_argument("--exchange", default="peer", choices=["nccl", "peer"],
                    help="longctx mode: combine the ranks' partials with an NCCL all-gather, or let the kernels store "
                         "them into every rank's buffer over NVLink (torch symmetric memory)")
    ap.add_argument("--general-kernel", action="store_true",
                    help="decode mode: force the general-purpose kernels (for profiling them at a streaming shape)")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-append-bench", action="store_true")
    ap.add_argument("--skip-longctx", action="store_true", help="leave the long-context measurement out of the default line")
    ap.add_argument("--skip-parity-sample", action="store_true")
    ap.add_argument("--longctx-steps", type=int, default=20)
    ap.add_argument("--cpu-sample-heads", type=int, default=0)
    return ap.parse_args()


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, an earlier measurement of the same copy on a B200)"


# --------------------------------------------------------------------------
# clocks sampled during the timed region (NVML, read-only)
# --------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def start(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t is not None:
            self._t.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# --------------------------------------------------------------------------
# CPU arm: the upstream implementation (oracle/_ref) on the host cores
# --------------------------------------------------------------------------
def cpu_arm(n_heads_sample: int, context: int, steps: int, warmup: int, seqs: int, threads: int):
    """Times the upstream CPU build on `n_heads_sample` head-instances of the same
    shape and distribution, scales linearly to the full head count (heads are
    independent).  One CPU step = what one GPU step is: append one token to every
    head of the sample (full ring, so it evicts) + one query per head.  Also times a
    single thread on a few heads.  Returns (tokens_per_s, description dict)."""
    import numpy as np
    from oracle import loader
    kind = "reference" if loader.ref_available(fast=True) else "port"
    rng = np.random.default_rng(1234)
    shape = (n_heads_sample, context, DIM)
    keys = rng.standard_normal(shape, dtype=np.float32)
    vals = rng.standard_normal(shape, dtype=np.float32)
    for a in (keys, vals):
        m = rng.random(shape) < 0.01
        a[m] = (rng.standard_normal(int(m.sum())) * 20.0).astype(np.float32)
    q = rng.standard_normal((n_heads_sample, DIM), dtype=np.float32)
    total_heads = seqs * LAYERS * KV_HEADS
    one_thread = None
    if kind == "reference":
        loader.time_reference_heads(min(n_heads_sample, threads), DIM, K_BITS, V_BITS, 64, 42,
                                    keys[:threads, :64], vals[:threads, :64], q[:threads], max(1, warmup), threads)
        t_app, t_cmp, _ = loader.time_reference_heads(n_heads_sample, DIM, K_BITS, V_BITS, context, 42, keys, vals, q,
                                                      steps, threads)
        n1 = min(4, n_heads_sample)
        _, t1, _ = loader.time_reference_heads(n1, DIM, K_BITS, V_BITS, context, 42, keys[:n1], vals[:n1], q[:n1], steps, 1)
        one_thread = seqs / ((t1 / steps) * (total_heads / n1))
    else:  # the C restatement, single thread
        threads = 1
        O = loader.oracle()
        hs = [loader.Head(O, DIM, K_BITS, V_BITS, context, loader.mha_head_seed(42, h)) for h in range(n_heads_sample)]
        t0 = time.perf_counter()
        for h, hd in enumerate(hs):
            hd.append_many(keys[h], vals[h])
        t_app = time.perf_counter() - t0
        t0 = time.perf_counter()
        for s_ in range(steps):
            for h, hd in enumerate(hs):
                hd.append(keys[h, s_ % context], vals[h, s_ % context])
                hd.compute(q[h])
        t_cmp = time.perf_counter() - t0
    step_s = (t_cmp / steps) * (total_heads / n_heads_sample)
    tok_s = seqs / step_s
    sample_mb = n_heads_sample * context * (DIM * K_BITS // 8 + DIM * V_BITS // 8 + 8) / 1e6
    desc = {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": kind,
            "sample": f"{n_heads_sample} of {total_heads} head-instances (dim {DIM}, context {context}, K{K_BITS}/V{V_BITS}, "
                      f"dense V), {steps} decode steps (append 1 token per head into the full ring + 1 query per head), "
                      f"one worker per head on {threads} threads, scaled linearly by head count; the sample's packed cache "
                      f"is {sample_mb:.0f} MB (the full one is {sample_mb * total_heads / n_heads_sample / 1e3:.1f} GB), so it "
                      f"enjoys more of the host's caches than the full job would; bulk append "
                      f"{2 * n_heads_sample * context / t_app:.3g} vectors/s on the same cores",
            "value_one_thread": one_thread,
            "append_vectors_per_s": 2 * n_heads_sample * context / t_app,
            "ms_per_step_scaled": step_s * 1e3}
    return tok_s, desc


def host_threads() -> int:
    """CPU threads this process may use.  Not omp_get_max_threads(): torchrun exports
    OMP_NUM_THREADS=1 to its children, which would make the CPU arm single-threaded at
    N > 1 only; the timing routine sets its thread count explicitly."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    n_sample = args.cpu_sample_heads or max(2 * threads, 64)
    tok_s, desc = cpu_arm(n_sample, args.context, max(1, args.steps), args.warmup, args.seqs, threads)
    line = {"impl": "reference", "metric": "decode_attn_tokens_per_s", "value": tok_s, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": desc["ms_per_step_scaled"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args), "cpu_baseline": desc,
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def workload_config(args):
    return {"workload": "batched decode, Llama-3-8B KV shape (BASELINE configs[3])", "sequences_per_gpu": args.seqs,
            "layers": LAYERS, "kv_heads": KV_HEADS, "head_dim": DIM, "context": args.context, "k_bits": K_BITS,
            "v_bits": V_BITS, "v_mass": 0.0, "hybrid_thresh": 0,
            "step": "append 1 token to every head (ring full, FIFO eviction) + decode attention, 1 query per head",
            "l2": "inputs larger than L2 (KV cache >> 126 MB per step)", "sharding": "sequences per rank, no collective"}


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def fill_cache(ctx, heads, context, torch, gen, keep_heads=()):
    """Fill every head with `context` tokens.  The inputs of the heads in `keep_heads`
    are also returned as host arrays [context, len(keep_heads), DIM] (keys, values), for
    the CPU check of the timed cache."""
    chunk = max(1, min(64, (1 << 28) // (heads * DIM)))  # <= 1 GiB per tensor
    done = 0
    kept_k, kept_v = [], []
    idx = torch.tensor(list(keep_heads), device="cuda", dtype=torch.long) if len(keep_heads) else None
    while done < context:
        t = min(chunk, context - done)
        k = torch.randn((t, heads, DIM), device="cuda", generator=gen)
        v = torch.randn((t, heads, DIM), device="cuda", generator=gen)
        for a in (k, v):
            m = torch.rand(a.shape, device="cuda", generator=gen) < 0.01
            a[m] = torch.randn(int(m.sum().item()), device="cuda", generator=gen) * 20.0
        ctx.append_all(k, v, done)
        if idx is not None:
            kept_k.append(k.index_select(1, idx).cpu())
            kept_v.append(v.index_select(1, idx).cpu())
        done += t
    ctx.synchronize()
    if idx is None:
        return None, None
    return torch.cat(kept_k).numpy(), torch.cat(kept_v).numpy()


def parity_sample(ctx, sample_heads, seeds, kept_k, kept_v, steps_k, steps_v, q_dev, out_dev, n):
    """CPU check of the cache that was just timed (outside every timed region): the sampled
    head-instances are rebuilt on the CPU oracle from the same inputs -- the fill plus every
    decode-step token appended since -- and compared with what the GPU holds: packed rows and
    scales bit for bit, the last step's attention outputs within 1e-5 relative / 1e-4 absolute."""
    import numpy as np
    from oracle import loader
    O = loader.oracle()
    rows_equal, max_err, worst_excess = True, 0.0, 0.0
    for j, h in enumerate(sample_heads):
        hd = loader.Head(O, DIM, K_BITS, V_BITS, n, seeds[h] & (2**64 - 1))
        hd.append_many(kept_k[:, j], kept_v[:, j])
        for sk, sv in zip(steps_k, steps_v):
            hd.append(sk[j], sv[j])
        e = ctx.export_head(h)
        live = slice(0, hd.size)
        rows_equal &= bool((e["k_rows"][live] == hd.k_data()[live]).all() and (e["v_rows"][live] == hd.v_data()[live]).all()
                           and (e["k_scale"][live].view(np.uint32) == hd.k_scale()[live].view(np.uint32)).all()
                           and (e["v_scale"][live].view(np.uint32) == hd.v_scale()[live].view(np.uint32)).all()
                           and e["ring_head"] == hd.ring_head and e["ring_size"] == hd.size)
        want, _ = hd.compute(q_dev[h].cpu().numpy())
        got = out_dev[h].cpu().numpy()
        err = np.abs(got.astype(np.float64) - want.astype(np.float64))
        max_err = max(max_err, float(err.max()))
        worst_excess = max(worst_excess, float((err - (1e-4 + 1e-5 * np.abs(want))).max()))
    return {"heads": len(sample_heads), "head_indices": list(sample_heads), "tokens_per_head": n, "rows_equal": rows_equal,
            "max_abs_err": max_err, "outputs_within_tolerance": worst_excess <= 0.0,
            "tolerance": "1e-5 relative + 1e-4 absolute", "checker": "oracle/adaptq_oracle.c"}


def append_bench(torch, L, peak):
    """The contract's bulk append: 32768 tokens x 8 heads x 128, K and V, bits 2/3/4."""
    import adaptq_b200
    out = {}
    T, H = 32768, 8
    k = torch.randn((T, H, DIM), device="cuda")
    v = torch.randn((T, H, DIM), device="cuda")
    for bits in (4, 3, 2):
        ctx = adaptq_b200.MHAContext(H, DIM, bits, bits, T, seed=42, v_mass=0.0, hybrid_thresh=0)
        for _ in range(3):
            ctx.append_all(k, v)
        torch.cuda.synchronize()
        reps, batches = 20, []
        for _ in range(5):  # median of five batches of 20 back-to-back calls
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                ctx.append_all(k, v)
            e1.record()
            torch.cuda.synchronize()
            batches.append(e0.elapsed_time(e1) / 1e3 / reps)
        s = sorted(batches)[len(batches) // 2]
        vecs = 2 * T * H
        bytes_per_vec = 4 * DIM + DIM * bits // 8 + 4
        out[f"k{bits}v{bits}"] = {"vectors_per_s": vecs / s, "us_per_call": s * 1e6,
                                  "achieved_gbs": vecs * bytes_per_vec / s / 1e9,
                                  "frac_of_peak": vecs * bytes_per_vec / s / 1e9 / peak,
                                  "bytes_per_vector": bytes_per_vec}
        ctx.close()
    return {"workload": f"{T} tokens x {H} heads x {DIM}, K and V ({2 * T * H} vectors per call, 268 MB read: "
                        "larger than L2)", "results": out}


def latency_bench(torch):
    """Per-token decode latency of the small configurations: one engine per layer
    (seed 42 ^ layer), per step and layer one decode-step call (append of the new
    token + attention), device tensors in place.  These shapes move 0.5-25 MB per
    step, so they are launch/latency bound; the figure of merit is us per token."""
    import numpy as np
    import adaptq_b200
    out = {}
    cfgs = [
        ("config0_engine_d64_h4_k4v2_ctx2048_dense", 1, 4, 64, 2048, 2048, [(4, 2)], 0.0, 0, "normal"),
        ("config0_engine_defaults_sparse_v", 1, 4, 64, 2048, 2048, [(4, 2)], 0.95, 512, "normal"),
        ("config1_qwen2_0.5b_24x14_d64_ctx1024", 24, 14, 64, 1024, 1152, [(16, 2)] + [(4, 2)] * 23, 0.0, 0, "student4"),
        ("config2_tinyllama_22x4_d64_ctx2048", 22, 4, 64, 2048, 2304, [(16, 2)] + [(3, 2)] * 21, 0.0, 0, "normal"),
    ]
    g = torch.Generator(device="cuda").manual_seed(7)
    for name, layers, heads, dim, ctx_len, cap, bits, v_mass, hyb, dist in cfgs:
        def inputs():
            k = torch.randn((ctx_len, layers, heads, dim), device="cuda", generator=g)
            v = torch.randn((ctx_len, layers, heads, dim), device="cuda", generator=g)
            if dist == "student4":  # heavy tails, crude stand-in: normal / sqrt(chi2/4)
                k = k / torch.sqrt(torch.randn((ctx_len, layers, heads, dim, 4), device="cuda", generator=g).pow(2).mean(-1))
            return k, v
        kn = torch.randn((layers, heads, dim), device="cuda", generator=g)
        q = torch.randn((layers, heads, dim), device="cuda", generator=g)
        o = torch.empty((layers, heads, dim), device="cuda")
        res = {"layers": layers, "heads": heads, "context": ctx_len}

        def time_it(step):
            for _ in range(5):
                step()
            torch.cuda.synchronize()
            steps = 200
            t0 = time.perf_counter()
            for _ in range(steps):
                step()
            torch.cuda.synchronize()
            return (time.perf_counter() - t0) / steps

        # (a) one handle for the whole model: a token is ONE library call
        stack = adaptq_b200.LayerStack(layers, heads, dim, k_bits=[b[0] for b in bits], v_bits=[b[1] for b in bits],
                                       capacity=cap, seed=42, v_mass=v_mass, hybrid_thresh=hyb)
        k, v = inputs()
        stack.append(k, v)
        launches0 = adaptq_b200.load().adaptq_kernel_launches()
        dt = time_it(lambda: stack.step(kn, kn, q, out=o))
        res.update({"us_per_token": dt * 1e6, "us_per_layer": dt * 1e6 / layers, "tokens_per_s": 1.0 / dt,
                    "launches_per_token": (adaptq_b200.load().adaptq_kernel_launches() - launches0) / 205, "parts": stack.parts})
        # the same step through the C ABI alone (adaptq_stack_decode_step with ready-made pointers)
        import ctypes as C
        Lc = adaptq_b200.load()
        cargs = [C.c_void_p(kn.data_ptr()), C.c_void_p(kn.data_ptr()), C.c_void_p(q.data_ptr()), C.c_void_p(o.data_ptr())]
        res["us_per_token_c_abi"] = time_it(lambda: Lc.adaptq_stack_decode_step(stack._h, *cargs, 0)) * 1e6
        stack.close()
        # (b) upstream's shape: one engine per layer, one decode-step call per layer
        if layers > 1:
            engines = [adaptq_b200.MHAContext(heads, dim, bits[l][0], bits[l][1], cap, seed=42 ^ l, v_mass=v_mass,
                                              hybrid_thresh=hyb) for l in range(layers)]
            for l, e in enumerate(engines):
                e.append_all(k[:, l].contiguous(), v[:, l].contiguous())

            def step_layers():
                for l, e in enumerate(engines):
                    e.decode_step(kn[l], kn[l], q[l], out=o[l])
            res["us_per_token_engine_per_layer"] = time_it(step_layers) * 1e6
            for e in engines:
                e.close()
        del k, v
        out[name] = res
    return out


def longctx_check(torch, dist, world, rank, ctx, keep_k, keep_v, q, o, kb, vb, N):
    """Rank 0 rebuilds head 0 of the sharded sequence on the CPU oracle (token t came from
    rank t mod G, local position t div G) and compares the merged output of the last step."""
    import numpy as np
    local = torch.stack([torch.cat(keep_k), torch.cat(keep_v)])  # [2, local_n, D] on the host
    if dist is not None:
        dev = local.cuda()
        gathered = [torch.empty_like(dev) for _ in range(world)] if rank == 0 else None
        dist.gather(dev, gathered, dst=0)
        parts = [g.cpu() for g in gathered] if rank == 0 else None
    else:
        parts = [local]
    if rank != 0:
        return None
    from oracle import loader
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import assert_close_conditioned, exact_attention_f64
    full = torch.stack(parts, dim=2).reshape(2, N, DIM).numpy()  # [2, local_n, G, D] -> token t = local*G + rank
    O = loader.oracle()
    hd = loader.Head(O, DIM, kb, vb, N, loader.mha_head_seed(42, 0))
    hd.append_many(full[0], full[1])
    q0 = q[0].cpu().numpy()
    want, _ = hd.compute(q0)
    got = o[0, 0].cpu().numpy()
    exact = exact_attention_f64(O, hd, q0)
    try:
        assert_close_conditioned(got, want, exact, "long-context head 0")
        outcome = "ok"
    except AssertionError as ex:
        outcome = f"FAILED: {ex}"
    return {"result": outcome, "max_abs_err_vs_oracle": float(np.abs(got - want).max()),
            "oracle_abs_err_vs_float64": float(np.abs(want - exact).max()), "head": 0, "tokens": N}


def longctx_bench(torch, dist, world, rank, steps, warmup, peak, exchange="nccl", check=False):
    """Contract configuration 5: ONE sequence, 1 layer, 32 KV heads, dim 128, context
    131072, K2/V2 and K4/V4, K/V Student-t(nu=3), dense V.  Token t lives on rank
    t mod G (local ring of 131072/G tokens).  One step = one decode query per
    head: every rank runs the split-KV kernel over its shard, the (max, sum,
    acc[128]) partials -- 16.6 KB per rank -- are all-gathered with NCCL and
    merged, one inverse transform finishes.  Total work is fixed (strong
    scaling).  L2 is flushed before every timed step, because at G >= 4 a
    rank's shard (<= 71 MB) would otherwise stay in the 126 MB L2."""
    import adaptq_b200
    H, D, N = 32, 128, 131072
    local_n = N // world
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    out = {}
    for kb, vb in ((2, 2), (4, 4)):
        ctx = adaptq_b200.MHAContext(H, D, kb, vb, local_n, seed=42, v_mass=0.0, hybrid_thresh=0)
        g = torch.Generator(device="cuda").manual_seed(500 + rank)
        done = 0
        keep_k, keep_v = [], []  # head 0's inputs, for the CPU check
        while done < local_n:
            t = min(4096, local_n - done)
            kv = []
            for _ in range(2):
                z = torch.randn((t, H, D), device="cuda", generator=g)
                chi = torch.randn((t, H, D, 3), device="cuda", generator=g).pow(2).mean(-1)
                kv.append(z / torch.sqrt(chi))  # Student-t, nu = 3
            ctx.append_all(kv[0], kv[1], done)
            if check:
                keep_k.append(kv[0][:, 0].cpu())
                keep_v.append(kv[1][:, 0].cpu())
            done += t
        gq = torch.Generator(device="cuda").manual_seed(77)  # the same query on every rank
        q = torch.randn((H, D), device="cuda", generator=gq)
        o = torch.empty((H, 1, D), device="cuda")
        part = torch.empty((H, 1, 2 + D), device="cuda")
        parts = torch.empty((world, H, 1, 2 + D), device="cuda")

        pg = None
        if exchange == "peer" and dist is None:
            # one rank: the same two kernels with this GPU's own buffers as the only "peer"
            class _Local:
                pass
            pg = _Local()
            n_buf = H * (2 + D)
            pg._t = torch.zeros(2 * n_buf + 64, dtype=torch.float32, device="cuda")
            pg.items, pg.step = H, 0
            base = pg._t.data_ptr()
            pg.buf_ptrs = [[base + 4 * par * n_buf] for par in (0, 1)]
            pg.flag_ptrs = [base + 8 * n_buf]
        if exchange == "peer" and dist is not None:
            from adaptq_b200.sharded import PeerGather
            ok = torch.ones(1, device="cuda")
            try:
                pg = PeerGather(H, 2 + D, world, rank)
            except Exception as ex:  # no mappable peer memory on this box: every rank falls back together
                print(f"peer exchange unavailable ({ex!r}); using the NCCL all-gather", file=sys.stderr)
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if float(ok.item()) == 0.0:
                pg = None

        def step_sharded():
            if pg is not None:  # the kernels deliver to every rank's buffer; the merge waits on arrival counts
                par = pg.step & 1
                ctx.compute_partial_to_peers(q, pg.buf_ptrs[par], pg.flag_ptrs, rank)
                pg.step += 1
                ctx.merge_from_peers(pg.buf_ptrs[par][rank], pg.flag_ptrs[rank], world, pg.step * pg.items, 1, out=o)
                return
            ctx.compute_partial(q, out=part)
            if dist is not None:
                dist.all_gather_into_tensor(parts, part)
                ctx.merge_partials(parts, nq=1, out=o)
            else:
                ctx.merge_partials(part.unsqueeze(0), nq=1, out=o)

        def step_local():
            ctx.compute_partial(q, out=part)

        def step_single():
            ctx.compute_all(q, out=o[:, 0])

        def timed(fn, queued=True):
            """Median device time of one step (CUDA events around it), max over ranks.  L2 is flushed
            before every step.  queued=True: the step is enqueued while the flush kernel still runs, so
            the events bracket the step's own device work; queued=False: the device is idle when the
            step is issued, so the figure also contains the host's launch latency."""
            for _ in range(max(3, warmup)):
                fn()
            samples = []
            for _ in range(steps):
                torch.cuda.synchronize()
                if dist is not None:
                    dist.barrier()
                    torch.cuda.synchronize()
                flush.fill_(1)
                if not queued:
                    torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                samples.append(a.elapsed_time(b))
            samples.sort()  # the median: a step that catches a stray millisecond must not carry the figure
            t = torch.tensor([samples[len(samples) // 2]], device="cuda")
            if dist is not None:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item()) * 1e3  # us

        alg = H * (N * (D * kb // 8 + D * vb // 8 + 8) + 8 * D)
        us_total = timed(step_sharded)
        us_local = timed(step_local)
        res = {"exchange": ("peer" if pg is not None else "nccl") if (dist is not None or pg is not None) else "none", "us_per_step": us_total, "us_local_kernels": us_local, "us_gather_and_merge": us_total - us_local,
               "effective_kv_gbs_all_ranks": alg / us_total / 1e3, "local_kernel_gbs_per_gpu": alg / world / us_local / 1e3,
               "local_kernel_frac_of_peak": alg / world / us_local / 1e3 / peak,
               "algorithmic_bytes": alg, "tokens_per_rank": local_n}
        res["us_per_step_incl_host_launch"] = timed(step_sharded, queued=False)
        res["exchange_share"] = max(0.0, us_total - us_local) / us_total
        res["frac_of_peak_all_ranks"] = alg / us_total / 1e3 / (peak * world)
        if world == 1:
            res["us_per_step_compute_all"] = timed(step_single)
        if check:
            step_sharded()
            torch.cuda.synchronize()
            res["sharded_check"] = longctx_check(torch, dist, world, rank, ctx, keep_k, keep_v, q, o, kb, vb, N)
        out[f"k{kb}v{vb}"] = res
        ctx.close()
    return out


def run_ours(args):
    import numpy as np
    import torch
    import adaptq_b200

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = adaptq_b200.load()
    if args.general_kernel:
        L.adaptq_set_kernel_policy(1)
    peak, peak_src = measured_peak()
    if args.mode == "append":
        if rank == 0:
            emit({"metric": "bulk_append_vectors_per_s", "append": append_bench(torch, L, peak)})
        return
    if args.mode == "latency":
        if rank == 0:
            emit({"metric": "decode_latency_us_per_token", "latency": latency_bench(torch)})
        return

    if args.mode == "longctx":
        res = longctx_bench(torch, dist, world, rank, args.steps, args.warmup, peak, args.exchange)
        if rank == 0:
            emit({"metric": "long_context_decode_us_per_step", "unit": "us", "n_gpus": world,
                              "steps": args.steps, "higher_is_better": False, "scaling": "strong", "dtype": "f32",
                              "data": "synthetic",
                              "config": {"workload": "one sequence, 32 KV heads, dim 128, context 131072, KV range split "
                                                     "by token over the ranks, split-KV partials combined by "
                                                     + ("an NCCL all-gather" if args.exchange == "nccl" else
                                                        "kernel stores into peer memory over NVLink")
                                                     + " (BASELINE configs[4])", "l2": "L2 flushed before every timed step"},
                              "results": res})
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    heads = args.seqs * LAYERS * KV_HEADS
    n = args.context
    seeds = [(42 ^ layer) ^ (hd * 0xDEADBEEFCAFE) for _s in range(args.seqs) for layer in range(LAYERS)
             for hd in range(KV_HEADS)]
    ctx = adaptq_b200.MHAContext(heads, DIM, K_BITS, V_BITS, n, seeds=seeds, v_mass=0.0, hybrid_thresh=0)
    gen = torch.Generator(device="cuda").manual_seed(1000 + rank)
    do_parity = rank == 0 and not args.skip_parity_sample
    sample_heads = sorted({0, heads // 3, (2 * heads) // 3 + 1, heads - 1}) if do_parity else []
    kept_k, kept_v = fill_cache(ctx, heads, n, torch, gen, sample_heads)

    # device-resident inputs for `value`, pinned host inputs for `e2e`
    d_k = torch.randn((heads, DIM), device="cuda", generator=gen)
    d_v = torch.randn((heads, DIM), device="cuda", generator=gen)
    d_q = torch.randn((heads, DIM), device="cuda", generator=gen)
    d_o = torch.empty((heads, DIM), device="cuda")
    h_k, h_v, h_q = (t.cpu().pin_memory() for t in (d_k, d_v, d_q))
    h_o = torch.empty((heads, DIM)).pin_memory()

    n_steps_done = [0]  # every step appends (d_k, d_v) once more; the CPU check replays them

    def step_device():
        ctx.append_all(d_k, d_v)
        ctx.compute_all(d_q, out=d_o)
        n_steps_done[0] += 1

    def step_host():  # one C-ABI call: uploads, kernels and the download are pipelined inside
        ctx.decode_step(h_k, h_v, h_q, out=h_o)
        n_steps_done[0] += 1

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, with_kernel_events=False):
        evs = []
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        launches0 = L.adaptq_kernel_launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            if with_kernel_events:
                ctx.append_all(d_k, d_v)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                ctx.compute_all(d_q, out=d_o)
                b.record()
                evs.append((a, b))
                n_steps_done[0] += 1
            else:
                fn()
        e1.record()
        barrier()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        kern_ms = [a.elapsed_time(b) for a, b in evs]
        return ms, clocks, L.adaptq_kernel_launches() - launches0, kern_ms

    for _ in range(max(3, args.warmup)):
        step_device()
    ms, clocks, launches, kern_ms = timed(step_device, args.steps, with_kernel_events=True)
    ctx.synchronize()
    for _ in range(2):
        step_host()
    ms_h, clocks_h, _, _ = timed(step_host, args.steps)
    ctx.synchronize()

    seqs_total = args.seqs * world
    value = seqs_total * args.steps / (ms / 1e3)
    e2e = seqs_total * args.steps / (ms_h / 1e3)
    alg_bytes = heads * (n * (DIM * K_BITS // 8 + DIM * V_BITS // 8 + 8) + 8 * DIM)
    kt = sum(kern_ms) / len(kern_ms) / 1e3
    clk = clocks["sm_mhz"] / clocks["sm_max_mhz"] if clocks.get("sm_mhz") and clocks.get("sm_max_mhz") else None
    roof = {"bound": "hbm", "kernel": (f"compute_general_kernel<by words> K{K_BITS}/V{V_BITS} dim128" if args.general_kernel else
                       f"compute_stream_kernel<K{K_BITS},V{V_BITS},dim128>"), "achieved": alg_bytes / kt / 1e9,
            "peak": peak, "unit": "GB/s", "frac": alg_bytes / kt / 1e9 / peak, "peak_source": peak_src,
            # the same fraction had the SM clock stayed at its maximum (kernel time x median MHz / max MHz):
            # separates the share of the power cap from the kernel's own
            "frac_at_max_sm_clock": (alg_bytes / (kt * clk) / 1e9 / peak) if clk else None,
            "traffic": alg_bytes * STREAM_TRAFFIC_PER_ALG_BYTE,
            "traffic_source": "ncu dram__bytes_read+write on a 1024-head launch, scaled by heads (profiles/)",
            "algorithmic_bytes_per_launch": alg_bytes, "kernel_ms": kt * 1e3,
            "of_nominal_8TBs": alg_bytes / kt / 8e12}

    line = {"metric": "decode_attn_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args), "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 3 * heads * DIM * 4,
                    "d2h_bytes_per_step": heads * DIM * 4, "ms_per_step": ms_h / args.steps, "clocks": clocks_h},
            "gpu_launches": int(launches), "roofline": roof,
            "effective_kv_gbs": alg_bytes * world / (ms / args.steps / 1e3) / 1e9}
    if do_parity:
        try:
            # one more device step so that d_o belongs to the cache state the CPU replays
            step_device()
            ctx.synchronize()
            hk, hv = d_k[sample_heads].cpu().numpy(), d_v[sample_heads].cpu().numpy()
            line["parity_sample"] = parity_sample(ctx, sample_heads, seeds, kept_k, kept_v, [hk] * n_steps_done[0],
                                                  [hv] * n_steps_done[0], d_q, d_o, n)
        except Exception as ex:  # the headline must still print
            line["parity_sample"] = {"error": repr(ex)}
    ctx.close()
    del ctx
    torch.cuda.empty_cache()
    if not args.skip_longctx:
        # the long-context configuration on the same ranks (KV range split by token; strong scaling)
        try:
            lres = longctx_bench(torch, dist, world, rank, args.longctx_steps, args.warmup, peak, args.exchange, check=True)
            if rank == 0:
                line["longctx"] = {"workload": "one sequence, 32 KV heads, dim 128, context 131072, Student-t(3), KV range "
                                               "split by token over the ranks (BASELINE configs[4]); L2 flushed before "
                                               "every timed step, the step enqueued behind the flush (device time of the "
                                               "step; us_per_step_incl_host_launch: issued on an idle device); medians; "
                                               "max over ranks", "scaling": "strong",
                                   "n_gpus": world, "results": lres}
        except Exception as ex:
            line["longctx"] = {"error": repr(ex)}
    if rank == 0:
        if not args.skip_append_bench:
            try:
                line["append"] = append_bench(torch, L, peak)
            except Exception as ex:  # the headline must still print
                line["append"] = {"error": repr(ex)}
        if not args.skip_cpu_baseline and world == 1:
            try:
                threads = host_threads()
                _, desc = cpu_arm(args.cpu_sample_heads or max(2 * threads, 64), n, 4, 1, args.seqs, threads)
                line["cpu_baseline"] = desc
            except Exception as ex:
                line["cpu_baseline"] = {"error": repr(ex)}
        emit(line)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    global K_BITS, V_BITS
    args = parse()
    K_BITS, V_BITS = args.k_bits, args.v_bits
    claim_stdout()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
