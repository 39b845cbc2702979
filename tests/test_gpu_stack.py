"""LayerStack (adaptq_stack_*): every layer of a model behind one handle.  A stack
must hold exactly what a list of per-layer Engines holds (seed ^ layer, upstream's
convention) and return what they return -- checked against the CPU oracle, with the
layer-aware policy's mixed bit widths (FP32 keys in layer 0), host and device
buffers, Engine defaults (sparse V + FP32 window) and a wrapped ring."""
import numpy as np
import pytest

from helpers import CpuHeads, assert_cache_equal, assert_close, assert_sparse_close, make_kv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kb,vb,kw,device", [
    ([16, 4, 4, 4], [2, 2, 2, 2], dict(v_mass=0.0, hybrid_thresh=0), True),
    ([16, 3, 3, 2, 2], [2, 2, 2, 4, 4], dict(v_mass=0.0, hybrid_thresh=0), False),   # three parts, host buffers
    ([4, 4, 4, 3, 3, 4], [2, 2, 2, 2, 4, 4], dict(v_mass=0.0, hybrid_thresh=0), True), # four parts, all on the persistent kernel, own streams
    ([16, 4, 4], [2, 2, 2], dict(), True),                                           # Engine defaults
    (4, 4, dict(v_mass=0.0, hybrid_thresh=0), True),                                 # one part
])
def test_stack_equals_per_layer_engines(gpu_lib, orc, kb, vb, kw, device):
    import torch
    from adaptq_b200.stack import LayerStack
    layers = len(kb) if isinstance(kb, list) else 3
    kbl = kb if isinstance(kb, list) else [kb] * layers
    vbl = vb if isinstance(vb, list) else [vb] * layers
    heads, dim, cap, prefill, steps = 3, 64, 40, 30, 25
    vm, hyb = kw.get("v_mass", 0.95), kw.get("hybrid_thresh", 512)
    st = LayerStack(layers, heads, dim, k_bits=kb, v_bits=vb, capacity=cap, seed=42, **kw)
    assert st.parts == len({(a, b, i) for i, (a, b) in enumerate(zip(kbl, vbl)) if i == 0 or (a, b) != (kbl[i - 1], vbl[i - 1])})
    cpus = [CpuHeads(orc, heads, dim, kbl[l], vbl[l], cap, 42 ^ l, vm, hyb) for l in range(layers)]
    rng = np.random.default_rng(layers)
    conv = (lambda a: torch.from_numpy(a).cuda()) if device else (lambda a: a)
    back = (lambda t: t.cpu().numpy()) if device else (lambda t: t)
    k = rng.standard_normal((prefill + steps, layers, heads, dim)).astype(np.float32)
    v = rng.standard_normal((prefill + steps, layers, heads, dim)).astype(np.float32)
    st.append(conv(k[:prefill]), conv(v[:prefill]))
    for l in range(layers):
        cpus[l].append_many(k[:prefill, l], v[:prefill, l])
    for s in range(steps):                      # wraps the ring at step 10
        t = prefill + s
        q = rng.standard_normal((layers, heads, dim)).astype(np.float32)
        out = back(st.step(conv(k[t]), conv(v[t]), conv(q)))
        for l in range(layers):
            cpus[l].append_many(k[t:t + 1, l], v[t:t + 1, l])
            hd0 = cpus[l].heads[0]
            sparse = vm > 0 and kbl[l] != 16 and hd0.mirror_tokens != hd0.size
            for h in range(heads):
                if sparse:
                    assert_sparse_close(out[l, h], cpus[l].heads[h], q[l, h], vm, f"step {s} layer {l} head {h}")
                else:
                    assert_close(out[l, h], cpus[l].heads[h].compute(q[l, h])[0], f"step {s} layer {l} head {h}")
    assert st.pos == prefill + steps
    assert st.kv_bytes == sum(h.kv_bytes for c in cpus for h in c.heads)
    for l in range(layers):
        for h in (0, heads - 1):
            assert_cache_equal(st.export_head(l, h), cpus[l].heads[h], f"layer {l} head {h}")
    st.synchronize()
    q = rng.standard_normal((layers, heads, dim)).astype(np.float32)
    again = back(st.compute(conv(q)))
    st.reset()
    assert st.kv_bytes == 0 and st.pos == 0
    assert not np.any(back(st.compute(conv(q)))) and np.any(again)


def test_stack_argument_errors(gpu_lib):
    import ctypes as C
    from adaptq_b200.stack import LayerStack
    L = gpu_lib
    with pytest.raises(ValueError):
        LayerStack(3, 2, 64, k_bits=[4, 4], v_bits=2)
    with pytest.raises(RuntimeError):
        LayerStack(2, 2, 64, k_bits=[4, 5], v_bits=2)
    st = LayerStack(2, 2, 64, k_bits=4, v_bits=2, capacity=8)
    with pytest.raises(ValueError):
        st.append(np.zeros((2, 3, 64), np.float32), np.zeros((2, 3, 64), np.float32))
    assert L.adaptq_stack_decode_step(st._h, None, None, None, None, 0) == -1
    assert L.adaptq_last_error().decode() == "adaptq_stack_decode_step: null keys"
    assert L.adaptq_stack_compute(None, None, None) == -1
    assert L.adaptq_last_error().decode() == "adaptq_stack_compute: null handle"
    assert L.adaptq_stack_layer_handle(st._h, 5, None) is None
