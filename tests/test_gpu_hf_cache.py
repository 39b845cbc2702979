"""AdapTQCache + the fused attention function inside a Hugging Face model (a tiny
randomly initialised Llama; no weights or tokenizer are downloaded): the logits of
prompt + decode steps equal those of the same model attending, with its stock eager
attention, to the dequantised history that upstream's AdapTQCache would hand it
(adaptq/runtime_py/backends/transformers_hf.py:107-171) -- and the device caches
behind both hold the rows the CPU oracle packs from the same K/V."""
import numpy as np
import pytest

from helpers import CpuHeads, assert_cache_equal, assert_close

pytestmark = pytest.mark.gpu


def _tiny_llama(attn, torch):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=97, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=32, max_position_embeddings=128, attn_implementation=attn)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).to("cuda").eval()


@pytest.mark.parametrize("kb,vb", [(4, 4), (4, 2), (16, 2)])
def test_fused_cache_equals_dequantised_history(gpu_lib, orc, kb, vb):
    import torch
    from adaptq_b200.hf_cache import AdapTQCache, register_attention
    name = register_attention()
    fused_model, eager_model = _tiny_llama(name, torch), _tiny_llama("eager", torch)
    eager_model.load_state_dict(fused_model.state_dict())
    mk = lambda: AdapTQCache(n_layers=2, n_heads=4, head_dim=32, n_kv_heads=2, adaptq_capacity=64, k_bits=kb, v_bits=vb)
    fused_cache, ref_cache = mk(), mk()
    ref_cache.fused = False                       # update() returns the dequantised history, as upstream's class does
    torch.manual_seed(1)
    ids = torch.randint(0, 97, (1, 12), device="cuda")
    with torch.no_grad():
        a = fused_model(ids, past_key_values=fused_cache, use_cache=True).logits
        b = eager_model(ids, past_key_values=ref_cache, use_cache=True).logits
        torch.testing.assert_close(a, b, rtol=2e-4, atol=2e-4)
        for step in range(6):                     # greedy decode, one token at a time
            nxt = b[:, -1:].argmax(-1)
            a = fused_model(nxt, past_key_values=fused_cache, use_cache=True).logits
            b = eager_model(nxt, past_key_values=ref_cache, use_cache=True).logits
            torch.testing.assert_close(a, b, rtol=2e-4, atol=2e-4, msg=f"decode step {step}")
    assert fused_cache.get_seq_length() == ref_cache.get_seq_length() == 18
    assert fused_cache.kv_bytes() == ref_cache.kv_bytes() > 0
    # Both caches were fed the same K/V up to the rounding of the two attention paths (layer 1's
    # K/V depend on layer 0's attention output): layer 0 identical, layer 1 all but identical.
    for l in range(2):
        for h in range(2):
            ea, eb = fused_cache._ctx[l].export_head(h), ref_cache._ctx[l].export_head(h)
            for key, bits in (("k_rows", kb), ("v_rows", vb)):
                if l == 0:
                    assert np.array_equal(ea[key], eb[key]), (l, h, key)
                elif bits == 16:
                    np.testing.assert_allclose(ea[key].view(np.float32), eb[key].view(np.float32), rtol=1e-3, atol=1e-4)
                else:
                    assert (ea[key] == eb[key]).mean() > 0.98, (l, h, key)


def test_dequantised_history_is_upstreams_arithmetic(gpu_lib, orc):
    """AdapTQCache.dequantized() against the oracle's restatement of dequantize_raw, row by row, on a wrapped ring."""
    import ctypes as C
    import torch
    from adaptq_b200.hf_cache import AdapTQCache
    from oracle import loader
    cache = AdapTQCache(n_layers=1, n_heads=2, head_dim=64, adaptq_capacity=20, k_bits=3, v_bits=4)
    rng = np.random.default_rng(0)
    k = rng.standard_normal((1, 2, 30, 64)).astype(np.float32)
    v = rng.standard_normal((1, 2, 30, 64)).astype(np.float32)
    cache.fused = False
    kd, vd = cache.update(torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), 0)
    assert kd.shape == (1, 2, 20, 64)
    cpu = CpuHeads(orc, 2, 64, 3, 4, 20, 42)
    cpu.append_many(np.ascontiguousarray(k[0].transpose(1, 0, 2)), np.ascontiguousarray(v[0].transpose(1, 0, 2)))
    f = orc.lib.orc_dequantize_raw
    f.argtypes = [C.c_void_p, C.c_float, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    f.restype = None
    for h in range(2):
        hd = cpu.heads[h]
        assert_cache_equal(cache._ctx[0].export_head(h), hd, f"head {h}")
        order = (np.arange(20) + hd.ring_head) % 20      # oldest first on the full ring
        for side, bits, got in (("k", 3, kd), ("v", 4, vd)):
            rows = (hd.k_data() if side == "k" else hd.v_data())[order]
            sc = (hd.k_scale() if side == "k" else hd.v_scale())[order]
            D = hd.signs()
            for i in range(20):
                out = np.zeros(64, np.float32)
                row = np.ascontiguousarray(rows[i])
                f(row.ctypes.data, C.c_float(float(sc[i])), 64, D.ctypes.data, bits, out.ctypes.data)
                assert_close(got[0, h, i].cpu().numpy(), out, f"{side} row {i} head {h}", atol=1e-5)
