"""GPU tests of the HuggingFace cache class and the C-ABI error behaviour."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from util import attention_close

pytestmark = pytest.mark.gpu


def test_hf_cache_update_returns_old_dequantised_new_exact(orc):
    from turboquant_kv import TurboQuantCache

    cache = TurboQuantCache(key_bits=4, value_bits=2, seed=42)
    gen = torch.Generator().manual_seed(0)
    k0, v0 = torch.randn(2, 4, 12, 64, generator=gen).cuda(), torch.randn(2, 4, 12, 64, generator=gen).cuda()
    k1, v1 = torch.randn(2, 4, 1, 64, generator=gen).cuda(), torch.randn(2, 4, 1, 64, generator=gen).cuda()
    ka, va = cache.update(k0, v0, 0)
    assert torch.equal(ka, k0) and torch.equal(va, v0)          # first call: everything is "new", exact
    kb, vb = cache.update(k1, v1, 0)
    assert kb.shape == (2, 4, 13, 64) and torch.equal(kb[:, :, 12:], k1) and torch.equal(vb[:, :, 12:], v1)
    rk = orc.make_rotation_matrix(64, 42)
    bk, ck = orc.lloyd_max_codebook(4, 64)
    p, n = orc.quantize_mse(k0.cpu().numpy().reshape(-1, 64), 4, rk, bk)
    want = orc.dequantize_mse(p, n, 4, 64, rk, ck).reshape(2, 4, 12, 64)
    assert np.abs(kb[:, :, :12].cpu().numpy() - want).max() < 2e-2 * np.abs(want).max()
    assert cache.get_seq_length(0) == 13 and len(cache) == 1 and cache.seen_tokens == 13
    assert cache.memory_bytes() == 2 * 4 * 13 * (32 + 16 + 8)
    # fast path: the same attention without the dense round trip
    q = torch.randn(2, 8, 64, generator=gen).cuda()
    out = cache.decode_attention(q, 0)
    st = cache._layer_stores[0]
    rv = orc.make_rotation_matrix(64, 43)
    _, cv = orc.lloyd_max_codebook(2, 64)
    kp, kn, vp, vn = (t.cpu().numpy() for t in st.export())
    ref = orc.decode_attention(q.cpu().numpy(), kp, kn, vp, vn, np.full(2, 13, np.int32), rk, ck, 4, rv, cv, 2)
    attention_close(out.cpu().numpy(), ref)
    k_it, v_it = cache[0]
    assert k_it.shape == (2, 4, 13, 64)


def test_hf_cache_protected_layers_keep_full_precision():
    from turboquant_kv import TurboQuantCache

    cache = TurboQuantCache(protected_layers=1)
    k, v = torch.randn(1, 2, 3, 64, device="cuda"), torch.randn(1, 2, 3, 64, device="cuda")
    ka, _ = cache.update(k, v, 0)
    kb, _ = cache.update(k, v, 0)
    assert torch.equal(kb, torch.cat([k, k], 2)) and cache.get_seq_length(0) == 6


def test_c_abi_reports_errors_without_raising_across_the_boundary():
    from turboquant_kv import _native as N

    L = N.lib()
    x = torch.zeros(4, 64, device="cuda")
    rc = L.tqb_quantize_mse(N.ptr(x), 0, 4, 64, 64, N.ptr(x), N.ptr(x), 9, N.ptr(x), N.ptr(x), None, None)
    assert rc == -1 and b"bit_width" in L.tqb_last_error()
    rc = L.tqb_quantize_mse(N.ptr(x), 0, 4, 1000, 1000, N.ptr(x), N.ptr(x), 4, N.ptr(x), N.ptr(x), None, None)
    assert rc == -2
    rc = L.tqb_decode_attention(N.ptr(x), 0, 1, 4, 4, 64, N.ptr(x), 16, N.ptr(x), 16,
                                None, 0, 0, N.ptr(x), N.ptr(x), 4, N.ptr(x), N.ptr(x), 2, ctypes.c_float(1.0),
                                N.ptr(x), 16, N.ptr(x), 0, None)
    assert rc == -4 and b"workspace" in L.tqb_last_error()
    # unsupported bit widths and absurd lengths are refused before anything is launched
    before = N.launch_count()
    big = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    rc = L.tqb_decode_attention(N.ptr(x), 0, 1, 4, 4, 64, N.ptr(x), 16, N.ptr(x), 16,
                                None, 0, 0, N.ptr(x), N.ptr(x), 5, N.ptr(x), N.ptr(x), 2, ctypes.c_float(1.0),
                                N.ptr(big), big.numel(), N.ptr(x), 0, None)
    assert rc == -2 and b"bits" in L.tqb_last_error() and N.launch_count() == before
    assert L.tqb_decode_attention_workspace_bytes(1, 4, 4, 64, 1 << 40) == 0
    before = N.launch_count()
    y = torch.zeros(4, 8, dtype=torch.uint8, device="cuda")
    assert L.tqb_pack_codes(N.ptr(torch.zeros(4, 64, dtype=torch.uint8, device="cuda")), 4, 64, 1, N.ptr(y), None) == 0
    assert N.launch_count() == before + 1
    torch.cuda.synchronize()


def test_hf_cache_prod_mode_matches_upstream_fixture(orc, golden):
    """TurboQuantCache(mode="prod") (upstream hf_integration.py:82-236): update() returns the Algorithm-2
    reconstruction of the old tokens and the new tokens exactly; compared with the outputs of the upstream
    class on the same inputs and with the CPU checker's quantize_prod / dequantize_prod."""
    from turboquant_kv import TurboQuantCache

    g = golden("hf_prod")
    cache = TurboQuantCache(key_bits=3, value_bits=4, mode="prod", seed=42)
    seen = 0
    for step in (0, 1):
        k, v = torch.from_numpy(g[f"k{step}"]).cuda(), torch.from_numpy(g[f"v{step}"]).cuda()
        ko, vo = cache.update(k, v, 0)
        assert ko.shape == tuple(g[f"keys_out{step}"].shape) and vo.shape == ko.shape
        assert torch.equal(ko[:, :, seen:], k) and torch.equal(vo[:, :, seen:], v)       # new tokens exact
        np.testing.assert_allclose(ko.cpu().numpy(), g[f"keys_out{step}"], atol=3e-5)
        np.testing.assert_allclose(vo.cpu().numpy(), g[f"values_out{step}"], atol=3e-5)
        seen += k.shape[2]
    assert cache.get_seq_length(0) == 8
    # the stored rows against the checker
    st = cache._layer_stores[0]
    for which, bits, seed in (("key", 3, 42), ("value", 4, 43)):
        x = np.concatenate([g[f"{which[0]}0"], g[f"{which[0]}1"]], axis=2).reshape(-1, 64)
        rot = orc.make_rotation_matrix(64, seed)
        bnd, cent = orc.lloyd_max_codebook(bits - 1, 64)
        S = orc.make_qjl_matrix(64, 64, seed)
        mp, sg, rn, nr = orc.quantize_prod(x, bits, rot, bnd, cent, S)
        got = [t.reshape((-1,) + tuple(t.shape[3:])).cpu().numpy() for t in st.export(which)]
        assert np.array_equal(got[0], mp) and np.array_equal(got[1], sg)
        np.testing.assert_allclose(got[2], rn, rtol=1e-5)
        np.testing.assert_allclose(got[3], nr, rtol=2e-6)
    assert cache.memory_bytes() == 2 * 2 * 8 * ((2 * 8 + 8 + 8) + (3 * 8 + 8 + 8))
    with pytest.raises(RuntimeError):
        cache.decode_attention(torch.zeros(2, 2, 64, device="cuda"), 0)


def _tiny_llama(dtype=torch.float16):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, max_position_embeddings=512)
    return LlamaForCausalLM(cfg).to("cuda", dtype).eval()


def test_hf_model_runs_the_fused_kernel_through_the_attention_registry(monkeypatch):
    """A stock transformers model with an attached cache: decode steps never rebuild the dense history
    (upstream hf_integration.py:373-390 does), and the logits stay those of the dense contract up to the
    quantisation of the one new token."""
    from turboquant_kv import TurboQuantCache
    from turboquant_kv import hf_integration as hf

    model = _tiny_llama()
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 512, (2, 40), generator=gen).cuda()
    steps = torch.randint(0, 512, (2, 6), generator=gen).cuda()

    def run(cache, mask=None):
        logits = []
        with torch.no_grad():
            out = model(input_ids=prompt, past_key_values=cache, attention_mask=mask, use_cache=True)
            logits.append(out.logits[:, -1].float())
            for t in range(steps.shape[1]):
                if mask is not None:
                    mask = torch.cat([mask, mask.new_ones(2, 1)], dim=1)
                out = model(input_ids=steps[:, t:t + 1], past_key_values=cache, attention_mask=mask, use_cache=True)
                logits.append(out.logits[:, -1].float())
        return torch.stack(logits)

    model.set_attn_implementation("sdpa")
    dense_cache = TurboQuantCache(key_bits=4, value_bits=2, seed=42)
    dense = run(dense_cache)

    calls = {"fused": 0, "dense": 0}
    real_decode, real_dense = hf._LayerQuantStore.decode_attention, hf._LayerQuantStore._dense
    monkeypatch.setattr(hf._LayerQuantStore, "decode_attention",
                        lambda self, *a, **k: (calls.__setitem__("fused", calls["fused"] + 1), real_decode(self, *a, **k))[1])
    monkeypatch.setattr(hf._LayerQuantStore, "_dense",
                        lambda self, *a, **k: (calls.__setitem__("dense", calls["dense"] + (self.seq_len > 0)), real_dense(self, *a, **k))[1])
    fused_cache = TurboQuantCache(key_bits=4, value_bits=2, seed=42).attach(model)
    assert model.config._attn_implementation == hf.ATTENTION_NAME
    fused = run(fused_cache)
    assert calls == {"fused": 2 * steps.shape[1], "dense": 0}        # 2 layers x 6 steps, no dequantisation at all
    assert fused_cache.get_seq_length(0) == 46 and fused_cache.get_mask_sizes(1, 0) == (47, 0)
    # layer 0 sees the same tokens in both runs: its packed records are the same bytes
    for a, b in zip(dense_cache._layer_stores[0].export(), fused_cache._layer_stores[0].export()):
        assert torch.equal(a, b)
    assert torch.equal(dense[0], fused[0])                            # the prompt pass is the same computation
    cos = torch.nn.functional.cosine_similarity(dense.flatten(1), fused.flatten(1), dim=1)
    assert float(cos.min()) > 0.999, cos
    assert float((dense - fused).abs().max()) < 0.05 * float(dense.abs().max())

    # a padded batch keeps the dense contract (old tokens dequantised, new token exact): same logits as before attach
    mask = torch.ones(2, 40, dtype=torch.long, device="cuda")
    mask[1, :5] = 0
    model.set_attn_implementation("sdpa")
    want = run(TurboQuantCache(key_bits=4, value_bits=2, seed=42), mask)
    calls.update(fused=0, dense=0)
    got = run(TurboQuantCache(key_bits=4, value_bits=2, seed=42).attach(model), mask)
    assert calls["fused"] == 0 and calls["dense"] > 0
    assert torch.allclose(want, got, atol=2e-3, rtol=2e-3)

    # generate() drives the same path: every decode step of every layer runs the fused kernel
    calls.update(fused=0, dense=0)
    cache = TurboQuantCache(key_bits=4, value_bits=2, seed=42).attach(model)
    tokens = model.generate(input_ids=prompt, attention_mask=torch.ones_like(prompt), past_key_values=cache,
                            max_new_tokens=5, min_new_tokens=5, do_sample=False, pad_token_id=0)
    assert tokens.shape == (2, 45) and cache.get_seq_length(0) == 44
    assert calls == {"fused": 2 * 4, "dense": 0}
