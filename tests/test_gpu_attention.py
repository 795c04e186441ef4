"""GPU parity: operator-level attention, the cache API and the fused decode kernel.

Bar (float): within 1e-2 max-abs and cosine >= 0.9999 of the dequantise-then-attend result, which is
what the oracle computes (oracle/tq_oracle.c, tqo_decode_attention) and what the golden fixtures
hold from the upstream cache."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from util import attention_close

pytestmark = pytest.mark.gpu


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def exported(cache, layer, seq):
    """Upstream-layout numpy copies (batch, heads, seq, ...) of a QuantizedKVCache layer."""
    B, H = cache._batch, cache.num_heads
    kp, kn, vp, vn = cache._export(layer, seq)
    return (kp.view(B, H, seq, -1).cpu().numpy(), kn.view(B, H, seq).cpu().numpy(),
            vp.view(B, H, seq, -1).cpu().numpy(), vn.view(B, H, seq).cpu().numpy())


@pytest.mark.parametrize("tag,dim,kb,vb", [("k4v2_d64", 64, 4, 2), ("k4v3_d128", 128, 4, 3), ("k2v4_d64", 64, 2, 4)])
def test_operator_level_scores_and_values(orc, golden, tag, dim, kb, vb):
    from turboquant_kv import ops

    g = golden("attention")
    q = g[f"{tag}_q"]
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    _, ck = orc.lloyd_max_codebook(kb, dim)
    _, cv = orc.lloyd_max_codebook(vb, dim)
    for h in range(g[f"{tag}_k"].shape[0]):
        kp, kn = g[f"{tag}_key_packed"][h], g[f"{tag}_key_norms"][h]
        sc = ops.attention_scores_packed(cuda(q[:, h:h + 1, 0, :]), cuda(kp), cuda(kn), cuda(ck), cuda(rk), kb)
        want = orc.attention_scores_packed(q[:, h:h + 1, 0, :], kp, kn, ck, rk, kb)
        np.testing.assert_allclose(sc.cpu().numpy(), want, rtol=1e-4, atol=1e-4 * np.abs(want).max())
        ref_l = g[f"{tag}_logits"][:, h, 0, :] * math.sqrt(dim)
        np.testing.assert_allclose(sc.cpu().numpy()[:, 0], ref_l, rtol=1e-3, atol=1e-4 * np.abs(ref_l).max())
        w = torch.softmax(torch.from_numpy(g[f"{tag}_logits"][:, h, 0, :]), -1).numpy()[:, None, :]
        vp, vn = g[f"{tag}_val_packed"][h], g[f"{tag}_val_norms"][h]
        o = ops.attention_values_packed(cuda(w), cuda(vp), cuda(vn), cuda(cv), cuda(rv), vb)
        np.testing.assert_allclose(o.cpu().numpy()[:, 0], g[f"{tag}_out"][:, h, 0, :], atol=2e-4)


def test_torch_operator_library_is_registered():
    from turboquant_kv import ops

    ops.register_torch_ops()
    codes = torch.randint(0, 16, (5, 64), dtype=torch.uint8, device="cuda")
    packed = torch.ops.turboquant.pack_codes(codes, 4)
    assert torch.equal(torch.ops.turboquant.unpack_codes(packed, 4, 64), codes)


@pytest.mark.parametrize("tag,dim,kb,vb", [("k4v2_d64", 64, 4, 2), ("k4v3_d128", 128, 4, 3), ("k2v4_d64", 64, 2, 4)])
def test_cache_api_matches_upstream(golden, tag, dim, kb, vb):
    """append + attention_scores + attention_values + fused decode against the upstream cache's outputs."""
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig

    g = golden("attention")
    k, v, q = g[f"{tag}_k"], g[f"{tag}_v"], g[f"{tag}_q"]
    heads, seq, _ = k.shape
    cache = QuantizedKVCache(TurboQuantConfig(key_bits=kb, value_bits=vb, seed=42), num_layers=1, max_seq_len=256,
                             num_heads=heads, head_dim=dim, device="cuda")
    cut = min(150, seq)
    cache.append(0, cuda(k[:, :cut]), cuda(v[:, :cut]))
    if cut < seq:
        cache.append(0, cuda(k[:, cut:]), cuda(v[:, cut:]))
    assert int(cache.seq_lens[0]) == seq
    kp = cache._key_packed[0][:, :seq].cpu().numpy()
    assert (kp != g[f"{tag}_key_packed"]).mean() < 1e-3          # boundary ties only
    np.testing.assert_allclose(cache._key_norms[0][:, :seq].cpu().numpy(), g[f"{tag}_key_norms"], rtol=2e-6)
    logits = cache.attention_scores(0, cuda(q))
    ref_l = g[f"{tag}_logits"]
    assert logits.shape == ref_l.shape
    np.testing.assert_allclose(logits.cpu().numpy(), ref_l, rtol=2e-3, atol=2e-3 * np.abs(ref_l).max())
    out = cache.attention_values(0, torch.softmax(logits, dim=-1))
    attention_close(out.cpu().numpy(), g[f"{tag}_out"], max_abs=5e-3)
    assert cache.memory_bytes() == int(g[f"{tag}_memory_bytes"])
    assert abs(cache.compression_ratio - float(g[f"{tag}_compression_ratio"])) < 1e-9
    # fused path, one query at a time (the cache holds a single sequence)
    for b in range(q.shape[0]):
        fused = cache.decode_attention(0, cuda(q[b:b + 1, :, 0, :]))
        attention_close(fused.float().cpu().numpy(), g[f"{tag}_out"][b:b + 1, :, 0, :])
    assert cache.decode_status() == 0


def _fill(batch, kv_heads, ctx, dim, seed, outliers=True):
    gen = torch.Generator().manual_seed(seed)
    k = torch.randn(batch, kv_heads, ctx, dim, generator=gen)
    v = torch.randn(batch, kv_heads, ctx, dim, generator=gen)
    if outliers:
        for h in range(kv_heads):
            ch = torch.randperm(dim, generator=gen)[:4]
            k[:, h, :, ch] *= 20.0
    return k, v


@pytest.mark.parametrize("dim,kb,vb,kv_heads,group,ctx", [
    (64, 4, 2, 8, 4, 1024),     # Llama-3.2-1B geometry
    (64, 4, 2, 2, 4, 1),
    (64, 4, 2, 2, 4, 17),
    (64, 4, 2, 2, 1, 333),
    (64, 3, 3, 2, 8, 100),
    (64, 2, 4, 1, 2, 250),
    (128, 4, 3, 8, 4, 700),     # Llama-3-8B geometry
    (128, 4, 4, 2, 4, 65),
    (128, 3, 2, 2, 3, 129),
    (128, 2, 2, 1, 1, 48),
])
def test_fused_decode_matches_dequantise_then_attend(orc, dim, kb, vb, kv_heads, group, ctx):
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig

    batch = 2
    k, v = _fill(batch, kv_heads, ctx, dim, seed=4000 + ctx)
    gen = torch.Generator().manual_seed(99)
    q = torch.randn(batch, kv_heads * group, dim, generator=gen)
    cache = QuantizedKVCache(TurboQuantConfig(key_bits=kb, value_bits=vb, seed=42), num_layers=2, max_seq_len=ctx + 3,
                             num_heads=kv_heads, head_dim=dim, device="cuda", batch_size=batch)
    cache.append(1, k.cuda().bfloat16(), v.cuda().bfloat16())
    out = cache.decode_attention(1, q.cuda().bfloat16())
    assert out.dtype == torch.bfloat16 and out.shape == (batch, kv_heads * group, dim)
    assert cache.decode_status() == 0
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    _, ck = orc.lloyd_max_codebook(kb, dim)
    _, cv = orc.lloyd_max_codebook(vb, dim)
    kp, kn, vp, vn = exported(cache, 1, ctx)
    ref = orc.decode_attention(q.bfloat16().float().numpy(), kp, kn, vp, vn,
                               np.full(batch, ctx, np.int32), rk, ck, kb, rv, cv, vb)
    attention_close(out.float().cpu().numpy(), ref)
    # the cache contents themselves equal the oracle's quantisation of the same bf16 inputs
    kq = k.bfloat16().float().numpy().reshape(-1, dim)
    bk, _ = orc.lloyd_max_codebook(kb, dim)
    o_packed, o_norms = orc.quantize_mse(kq, kb, rk, bk)
    got = kp.reshape(-1, o_packed.shape[1])
    assert (got != o_packed).mean() < 1e-3
    np.testing.assert_allclose(kn.reshape(-1), o_norms, rtol=2e-6)


def test_decode_appends_token_by_token(orc):
    """Prefill, then single-token steps: every step attends over everything appended so far."""
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig

    batch, kv_heads, group, dim = 3, 2, 4, 64
    k, v = _fill(batch, kv_heads, 40, dim, seed=7)
    cache = QuantizedKVCache(TurboQuantConfig(seed=42), 1, 64, kv_heads, dim, device="cuda", batch_size=batch)
    cache.append(0, k[:, :, :30].cuda(), v[:, :, :30].cuda())
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    _, ck = orc.lloyd_max_codebook(4, dim)
    _, cv = orc.lloyd_max_codebook(2, dim)
    gen = torch.Generator().manual_seed(3)
    for step in range(30, 40):
        cache.append(0, k[:, :, step:step + 1].cuda(), v[:, :, step:step + 1].cuda())
        q = torch.randn(batch, kv_heads * group, 1, dim, generator=gen)
        out = cache.decode_attention(0, q.cuda())
        assert out.shape == q.shape
        kp, kn, vp, vn = exported(cache, 0, step + 1)
        ref = orc.decode_attention(q[:, :, 0].numpy(), kp, kn, vp, vn,
                                   np.full(batch, step + 1, np.int32), rk, ck, 4, rv, cv, 2)
        attention_close(out[:, :, 0].cpu().numpy(), ref)


@pytest.mark.parametrize("dim,kb,vb,kv_heads,group,dtype", [
    (64, 4, 2, 8, 4, torch.bfloat16),
    (64, 3, 3, 2, 8, torch.float32),
    (64, 2, 4, 1, 2, torch.float16),
    (128, 4, 3, 4, 4, torch.bfloat16),
    (128, 2, 2, 2, 1, torch.float32),
])
def test_fused_step_equals_append_then_attend(dim, kb, vb, kv_heads, group, dtype):
    """decode_step stores the same bytes and returns the same attention as append + decode_attention."""
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig

    batch, pre, steps = 3, 29, 6
    k, v = _fill(batch, kv_heads, pre + steps, dim, seed=11)
    k, v = k.cuda().to(dtype), v.cuda().to(dtype)
    cfg = TurboQuantConfig(key_bits=kb, value_bits=vb, seed=42)
    two = QuantizedKVCache(cfg, 1, 48, kv_heads, dim, device="cuda", batch_size=batch)
    one = QuantizedKVCache(cfg, 1, 48, kv_heads, dim, device="cuda", batch_size=batch)
    for c in (two, one):
        c.append(0, k[:, :, :pre], v[:, :, :pre])
    gen = torch.Generator().manual_seed(5)
    for step in range(pre, pre + steps):
        q = torch.randn(batch, kv_heads * group, dim, generator=gen).cuda().to(dtype)
        two.append(0, k[:, :, step:step + 1], v[:, :, step:step + 1])
        ref = two.decode_attention(0, q)
        out = one.decode_step(0, q, k[:, :, step], v[:, :, step])
        assert one.decode_status() == 0
        assert int(one.seq_lens[0]) == step + 1
        assert torch.equal(one._seq_lens_dev[0], two._seq_lens_dev[0])
        assert torch.equal(one._store[0], two._store[0]), "fused step stored different record bytes"
        assert torch.equal(out, ref)
    with pytest.raises(RuntimeError, match="overflow"):
        for _ in range(48):
            one.decode_step(0, q, k[:, :, 0], v[:, :, 0])


@pytest.mark.parametrize("dim,kv_heads,group,batch,ctx", [(64, 8, 4, 60, 12000), (128, 8, 4, 60, 6000)])
def test_fused_step_with_several_long_items_per_cta(dim, kv_heads, group, batch, ctx):
    """More than three units per SM, each streamed in many pipeline stages, every one of them receiving a new
    token: the helper warp runs up to two items ahead of the point where the producer needs a unit's new token
    in the store (before the unit's LAST stage).  The step must store the same bytes and return the same
    attention as append + decode_attention, with no bounded wait expiring."""
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig

    steps = 3
    k, v = _fill(batch, kv_heads, ctx + steps, dim, seed=23)
    k, v = k.cuda().bfloat16(), v.cuda().bfloat16()
    cfg = TurboQuantConfig(key_bits=4, value_bits=2 if dim == 64 else 3, seed=42)
    cap = ctx + 16
    two = QuantizedKVCache(cfg, 1, cap, kv_heads, dim, device="cuda", batch_size=batch)
    one = QuantizedKVCache(cfg, 1, cap, kv_heads, dim, device="cuda", batch_size=batch)
    for c in (two, one):
        c.append(0, k[:, :, :ctx], v[:, :, :ctx])
    gen = torch.Generator().manual_seed(6)
    for step in range(ctx, ctx + steps):
        q = torch.randn(batch, kv_heads * group, dim, generator=gen).cuda().bfloat16()
        two.append(0, k[:, :, step:step + 1], v[:, :, step:step + 1])
        ref = two.decode_attention(0, q)
        out = one.decode_step(0, q, k[:, :, step], v[:, :, step])
        assert one.decode_status() == 0 and two.decode_status() == 0
        assert torch.equal(one._store[0], two._store[0]), "fused step stored different record bytes"
        assert torch.equal(out, ref)


def test_more_sequences_than_the_kernel_caches_lengths_for(orc):
    """Beyond 256 sequences the kernel reads lengths from global memory and deals (unit, chunk) items round-robin
    instead of cutting the flattened tile range into equal pieces: same results, ragged and empty sequences."""
    from turboquant_kv.kvstore import PackedKVStore
    from turboquant_kv import _native as N

    batch, kv_heads, group, dim, pitch = 300, 2, 2, 64, 96
    rng = np.random.default_rng(3)
    lens = rng.integers(0, 90, size=batch).astype(np.int32)
    lens[:3] = [0, 89, 16]
    kv = PackedKVStore(dim, 4, 2, 42, "dense_qr", "cuda")
    store = kv.alloc(batch * kv_heads, pitch)
    k, v = _fill(batch, kv_heads, pitch, dim, seed=41)
    kv.append(store, k.cuda(), v.cuda(), N.RowMap(pitch, pitch, 1, 0, None, 1, None, 1))
    q = torch.randn(batch, kv_heads * group, dim, generator=torch.Generator().manual_seed(4))
    seq = torch.from_numpy(lens).cuda()
    out = kv.decode_attention(store, q.cuda(), kv_heads, seq, int(lens.max()), pitch=pitch).cpu().numpy()
    assert kv.status() == 0
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    bk, ck = orc.lloyd_max_codebook(4, dim)
    bv, cv = orc.lloyd_max_codebook(2, dim)
    kp, kn = orc.quantize_mse(k.reshape(-1, dim).numpy(), 4, rk, bk)
    vp, vn = orc.quantize_mse(v.reshape(-1, dim).numpy(), 2, rv, bv)
    ref = orc.decode_attention(q.numpy(), kp.reshape(batch, kv_heads, pitch, -1), kn.reshape(batch, kv_heads, pitch),
                               vp.reshape(batch, kv_heads, pitch, -1), vn.reshape(batch, kv_heads, pitch), lens,
                               rk, ck, 4, rv, cv, 2)
    attention_close(out, ref)
    assert not out[0].any()                                            # the empty sequence


def test_many_long_ragged_sequences_take_equal_pieces_of_the_tile_range(orc):
    """Several units per SM and long contexts: the CTAs then cut the flattened tile range of all units into equal
    pieces (a unit's partials come from up to three CTAs).  Ragged lengths, empty sequences and lengths that
    are no multiple of the tile, against dequantise-then-attend."""
    from turboquant_kv.kvstore import PackedKVStore
    from turboquant_kv import _native as N

    batch, kv_heads, group, dim, pitch = 64, 8, 4, 64, 16016
    rng = np.random.default_rng(9)
    lens = rng.integers(10000, 16001, size=batch).astype(np.int32)
    lens[[0, 5, 63]] = [0, 16000, 1]
    kv = PackedKVStore(dim, 4, 2, 42, "dense_qr", "cuda")
    store = kv.alloc(batch * kv_heads, pitch)
    gen = torch.Generator(device="cuda").manual_seed(10)
    keep = {}
    for b in range(batch):                                               # one sequence at a time: (heads, tokens, dim)
        k = torch.randn(kv_heads, pitch, dim, device="cuda", generator=gen)
        v = torch.randn(kv_heads, pitch, dim, device="cuda", generator=gen)
        k[:, :, 3] *= 20.0
        kv.append(store, k, v, N.RowMap(pitch, pitch, 1, b * kv_heads * pitch, None, 1, None, 1))
        if b in (1, 5, 63):
            keep[b] = (k.cpu().numpy(), v.cpu().numpy())
    q = torch.randn(batch, kv_heads * group, dim, generator=torch.Generator().manual_seed(4))
    out = kv.decode_attention(store, q.cuda(), kv_heads, torch.from_numpy(lens).cuda(), 16000, pitch=pitch).cpu().numpy()
    assert kv.status() == 0
    assert not out[0].any()
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    bk, ck = orc.lloyd_max_codebook(4, dim)
    bv, cv = orc.lloyd_max_codebook(2, dim)
    for b, (k, v) in keep.items():
        l = int(lens[b])
        kp, kn = orc.quantize_mse(k[:, :l].reshape(-1, dim), 4, rk, bk)
        vp, vn = orc.quantize_mse(v[:, :l].reshape(-1, dim), 2, rv, bv)
        ref = orc.decode_attention(q[b:b + 1].numpy(), kp.reshape(1, kv_heads, l, -1), kn.reshape(1, kv_heads, l),
                                   vp.reshape(1, kv_heads, l, -1), vn.reshape(1, kv_heads, l), np.array([l], np.int32),
                                   rk, ck, 4, rv, cv, 2)
        attention_close(out[b:b + 1], ref)


def test_fused_step_replays_in_a_cuda_graph(orc):
    """A captured step keeps appending at the device-side position when the graph is replayed."""
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig

    batch, kv_heads, group, dim, pre = 2, 2, 4, 64, 20
    k, v = _fill(batch, kv_heads, pre + 8, dim, seed=13)
    cache = QuantizedKVCache(TurboQuantConfig(seed=42), 1, 64, kv_heads, dim, device="cuda", batch_size=batch)
    cache.append(0, k[:, :, :pre].cuda(), v[:, :, :pre].cuda())
    qs, ks, vs = (torch.zeros(batch, kv_heads * group, dim, device="cuda"),
                  torch.zeros(batch, kv_heads, dim, device="cuda"), torch.zeros(batch, kv_heads, dim, device="cuda"))
    out = torch.empty_like(qs)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        cache.decode_step(0, qs, ks, vs, out=out)           # warm-up outside capture (sets kernel attributes)
    torch.cuda.current_stream().wait_stream(side)
    cache.seq_lens[0] -= 1
    cache._seq_lens_dev[0] -= 1
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        cache.decode_step(0, qs, ks, vs, out=out)
    cache.seq_lens[0] -= 1                                   # capture does not run the kernels
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    _, ck = orc.lloyd_max_codebook(4, dim)
    _, cv = orc.lloyd_max_codebook(2, dim)
    gen = torch.Generator().manual_seed(17)
    for step in range(pre, pre + 8):
        q = torch.randn(batch, kv_heads * group, dim, generator=gen)
        qs.copy_(q.cuda()); ks.copy_(k[:, :, step].cuda()); vs.copy_(v[:, :, step].cuda())
        graph.replay()
        cache.seq_lens[0] += 1
        torch.cuda.synchronize()
        assert cache._seq_lens_dev[0].tolist() == [step + 1] * batch
        kp, kn, vp, vn = exported(cache, 0, step + 1)
        ref = orc.decode_attention(q.numpy(), kp, kn, vp, vn, np.full(batch, step + 1, np.int32),
                                   rk, ck, 4, rv, cv, 2)
        attention_close(out.cpu().numpy(), ref)
    assert cache.decode_status() == 0


def test_paged_decode_with_ragged_lengths(orc):
    """vLLM-style pools, permuted block tables, different length per sequence, K4/V3 at head_dim 128."""
    from turboquant_kv.vllm_plugin import TurboQuantAttentionImpl, TurboQuantKVCacheConfig, TurboQuantPagedKVCache

    kv_heads, group, dim, bs = 4, 4, 128, 16
    lens = [1, 16, 45, 200]
    batch = len(lens)
    nblocks = sum((l + bs - 1) // bs for l in lens) + 3
    cfg = TurboQuantKVCacheConfig(key_bits=4, value_bits=3, block_size=bs, num_gpu_blocks=nblocks, seed=42)
    pool = TurboQuantPagedKVCache(cfg, num_layers=1, num_heads=kv_heads, head_dim=dim, device="cuda")
    perm = torch.randperm(nblocks, generator=torch.Generator().manual_seed(0)).tolist()
    max_blocks = max((l + bs - 1) // bs for l in lens)
    tables = torch.zeros(batch, max_blocks, dtype=torch.int32)
    gen = torch.Generator().manual_seed(11)
    ks, vs, nxt = [], [], 0
    for b, l in enumerate(lens):
        k = torch.randn(l, kv_heads, dim, generator=gen)
        v = torch.randn(l, kv_heads, dim, generator=gen)
        k[:, :, :4] *= 20.0
        nb = (l + bs - 1) // bs
        blocks = perm[nxt:nxt + nb]
        nxt += nb
        tables[b, :nb] = torch.tensor(blocks, dtype=torch.int32)
        slots = torch.tensor([blocks[t // bs] * bs + t % bs for t in range(l)], dtype=torch.int64)
        # all but the last token are written ahead; the last one goes through forward()
        pool.append_slots(0, k[:-1].cuda(), v[:-1].cuda(), slots[:-1]) if l > 1 else None
        ks.append(k)
        vs.append(v)
    q = torch.randn(batch, kv_heads * group, dim, generator=gen)

    class Meta:
        layer_id = 0
        slot_mapping = torch.tensor([int(tables[b, (l - 1) // bs]) * bs + (l - 1) % bs for b, l in enumerate(lens)])
        block_tables = tables
        seq_lens = torch.tensor(lens, dtype=torch.int32)
        max_seq_len = max(lens)

    impl = TurboQuantAttentionImpl(kv_heads * group, dim, 1.0 / math.sqrt(dim), kv_heads)
    new_k = torch.stack([k[-1] for k in ks])
    new_v = torch.stack([v[-1] for v in vs])
    out = impl.forward(q.cuda(), new_k.cuda(), new_v.cuda(), pool, Meta())
    assert out.shape == (batch, kv_heads * group, dim)
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    bk, ck = orc.lloyd_max_codebook(4, dim)
    bv, cv = orc.lloyd_max_codebook(3, dim)
    for b, l in enumerate(lens):
        kp, kn = orc.quantize_mse(ks[b].transpose(0, 1).reshape(-1, dim).numpy(), 4, rk, bk)
        vp, vn = orc.quantize_mse(vs[b].transpose(0, 1).reshape(-1, dim).numpy(), 3, rv, bv)
        ref = orc.decode_attention(q[b:b + 1].numpy(), kp.reshape(1, kv_heads, l, -1), kn.reshape(1, kv_heads, l),
                                   vp.reshape(1, kv_heads, l, -1), vn.reshape(1, kv_heads, l),
                                   np.array([l], np.int32), rk, ck, 4, rv, cv, 3)
        attention_close(out[b:b + 1].cpu().numpy(), ref)


def test_paged_decode_llama3_8b_geometry_long_context(orc):
    """The paged Llama-3-8B geometry (head_dim 128, K4/V3, 8 KV heads x 4 query heads, 16-token pages) on REAL
    quantised data with thousands of tokens per sequence, pages scattered over the pool by a permutation,
    ragged lengths around page and chunk borders: against dequantise-then-attend on the exported rows."""
    from turboquant_kv.vllm_plugin import TurboQuantKVCacheConfig, TurboQuantPagedKVCache

    kv_heads, group, dim, bs = 8, 4, 128, 16
    lens = [4096, 4611, 4097]
    batch = len(lens)
    nblocks = sum((l + bs - 1) // bs for l in lens) + 5
    cfg = TurboQuantKVCacheConfig(key_bits=4, value_bits=3, block_size=bs, num_gpu_blocks=nblocks, seed=42)
    pool = TurboQuantPagedKVCache(cfg, num_layers=1, num_heads=kv_heads, head_dim=dim, device="cuda")
    gen = torch.Generator().manual_seed(8)
    perm = torch.randperm(nblocks, generator=gen)
    max_blocks = max((l + bs - 1) // bs for l in lens)
    tables = torch.zeros(batch, max_blocks, dtype=torch.int32)
    rows, nxt = [], 0
    for b, l in enumerate(lens):
        nb = (l + bs - 1) // bs
        blocks = perm[nxt:nxt + nb]
        nxt += nb
        tables[b, :nb] = blocks.to(torch.int32)
        k = torch.randn(l, kv_heads, dim, generator=gen)
        v = torch.randn(l, kv_heads, dim, generator=gen)
        for h in range(kv_heads):
            k[:, h, torch.randperm(dim, generator=gen)[:4]] *= 20.0
        t = torch.arange(l)
        slots = blocks[t // bs].to(torch.int64) * bs + t % bs
        pool.append_slots(0, k.cuda().bfloat16(), v.cuda().bfloat16(), slots)
        rows.append((k, v, slots))
    q = torch.randn(batch, kv_heads * group, dim, generator=gen)
    out = pool.paged_decode_attention(0, q.cuda().bfloat16(), tables, torch.tensor(lens, dtype=torch.int32),
                                      max_seq_len=max(lens)).float().cpu().numpy()
    assert pool.kv.status() == 0
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    bk, ck = orc.lloyd_max_codebook(4, dim)
    bv, cv = orc.lloyd_max_codebook(3, dim)
    for b, l in enumerate(lens):
        k, v, _ = rows[b]
        kp, kn = orc.quantize_mse(k.bfloat16().float().transpose(0, 1).reshape(-1, dim).numpy(), 4, rk, bk)
        vp, vn = orc.quantize_mse(v.bfloat16().float().transpose(0, 1).reshape(-1, dim).numpy(), 3, rv, bv)
        ref = orc.decode_attention(q[b:b + 1].bfloat16().float().numpy(), kp.reshape(1, kv_heads, l, -1),
                                   kn.reshape(1, kv_heads, l), vp.reshape(1, kv_heads, l, -1), vn.reshape(1, kv_heads, l),
                                   np.array([l], np.int32), rk, ck, 4, rv, cv, 3)
        attention_close(out[b:b + 1], ref)


@pytest.mark.parametrize("full", [0, 2])          # the full sequence first, or last in the batch
def test_fused_step_on_a_full_unit_reports_it(orc, full):
    """The device-side guard: a sequence already at its pitch stores nothing, keeps its length and raises
    STATUS_UNIT_FULL (wherever it sits in the batch); the other sequences advance normally, and everybody
    attends to what its unit holds."""
    from turboquant_kv.kvstore import STATUS_UNIT_FULL, PackedKVStore
    from turboquant_kv import _native as N

    batch, kv_heads, group, dim, pitch = 3, 2, 4, 64, 32
    kv = PackedKVStore(dim, 4, 2, 42, "dense_qr", "cuda")
    store = kv.alloc(batch * kv_heads, pitch)
    k, v = _fill(batch, kv_heads, pitch, dim, seed=31)
    kv.append(store, k.cuda(), v.cuda(), N.RowMap(pitch, pitch, 1, 0, None, 1, None, 1))
    start = [7, 9, 11]
    start[full] = pitch
    lens = torch.tensor(start, dtype=torch.int32, device="cuda")
    before = store.clone()
    q = torch.randn(batch, kv_heads * group, dim).cuda()
    newk, newv = torch.randn(batch, kv_heads, dim).cuda(), torch.randn(batch, kv_heads, dim).cuda()
    out = kv.decode_step(store, q, newk, newv, kv_heads, lens, pitch, pitch)
    assert kv.status() == STATUS_UNIT_FULL
    assert kv.status() == 0                                                 # reading the status clears it
    want = [l + 1 for l in start]
    want[full] = pitch
    assert lens.tolist() == want
    for b in range(batch):
        units = slice(b * kv_heads, (b + 1) * kv_heads)
        assert torch.equal(store[units], before[units]) == (b == full)      # records of the full sequence untouched
    # every sequence attended to exactly the tokens its unit now holds
    rm = N.RowMap(pitch, pitch, 1, 0, None, 1, None, 1)
    kp, kn, vp, vn = (t.cpu().numpy() for t in kv.export_rows(store, batch * kv_heads * pitch, rm))
    shape = (batch, kv_heads, pitch)
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    _, ck = orc.lloyd_max_codebook(4, dim)
    _, cv = orc.lloyd_max_codebook(2, dim)
    ref = orc.decode_attention(q.cpu().numpy(), kp.reshape(*shape, -1), kn.reshape(shape), vp.reshape(*shape, -1),
                               vn.reshape(shape), np.array(want, np.int32), rk, ck, 4, rv, cv, 2)
    attention_close(out.cpu().numpy(), ref)


def test_stale_host_bound_is_clamped_on_the_device(orc):
    """Lengths live on the device; a max_len the host forgot to raise must not send the kernel past its
    work plan: the sequence is attended up to max_len and STATUS_LEN_CLAMPED is raised.  A negative
    length counts as empty."""
    from turboquant_kv.kvstore import STATUS_LEN_CLAMPED, PackedKVStore
    from turboquant_kv import _native as N

    batch, kv_heads, group, dim, pitch = 3, 2, 4, 64, 128
    kv = PackedKVStore(dim, 4, 2, 42, "dense_qr", "cuda")
    store = kv.alloc(batch * kv_heads, pitch)
    k, v = _fill(batch, kv_heads, pitch, dim, seed=33)
    rm = N.RowMap(pitch, pitch, 1, 0, None, 1, None, 1)
    kv.append(store, k.cuda(), v.cuda(), rm)
    lens = torch.tensor([100, 40, -3], dtype=torch.int32, device="cuda")
    q = torch.randn(batch, kv_heads * group, dim, generator=torch.Generator().manual_seed(5))
    out = kv.decode_attention(store, q.cuda(), kv_heads, lens, 48, pitch=pitch).cpu().numpy()   # 48 < 100
    assert kv.status() == STATUS_LEN_CLAMPED
    kp, kn, vp, vn = (t.cpu().numpy() for t in kv.export_rows(store, batch * kv_heads * pitch, rm))
    shape = (batch, kv_heads, pitch)
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    _, ck = orc.lloyd_max_codebook(4, dim)
    _, cv = orc.lloyd_max_codebook(2, dim)
    ref = orc.decode_attention(q.numpy()[:2], kp.reshape(*shape, -1)[:2], kn.reshape(shape)[:2],
                               vp.reshape(*shape, -1)[:2], vn.reshape(shape)[:2], np.array([48, 40], np.int32),
                               rk, ck, 4, rv, cv, 2)
    attention_close(out[:2], ref)
    assert not out[2].any()
    # the same in a fused step: the position lies beyond max_len, so the token is dropped and the length kept
    lens2 = torch.tensor([100, 40, 5], dtype=torch.int32, device="cuda")
    newk, newv = torch.randn(batch, kv_heads, dim).cuda(), torch.randn(batch, kv_heads, dim).cuda()
    kv.decode_step(store, q.cuda(), newk, newv, kv_heads, lens2, 48, pitch)
    assert kv.status() == STATUS_LEN_CLAMPED
    assert lens2.tolist() == [100, 41, 6]


def test_decode_with_empty_and_ragged_sequences(orc):
    """Sequences of length 0 give zero rows; the others attend over exactly their own tokens."""
    from turboquant_kv.kvstore import PackedKVStore
    from turboquant_kv import _native as N

    kv_heads, group, dim, pitch = 2, 4, 64, 64
    lens = [0, 37, 0, 64, 5]
    batch = len(lens)
    kv = PackedKVStore(dim, 4, 2, 42, "dense_qr", "cuda")
    store = kv.alloc(batch * kv_heads, pitch)
    k, v = _fill(batch, kv_heads, pitch, dim, seed=21)
    rm = N.RowMap(pitch, pitch, 1, 0, None, 1, None, 1)              # row (unit, t) -> slot unit * pitch + t
    kv.append(store, k.cuda(), v.cuda(), rm)
    q = torch.randn(batch, kv_heads * group, dim, generator=torch.Generator().manual_seed(4))
    seq = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = kv.decode_attention(store, q.cuda(), kv_heads, seq, max(lens), pitch=pitch).cpu().numpy()
    assert kv.status() == 0
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    bk, ck = orc.lloyd_max_codebook(4, dim)
    bv, cv = orc.lloyd_max_codebook(2, dim)
    for b, l in enumerate(lens):
        if l == 0:
            assert not out[b].any()
            continue
        kp, kn = orc.quantize_mse(k[b, :, :l].reshape(-1, dim).numpy(), 4, rk, bk)
        vp, vn = orc.quantize_mse(v[b, :, :l].reshape(-1, dim).numpy(), 2, rv, bv)
        ref = orc.decode_attention(q[b:b + 1].numpy(), kp.reshape(1, kv_heads, l, -1), kn.reshape(1, kv_heads, l),
                                   vp.reshape(1, kv_heads, l, -1), vn.reshape(1, kv_heads, l),
                                   np.array([l], np.int32), rk, ck, 4, rv, cv, 2)
        attention_close(out[b:b + 1], ref)
    # nothing to attend to at all: every row is zero
    none = kv.decode_attention(store, q.cuda(), kv_heads, torch.zeros(batch, dtype=torch.int32, device="cuda"), 0,
                               pitch=pitch)
    assert not none.cpu().numpy().any()


def test_protected_layers_and_upstream_cache_checks():
    """The behaviours upstream tests/test_cache.py pins: incremental lengths, compression ratio in (3, 10),
    fp16-exact protected layers, outlier_channels accepted."""
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig

    cfg = TurboQuantConfig(key_bits=4, value_bits=2, protected_layers=1, outlier_channels=4)
    cache = QuantizedKVCache(cfg, num_layers=2, max_seq_len=128, num_heads=4, head_dim=64, device="cuda")
    assert cache._has_outliers
    k, v = torch.randn(4, 10, 64, device="cuda"), torch.randn(4, 10, 64, device="cuda")
    for layer in (0, 1):
        cache.append(layer, k, v)
        cache.append(layer, k[:, :5], v[:, :5])
    assert cache.seq_lens.tolist() == [15, 15]
    q = torch.randn(4, 1, 64, device="cuda")
    exact = torch.matmul(q, torch.cat([k, k[:, :5]], 1).half().float().transpose(-2, -1)) / 8.0
    assert torch.allclose(cache.attention_scores(0, q), exact, atol=1e-3)
    approx = cache.attention_scores(1, q)
    assert torch.corrcoef(torch.stack([approx.flatten(), exact.flatten()]))[0, 1] > 0.8
    only_q = QuantizedKVCache(TurboQuantConfig(), 1, 128, 4, 64, device="cuda")
    only_q.append(0, k, v)
    assert 3 < only_q.compression_ratio < 10 and only_q.memory_bytes() > 0
    with pytest.raises(RuntimeError):
        QuantizedKVCache(TurboQuantConfig(mode="prod"), 1, 16, 2, 64, device="cuda").append(0, k[:2], v[:2])


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("kb,vb", [(4, 2), (4, 3), (4, 4), (3, 3), (2, 2), (3, 2), (2, 4)])
def test_record_store_export_import_roundtrip(orc, dim, kb, vb):
    """Upstream rows -> records -> upstream rows is the identity, at ragged positions, and what append()
    stores equals the oracle's quantisation of the same inputs."""
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig

    rng = np.random.default_rng(dim + kb * 10 + vb)
    B, H, seq = 2, 3, 37
    cache = QuantizedKVCache(TurboQuantConfig(key_bits=kb, value_bits=vb, seed=42), 1, 50, H, dim, device="cuda", batch_size=B)
    kp = rng.integers(0, 256, size=(B, H, seq, kb * dim // 8), dtype=np.uint8)
    vp = rng.integers(0, 256, size=(B, H, seq, vb * dim // 8), dtype=np.uint8)
    kn = rng.random(size=(B, H, seq)).astype(np.float32)
    vn = rng.random(size=(B, H, seq)).astype(np.float32)
    cache.load_packed(0, cuda(kp), cuda(kn), cuda(vp), cuda(vn))
    assert int(cache.seq_lens[0]) == seq
    g_kp, g_kn, g_vp, g_vn = exported(cache, 0, seq)
    assert np.array_equal(g_kp, kp) and np.array_equal(g_vp, vp)
    assert np.array_equal(g_kn, kn) and np.array_equal(g_vn, vn)
    # overwrite in place (the clear-then-set path) and append behind it
    cache.load_packed(0, cuda(255 - kp), cuda(kn), cuda(255 - vp), cuda(vn))
    g_kp, _, g_vp, _ = exported(cache, 0, seq)
    assert np.array_equal(g_kp, 255 - kp) and np.array_equal(g_vp, 255 - vp)
    k = torch.randn(B, H, 5, dim, generator=torch.Generator().manual_seed(1))
    v = torch.randn(B, H, 5, dim, generator=torch.Generator().manual_seed(2))
    cache.append(0, k.cuda(), v.cuda())
    g_kp, g_kn, g_vp, g_vn = exported(cache, 0, seq + 5)
    assert np.array_equal(g_kp[:, :, :seq], 255 - kp)
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    bk, _ = orc.lloyd_max_codebook(kb, dim)
    bv, _ = orc.lloyd_max_codebook(vb, dim)
    o_kp, o_kn = orc.quantize_mse(k.numpy().reshape(-1, dim), kb, rk, bk)
    o_vp, o_vn = orc.quantize_mse(v.numpy().reshape(-1, dim), vb, rv, bv)
    assert (g_kp[:, :, seq:].reshape(o_kp.shape) != o_kp).mean() < 2e-3
    assert (g_vp[:, :, seq:].reshape(o_vp.shape) != o_vp).mean() < 2e-3
    np.testing.assert_allclose(g_kn[:, :, seq:].reshape(-1), o_kn, rtol=2e-6)
    np.testing.assert_allclose(g_vn[:, :, seq:].reshape(-1), o_vn, rtol=2e-6)
