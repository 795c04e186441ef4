"""GPU parity of the tensor-parallel cache: KV heads split over tp_size ranks (upstream
turboquant_kv/distributed.py:80-106), no collective on the attention path.  The ranks are emulated on one
GPU: every rank's DistributedQuantizedKVCache gets the slice of keys, values and queries a tensor-parallel
attention layer would hand it, and the concatenation of the ranks' outputs must be the unsharded answer."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from util import attention_close

pytestmark = pytest.mark.gpu


def _inputs(batch, kv_heads, group, ctx, dim, seed):
    gen = torch.Generator().manual_seed(seed)
    k = torch.randn(batch, kv_heads, ctx, dim, generator=gen)
    v = torch.randn(batch, kv_heads, ctx, dim, generator=gen)
    for h in range(kv_heads):
        k[:, h, :, torch.randperm(dim, generator=gen)[:4]] *= 20.0
    q = torch.randn(batch, kv_heads * group, dim, generator=gen)
    return k.cuda().bfloat16(), v.cuda().bfloat16(), q.cuda().bfloat16()


@pytest.mark.parametrize("tp_size,ctx", [(2, 300), (4, 300), (2, 3000)])
def test_head_sharded_cache_equals_the_unsharded_cache(orc, tp_size, ctx):
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig
    from turboquant_kv.distributed import DistributedQuantizedKVCache

    batch, kv_heads, group, dim = 3, 8, 4, 64
    cfg = TurboQuantConfig(key_bits=4, value_bits=2, seed=42)
    k, v, q = _inputs(batch, kv_heads, group, ctx, dim, seed=ctx + tp_size)
    whole = QuantizedKVCache(cfg, 1, ctx + 8, kv_heads, dim, device="cuda", batch_size=batch)
    whole.append(0, k, v)
    want = whole.decode_attention(0, q)
    assert whole.decode_status() == 0
    parts = []
    for rank in range(tp_size):
        shard = DistributedQuantizedKVCache.from_config(cfg, tp_size, rank, 1, ctx + 8, kv_heads, dim, device="cuda",
                                                        batch_size=batch)
        hs = shard.head_slice()
        assert shard.local_num_heads == kv_heads // tp_size and hs == slice(rank * kv_heads // tp_size,
                                                                             (rank + 1) * kv_heads // tp_size)
        shard.append(0, k[:, hs], v[:, hs])
        assert int(shard.seq_lens[0]) == ctx
        # the records of the rank's heads are exactly those of the unsharded cache
        B = batch
        assert torch.equal(shard.cache._store[0].view(B, shard.local_num_heads, -1),
                           whole._store[0].view(B, kv_heads, -1)[:, hs])
        qs = slice(hs.start * group, hs.stop * group)
        parts.append(shard.decode_attention(0, q[:, qs]))
        assert shard.cache.decode_status() == 0
        assert shard.memory_bytes() * tp_size == whole.memory_bytes()
    got = torch.cat(parts, dim=1)
    # the CTAs cut the flattened tile range of ALL units into equal pieces, so a shard (fewer units) splits its
    # sequences at other places than the unsharded cache and the partials merge in another order: the outputs
    # agree to bf16 rounding, not bit for bit
    np.testing.assert_allclose(got.float().cpu().numpy(), want.float().cpu().numpy(), atol=2e-2, rtol=0)
    assert (got != want).float().mean() < 0.05                         # bf16 roundings that fell the other way
    # and both agree with dequantise-then-attend
    kp, kn, vp, vn = (t.cpu().numpy() for t in whole._export(0, ctx))
    shape = (batch, kv_heads, ctx)
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    _, ck = orc.lloyd_max_codebook(4, dim)
    _, cv = orc.lloyd_max_codebook(2, dim)
    ref = orc.decode_attention(q.float().cpu().numpy(), kp.reshape(*shape, -1), kn.reshape(shape),
                               vp.reshape(*shape, -1), vn.reshape(shape), np.full(batch, ctx, np.int32),
                               rk, ck, 4, rv, cv, 2)
    attention_close(got.float().cpu().numpy(), ref)


def test_head_sharded_fused_step(orc):
    """decode_step through the sharded cache: both ranks append and attend; lengths and records advance together."""
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig
    from turboquant_kv.distributed import DistributedQuantizedKVCache

    batch, kv_heads, group, dim, ctx = 2, 4, 4, 64, 40
    cfg = TurboQuantConfig(key_bits=4, value_bits=2, seed=42)
    k, v, q = _inputs(batch, kv_heads, group, ctx + 1, dim, seed=5)
    whole = QuantizedKVCache(cfg, 1, 64, kv_heads, dim, device="cuda", batch_size=batch)
    whole.append(0, k[:, :, :ctx], v[:, :, :ctx])
    want = whole.decode_step(0, q, k[:, :, ctx], v[:, :, ctx])
    parts = []
    for rank in range(2):
        shard = DistributedQuantizedKVCache.from_config(cfg, 2, rank, 1, 64, kv_heads, dim, device="cuda", batch_size=batch)
        hs = shard.head_slice()
        shard.append(0, k[:, hs, :ctx], v[:, hs, :ctx])
        parts.append(shard.decode_step(0, q[:, hs.start * group:hs.stop * group], k[:, hs, ctx], v[:, hs, ctx]))
        assert int(shard.seq_lens[0]) == ctx + 1 and shard.cache._seq_lens_dev[0].tolist() == [ctx + 1] * batch
        assert torch.equal(shard.cache._store[0].view(batch, 2, -1), whole._store[0].view(batch, kv_heads, -1)[:, hs])
    assert torch.equal(torch.cat(parts, dim=1), want)
