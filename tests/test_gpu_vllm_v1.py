"""GPU parity of the vLLM v1 attention backend adapter (turboquant_kv/vllm_plugin/v1_backend.py): prefill,
decode and mixed batches through ``AttentionImpl.forward`` with hand-built ``CommonAttentionMetadata``,
checked against the oracle's dequantise-then-attend on the oracle's own quantisation of the same K/V."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from util import attention_close

pytestmark = pytest.mark.gpu

v1 = pytest.importorskip("turboquant_kv.vllm_plugin.v1_backend", reason="vLLM's v1 attention interface is not installed")


def _common(query_lens, seq_lens, tables, slots, device):
    from vllm.v1.attention.backend import CommonAttentionMetadata

    qsl = torch.tensor([0] + list(np.cumsum(query_lens)), dtype=torch.int32)
    return CommonAttentionMetadata(
        query_start_loc=qsl.to(device), query_start_loc_cpu=qsl, seq_lens=torch.tensor(seq_lens, dtype=torch.int32).to(device),
        num_reqs=len(query_lens), num_actual_tokens=int(sum(query_lens)), max_query_len=int(max(query_lens)),
        max_seq_len=int(max(seq_lens)), block_table_tensor=tables.to(device), slot_mapping=slots.to(device), causal=True)


@pytest.mark.parametrize("dim,kb,vb", [(64, 4, 2), (128, 4, 3)])
def test_v1_backend_prefill_decode_and_mixed_batches(orc, dim, kb, vb):
    B = v1.TurboQuantV1Backend
    B.configure(key_bits=kb, value_bits=vb, seed=42)
    try:
        kvh, group, bs, dev = 2, 4, 16, torch.device("cuda")
        H = kvh * group
        lens = [37, 5, 64]                                  # prompt lengths
        nblocks = sum((l + 8 + bs - 1) // bs for l in lens) + 2
        shape = B.get_kv_cache_shape(nblocks, bs, kvh, dim)
        cache = torch.zeros(shape, dtype=torch.uint8, device=dev)
        perm = torch.randperm(nblocks, generator=torch.Generator().manual_seed(3)).tolist()
        max_blocks = max((l + 8 + bs - 1) // bs for l in lens)
        tables = torch.zeros(len(lens), max_blocks, dtype=torch.int32)
        nxt = 0
        for r, l in enumerate(lens):
            nb = (l + 8 + bs - 1) // bs
            tables[r, :nb] = torch.tensor(perm[nxt:nxt + nb], dtype=torch.int32)
            nxt += nb
        slot = lambda r, t: int(tables[r, t // bs]) * bs + t % bs
        gen = torch.Generator().manual_seed(5)
        total = [l + 3 for l in lens]                       # prompt + 3 generated tokens
        K = [torch.randn(t, kvh, dim, generator=gen) for t in total]
        V = [torch.randn(t, kvh, dim, generator=gen) for t in total]
        Q = [torch.randn(t, H, dim, generator=gen) for t in total]
        for k in K:
            k[:, :, :4] *= 20.0
        impl = B.get_impl_cls()(H, dim, 1.0 / math.sqrt(dim), kvh)
        builder = B.get_builder_cls()(None, ["layer.0"], None, dev)
        rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
        bk, ck = orc.lloyd_max_codebook(kb, dim)
        bv, cv = orc.lloyd_max_codebook(vb, dim)

        def reference(r, t):
            """Attention of token t of request r over tokens 0..t (oracle quantisation of the same rows)."""
            n = t + 1
            kp, kn = orc.quantize_mse(K[r][:n].transpose(0, 1).reshape(-1, dim).numpy(), kb, rk, bk)
            vp, vn = orc.quantize_mse(V[r][:n].transpose(0, 1).reshape(-1, dim).numpy(), vb, rv, bv)
            return orc.decode_attention(Q[r][t:t + 1].numpy(), kp.reshape(1, kvh, n, -1), kn.reshape(1, kvh, n),
                                        vp.reshape(1, kvh, n, -1), vn.reshape(1, kvh, n), np.array([n], np.int32),
                                        rk, ck, kb, rv, cv, vb)

        def run(ranges):
            """ranges[r] = (t0, t1): request r contributes tokens t0..t1-1 this step."""
            act = [(r, a, b) for r, (a, b) in enumerate(ranges) if b > a]
            q = torch.cat([Q[r][a:b] for r, a, b in act]).cuda().view(-1, H * dim)
            k = torch.cat([K[r][a:b] for r, a, b in act]).cuda().view(-1, kvh * dim)
            v = torch.cat([V[r][a:b] for r, a, b in act]).cuda().view(-1, kvh * dim)
            slots = torch.tensor([slot(r, t) for r, a, b in act for t in range(a, b)], dtype=torch.int64)
            md = builder.build(0, _common([b - a for _, a, b in act], [b for _, _, b in act],
                                          tables[[r for r, _, _ in act]], slots, dev))
            out = impl.forward(None, q, k, v, cache, md, output=torch.empty_like(q)).view(-1, H, dim).cpu().numpy()
            i = 0
            for r, a, b in act:
                for t in range(a, b):
                    if t in (a, b - 1) or t % 7 == 0:       # first, last and a few inner tokens of every request
                        attention_close(out[i:i + 1], reference(r, t))
                    i += 1

        run([(0, 20), (0, 5), (0, 64)])                     # prefill (request 0 only its first chunk)
        run([(20, 37), (5, 6), (64, 65)])                   # mixed: chunked prefill + two decodes
        run([(37, 38), (6, 7), (65, 66)])                   # pure decode batch -> fused paged kernel
        run([(38, 40), (7, 8), (66, 67)])                   # a two-token query (speculative verification shape)
        # oversized expansions take several launches (here: one per query token) and give the same answers
        K2 = [k.clone() for k in K]
        impl.MAX_EXPANDED_TABLE = 0
        cache.zero_()
        run([(0, 20), (0, 5), (0, 64)])
        run([(20, 37), (5, 6), (64, 65)])
        assert all(torch.equal(a, b) for a, b in zip(K, K2))
    finally:
        B.configure()
