"""GPU parity of the tensor-core quantiser (csrc/quantize_tc.cu): large calls of tqb_quantize_mse /
tqb_kv_append run on tcgen05 with bf16 operand splits and an exact re-quantisation of rows near a decision
boundary.  Bar: the very same bytes as the float32 FFMA kernel (reached here by feeding it the rows in
batches below the tensor-core threshold), and the oracle's codes except at exact ties."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from util import MAX_TIE_RATE, code_mismatches

pytestmark = pytest.mark.gpu

SMALL = 256     # rows per call that stay on the FFMA kernel (the tensor-core path starts at 512)


def _rows(n, dim, dtype, seed, outliers=True):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(n, dim, generator=gen)
    if outliers:
        x[:, torch.randperm(dim, generator=gen)[:4]] *= 20.0
    x[::7] *= 0.01                      # a spread of norms
    x[5] = 0.0                          # a zero row (norm 0)
    return x.to(dtype).cuda()


def _status():
    from turboquant_kv import _native as N

    return N.lib().tqb_quantize_status(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("dim,bits", [(128, 4), (128, 3), (128, 2), (64, 4), (64, 3), (64, 2)])
def test_tensor_core_quantise_equals_ffma_kernel_and_oracle(orc, dtype, dim, bits):
    import turboquant_kv.reference as R

    n = 4 * 1024 + 3                    # 33 tiles, the last one ragged
    x = _rows(n, dim, dtype, seed=dim + bits)
    rot = orc.make_rotation_matrix(dim, 42)
    bnd, cent = orc.lloyd_max_codebook(bits, dim)
    cb = (torch.from_numpy(bnd).cuda(), torch.from_numpy(cent).cuda())
    rot_d = torch.from_numpy(rot).cuda()
    packed, norms = R.quantize_mse(x, bits, rotation=rot_d, codebook=cb)              # one large call
    assert _status() == 0, "a bounded wait of the tensor-core kernel expired"
    parts = [R.quantize_mse(x[lo:lo + SMALL], bits, rotation=rot_d, codebook=cb) for lo in range(0, n, SMALL)]
    packed_f = torch.cat([p[0] for p in parts])
    norms_f = torch.cat([p[1] for p in parts])
    assert torch.equal(norms, norms_f), "norms differ from the FFMA kernel"
    diff = (packed != packed_f).any(dim=1)
    assert not diff.any(), f"{int(diff.sum())} rows differ from the FFMA kernel, first {diff.nonzero()[:5].flatten().tolist()}"
    o_packed, o_norms, rotated = orc.quantize_mse(x.float().cpu().numpy(), bits, rot, bnd, return_rotated=True)
    rate, _ = code_mismatches(orc, packed.cpu().numpy(), o_packed, rotated, bnd, bits, dim)
    assert rate <= 1e-4                 # (a few thousand rows: a single tie is already 2e-6)
    np.testing.assert_allclose(norms.float().cpu().numpy(), o_norms, rtol=2e-6)


def test_tensor_core_quantise_full_c1_config(orc):
    """65,536 unit vectors of dim 128 at 4 bits (the quantise round-trip configuration): tie-only mismatches at
    a rate <= 1e-5 against the oracle."""
    import turboquant_kv.reference as R

    g = torch.Generator().manual_seed(0)
    x = torch.randn(65536, 128, generator=g)
    x = x / x.norm(dim=-1, keepdim=True)
    rot = orc.make_rotation_matrix(128, 42)
    bnd, cent = orc.lloyd_max_codebook(4, 128)
    packed, norms = R.quantize_mse(x.cuda(), 4, rotation=torch.from_numpy(rot).cuda(),
                                   codebook=(torch.from_numpy(bnd).cuda(), torch.from_numpy(cent).cuda()))
    assert _status() == 0
    o_packed, o_norms, rotated = orc.quantize_mse(x.numpy(), 4, rot, bnd, return_rotated=True)
    rate, worst = code_mismatches(orc, packed.cpu().numpy(), o_packed, rotated, bnd, 4, 128)
    assert rate <= MAX_TIE_RATE, f"mismatch rate {rate:.2e}"
    np.testing.assert_allclose(norms.cpu().numpy(), o_norms, rtol=2e-6)


@pytest.mark.parametrize("dim,kb,vb", [(64, 4, 2), (128, 4, 3), (128, 3, 4)])
def test_tensor_core_append_writes_the_same_records(dim, kb, vb):
    """tqb_kv_append of thousands of tokens (tensor cores) fills the record store exactly like appends of a few
    hundred tokens at a time (FFMA kernel)."""
    from turboquant_kv import _native as N
    from turboquant_kv.kvstore import PackedKVStore

    units, tokens = 6, 700              # rows are (unit, token): 4,200 rows per call
    kv = PackedKVStore(dim, kb, vb, 42, "dense_qr", "cuda")
    k = _rows(units * tokens, dim, torch.bfloat16, seed=1).view(units, tokens, dim)
    v = _rows(units * tokens, dim, torch.bfloat16, seed=2, outliers=False).view(units, tokens, dim)
    pitch = 704
    big, small = kv.alloc(units, pitch), kv.alloc(units, pitch)
    kv.append(big, k, v, N.RowMap(tokens, pitch, 1, 0, None, 1, None, 1))
    assert _status() == 0
    for lo in range(0, tokens, 40):     # 6 x 40 = 240 rows per call
        hi = min(tokens, lo + 40)
        kv.append(small, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(), N.RowMap(hi - lo, pitch, 1, lo, None, 1, None, 1))
    torch.cuda.synchronize()
    assert torch.equal(big, small)


@pytest.mark.parametrize("heads", [8, 4, 2, 1, 3])
@pytest.mark.parametrize("dim,kb,vb", [(128, 4, 3), (64, 3, 2), (128, 2, 4)])
def test_tensor_core_paged_append_writes_the_same_records(dim, kb, vb, heads):
    """append_slots of thousands of tokens (rows = token x head, pages scattered over the pool): whole pages
    are written as whole records by the tensor-core kernel, ragged starts, skipped tokens (slot -1) and head
    counts that do not tile a 128-row tile go row by row; either way the pool equals the one filled by appends
    of a few dozen tokens at a time (FFMA kernel)."""
    from turboquant_kv.vllm_plugin import TurboQuantKVCacheConfig, TurboQuantPagedKVCache

    bs, lens, starts = 16, [1500, 333, 2048, 40], [0, 5, 16, 0]      # tokens per sequence, position of the first one
    nblocks = sum((st + l + bs - 1) // bs for l, st in zip(lens, starts)) + 3
    gen = torch.Generator().manual_seed(heads * 100 + dim + kb)
    perm = torch.randperm(nblocks, generator=gen)
    pools = []
    for _ in range(2):
        cfg = TurboQuantKVCacheConfig(key_bits=kb, value_bits=vb, block_size=bs, num_gpu_blocks=nblocks, seed=42)
        pools.append(TurboQuantPagedKVCache(cfg, num_layers=1, num_heads=heads, head_dim=dim, device="cuda"))
    slots, nxt = [], 0
    for l, st in zip(lens, starts):
        nb = (st + l + bs - 1) // bs
        blocks = perm[nxt:nxt + nb].to(torch.int64)
        nxt += nb
        t = torch.arange(st, st + l)
        slots.append(blocks[t // bs] * bs + t % bs)
    slots = torch.cat(slots)
    slots[777] = -1                                                   # padding tokens are skipped
    slots[1000:1003] = -1
    T = slots.numel()
    k = _rows(T * heads, dim, torch.bfloat16, seed=5).view(T, heads, dim)
    v = _rows(T * heads, dim, torch.bfloat16, seed=6, outliers=False).view(T, heads, dim)
    pools[0].append_slots(0, k, v, slots)                             # T x heads rows at once
    assert _status() == 0
    step = max(1, 200 // heads)
    for lo in range(0, T, step):                                      # at most 200 rows per call
        pools[1].append_slots(0, k[lo:lo + step].contiguous(), v[lo:lo + step].contiguous(), slots[lo:lo + step])
    torch.cuda.synchronize()
    assert torch.equal(pools[0]._pools[0], pools[1]._pools[0])


def test_tensor_core_quantise_strided_rows(orc):
    """Rows that are not contiguous (x_stride > dim) go through one TMA copy per row."""
    from turboquant_kv import _native as N

    n, dim, bits, stride = 2048, 128, 4, 160
    buf = torch.randn(n, stride, generator=torch.Generator().manual_seed(3)).cuda()
    rot = torch.from_numpy(orc.make_rotation_matrix(dim, 42)).cuda()
    bnd, _ = orc.lloyd_max_codebook(bits, dim)
    bnd_d = torch.from_numpy(bnd).cuda()
    L = N.lib()
    st = torch.cuda.current_stream().cuda_stream
    outs = []
    for src, sstride in ((buf, stride), (buf[:, :dim].contiguous(), dim)):
        packed = torch.empty(n, bits * dim // 8, dtype=torch.uint8, device="cuda")
        norms = torch.empty(n, device="cuda")
        N.check(L.tqb_quantize_mse(src.data_ptr(), 0, n, dim, sstride, rot.data_ptr(), bnd_d.data_ptr(), bits,
                                   packed.data_ptr(), norms.data_ptr(), None, st))
        outs.append((packed, norms))
    torch.cuda.synchronize()
    assert _status() == 0
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
