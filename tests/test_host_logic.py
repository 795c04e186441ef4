"""CPU-only tests: host-side constant generators, the C-ABI surface, bookkeeping that needs no kernel,
and the multi-process gather/merge logic on gloo ranks."""
from __future__ import annotations

import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tqb200.h")
LIB = os.path.join(ROOT, "turboquant-kv_b200", "turboquant_kv", "libtqb200.so")


def test_host_constants_match_upstream(golden):
    """Codebooks, rotations and the QJL matrix are generated in Python; they must equal the upstream ones."""
    import turboquant_kv.reference as R

    g = golden("constants")
    for bits in (1, 2, 3, 4):
        for dim in (64, 128):
            b, c = R.lloyd_max_codebook(bits, dim)
            assert np.array_equal(b.numpy(), g[f"boundaries_b{bits}_d{dim}"])
            assert np.array_equal(c.numpy(), g[f"centroids_b{bits}_d{dim}"])
    for dim, seed in ((64, 42), (64, 43), (128, 42), (32, 7)):
        assert np.array_equal(R.make_rotation_matrix(dim, seed).numpy(), g[f"rotation_qr_d{dim}_s{seed}"])
    assert np.allclose(R.make_rotation_matrix(64, 42, "rht").numpy(), g["rotation_rht_d64_s42"], atol=1e-6)
    assert np.allclose(R.make_rht_rotation(48, 5).numpy(), g["rotation_rht_d48_s5"], atol=1e-6)
    for dim in (64, 128):
        assert np.array_equal(R._make_qjl_matrix(dim, dim, 42, "cpu").numpy(), g[f"qjl_d{dim}_s42"])
    with pytest.raises(ValueError):
        R.make_rotation_matrix(8, 1, "nope")


def test_codebook_properties():
    """What upstream tests/test_reference.py checks of the codebook: analytic 1-bit value, counts, order, symmetry."""
    import turboquant_kv.reference as R

    for d in (64, 128, 256):
        b, c = R.lloyd_max_codebook(1, d)
        assert abs(float(c[1]) - np.sqrt(2 / np.pi) / np.sqrt(d)) < 1e-4 and abs(float(c[0]) + float(c[1])) < 1e-7
    for bits in (1, 2, 3, 4):
        b, c = R.lloyd_max_codebook(bits, 128)
        assert b.shape == ((1 << bits) - 1,) and c.shape == (1 << bits,)
        assert torch.all(c[1:] > c[:-1]) and torch.all(b[1:] > b[:-1])
        assert torch.allclose(c, -c.flip(0), atol=1e-6)
    rot = R.make_rotation_matrix(128, 42)
    assert torch.allclose(rot @ rot.t(), torch.eye(128), atol=1e-5)
    assert torch.equal(rot, R.make_rotation_matrix(128, 42)) and not torch.equal(rot, R.make_rotation_matrix(128, 43))


def test_library_exports_every_declared_symbol():
    """libtqb200.so loads without a GPU and exports exactly the entry points include/tqb200.h declares."""
    sys.path.insert(0, os.path.join(ROOT, "turboquant-kv_b200", "csrc"))
    import build as native_build

    native_build.build()
    declared = set(re.findall(r"\b(tqb_[a-z0-9_]+)\s*\(", open(HEADER).read()))
    assert len(declared) >= 17
    lib = ctypes.CDLL(LIB)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in tqb200.h but not exported"
    lib.tqb_abi_version.restype = ctypes.c_int
    assert lib.tqb_abi_version() == 2
    out = subprocess.run(["nm", "-D", "--defined-only", LIB], capture_output=True, text=True).stdout
    exported = set(re.findall(r" T (tqb_[a-z0-9_]+)", out))
    assert exported == declared, exported ^ declared


def test_argument_errors_need_no_gpu():
    """Validation happens before any CUDA call: error codes and messages come back through the C ABI."""
    lib = ctypes.CDLL(LIB)
    lib.tqb_last_error.restype = ctypes.c_char_p
    assert lib.tqb_pack_codes(None, ctypes.c_int64(4), 64, 9, None, None) == -1
    assert b"bit_width must be 1-8" in lib.tqb_last_error()
    assert lib.tqb_pack_codes(None, ctypes.c_int64(0), 64, 4, None, None) == 0        # empty input: no launch
    lib.tqb_scan_topk_workspace_bytes.restype = ctypes.c_size_t
    lib.tqb_scan_topk_workspace_bytes.argtypes = [ctypes.c_int, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    assert lib.tqb_scan_topk_workspace_bytes(4, 1000, 128, 4, 10) > 0
    assert lib.tqb_scan_topk_workspace_bytes(4, 1000, 128, 4, 100000) == 0


def test_no_cpu_fallback():
    """Without CUDA the product refuses to compute instead of falling back to anything."""
    if torch.cuda.is_available():
        pytest.skip("this check is for GPU-less machines")
    import turboquant_kv as tq

    with pytest.raises(RuntimeError, match="CUDA"):
        tq.quantize_mse(torch.randn(4, 64), 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        tq.TurboQuantIndex(dim=64)
    with pytest.raises(RuntimeError, match="CUDA"):
        tq.QuantizedKVCache(tq.TurboQuantConfig(), 1, 16, 2, 64)


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "turboquant-kv_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "oracle" not in text.replace("the oracle", ""), f"{f} mentions the oracle folder"


def test_config_and_sharding_bookkeeping():
    from turboquant_kv import TurboQuantConfig
    from turboquant_kv.distributed import DistributedQuantizedKVCache, shard_rows
    from turboquant_kv.vllm_plugin import TurboQuantAttentionBackend, TurboQuantKVCacheConfig

    c = TurboQuantConfig()
    assert (c.key_bits, c.value_bits, c.mode, c.rotation, c.outlier_channels, c.protected_layers,
            c.quantize_on_append, c.block_size, c.seed) == (4, 2, "mse", "dense_qr", 0, 0, True, 0, 42)
    spans = [shard_rows(10_000_003, 8, r) for r in range(8)]
    assert spans[0][0] == 0 and spans[-1][1] == 10_000_003
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert max(e - b for b, e in spans) - min(e - b for b, e in spans) <= 1
    with pytest.raises(ValueError):
        DistributedQuantizedKVCache(c, 1, 16, 6, 64, tp_size=4)
    with pytest.raises(ValueError):
        DistributedQuantizedKVCache(c, 1, 16, 8, 64, tp_size=4, tp_rank=4)
    v = TurboQuantKVCacheConfig(key_bits=3, seed=5).to_turboquant_config()
    assert v.key_bits == 3 and v.seed == 5 and v.quantize_on_append
    assert TurboQuantAttentionBackend.get_name() == "turboquant"
    assert TurboQuantAttentionBackend.get_kv_cache_shape(7, 16, 8, 128) == (2, 7, 16, 8, 128)


def test_merge_topk_host_path_orders_by_score_then_id():
    from turboquant_kv.search import merge_topk

    s = torch.tensor([[[5.0, 3.0, 1.0], [5.0, 4.0, float("-inf")]]])
    i = torch.tensor([[[7, 2, 9], [3, 8, -1]]])
    ms, mi = merge_topk(s, i, 3)
    assert mi.tolist() == [[3, 7, 8]] and ms.tolist() == [[5.0, 5.0, 4.0]]
    ms, mi = merge_topk(s, i, 6)
    assert mi.tolist() == [[3, 7, 8, 2, 9, -1]] and ms[0, -1] == float("-inf")


_GLOO_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from turboquant_kv.distributed import gather_and_merge, shard_rows
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
# a fake "database" of scores: every rank owns a contiguous row range and reports its local top-k
g = torch.Generator().manual_seed(123)
Q, N, k = 5, 1001, 10
scores = torch.randn(Q, N, generator=g)
scores[:, 17] = scores[:, 600]           # an exact tie across shards: the lower id must win
lo, hi = shard_rows(N, world, rank)
ls, li = torch.topk(scores[:, lo:hi], k, dim=1)
ms, mi = gather_and_merge(ls, li + lo, k)
ws, wi = torch.topk(scores, k, dim=1)
assert torch.equal(ms, ws), (rank, ms, ws)
for q in range(Q):
    assert sorted(mi[q].tolist()) == sorted(wi[q].tolist())
    row = mi[q].tolist()
    if 17 in row and 600 in row:
        assert row.index(17) < row.index(600)
# a shard that holds fewer than k rows pads with (-inf, -1)
short = 3 if rank == 0 else k
ls2 = torch.full((Q, k), float("-inf")); li2 = torch.full((Q, k), -1, dtype=torch.int64)
ls2[:, :short], li2[:, :short] = ls[:, :short], (li + lo)[:, :short]
ms2, mi2 = gather_and_merge(ls2, li2, k)
assert (mi2 >= 0).all() and torch.isfinite(ms2).all()
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


@pytest.mark.timeout(300)
def test_row_sharded_merge_on_two_gloo_ranks(tmp_path):
    """world_size 2 on CPU: all-gather of per-shard candidates and the global merge."""
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29731", str(script),
           os.path.join(ROOT, "turboquant-kv_b200")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=280)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("ok") == 2


def test_vllm_v1_backend_conforms_to_the_installed_interface():
    """The v1 adapter subclasses the installed vLLM's abstract classes and is instantiable (no GPU work)."""
    v1 = pytest.importorskip("turboquant_kv.vllm_plugin.v1_backend")
    from vllm.v1.attention.backend import AttentionBackend, AttentionImpl, AttentionMetadataBuilder

    B = v1.TurboQuantV1Backend
    assert issubclass(B, AttentionBackend) and B.get_name() == "TURBOQUANT"
    assert issubclass(B.get_impl_cls(), AttentionImpl) and issubclass(B.get_builder_cls(), AttentionMetadataBuilder)
    assert B.get_kv_cache_shape(7, 32, 8, 64) == (7, 8, 2 * (2 * 64 * 6 + 128))
    assert B.get_kv_cache_block_dim(16, 8, 128) == 0
    assert B.supports_block_size(16) and not B.supports_block_size(8) and not B.supports_head_size(96)
    with pytest.raises(ValueError):
        B.get_kv_cache_shape(7, 24, 8, 64)
    impl = B.get_impl_cls()(32, 64, 0.125, 8)
    assert impl.num_kv_heads == 8 and impl.scale == 0.125
    with pytest.raises(NotImplementedError):
        B.get_impl_cls()(32, 64, 0.125, 8, sliding_window=128)
    builder = B.get_builder_cls()(None, ["l0"], None, "cpu")
    assert builder.layer_names == ["l0"]


def test_attention_function_registers_with_transformers_and_defaults_to_the_library_path():
    """Without an attached cache the registered attention function is transformers' own SDPA call."""
    pytest.importorskip("transformers")
    from transformers import DynamicCache, LlamaConfig, LlamaForCausalLM

    from turboquant_kv import hf_integration as hf

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=16)
    model = LlamaForCausalLM(cfg).eval()
    ids = torch.randint(0, 128, (2, 9))

    def run():
        cache = DynamicCache()
        with torch.no_grad():
            a = model(input_ids=ids[:, :8], past_key_values=cache, use_cache=True).logits
            b = model(input_ids=ids[:, 8:], past_key_values=cache, use_cache=True).logits
        return a, b

    model.set_attn_implementation("sdpa")
    want = run()
    name = hf.register_turboquant_attention()
    assert name == hf.ATTENTION_NAME == "turboquant"
    model.set_attn_implementation(name)
    got = run()
    assert torch.equal(want[0], got[0]) and torch.equal(want[1], got[1])
    # an empty cache announces masks of the size of the new tokens (DynamicCache's convention)
    assert hf.TurboQuantCache().get_mask_sizes(5, 0) == (5, 0)
    assert hf.TurboQuantCache().get_mask_sizes(torch.arange(3), 1) == (3, 0)


def test_attention_function_dispatch_rules_with_a_stand_in_store():
    """Which path the registered attention function takes: the fused kernel for a one-token step on an attached,
    quantised layer without a mask; old tokens dequantised + the new token exact when a mask is given; the plain
    library call for everything else (prefill, a detached module)."""
    pytest.importorskip("transformers")
    import weakref

    from turboquant_kv import hf_integration as hf

    B, HK, G, S, D = 2, 2, 2, 7, 16
    gen = torch.Generator().manual_seed(0)
    old_k, old_v = torch.randn(B, HK, S - 1, D, generator=gen), torch.randn(B, HK, S - 1, D, generator=gen)
    marker = torch.full((B, HK * G, D), 3.0)

    class Store(hf._LayerQuantStore):
        def __init__(self):                      # no device buffers: only what the attention function touches
            self.seq_len, self.asked = S, []

        def get_keys(self, dtype=torch.float32, upto=None):
            self.asked.append(("k", upto))
            return old_k[:, :, :upto].to(dtype)

        def get_values(self, dtype=torch.float32, upto=None):
            self.asked.append(("v", upto))
            return old_v[:, :, :upto].to(dtype)

        def decode_attention(self, query, scale):
            self.asked.append(("fused", tuple(query.shape), scale))
            return marker

    class Cache:
        fused_attention = True

        def __init__(self):
            self._layer_stores = {0: Store()}

    class Module(torch.nn.Module):
        layer_idx, num_key_value_groups = 0, G

    cache, mod = Cache(), Module()
    mod._turboquant_cache = weakref.ref(cache)
    q = torch.randn(B, HK * G, 1, D, generator=gen)
    k_new, v_new = torch.randn(B, HK, 1, D, generator=gen), torch.randn(B, HK, 1, D, generator=gen)

    out, weights = hf.turboquant_attention_forward(mod, q, k_new, v_new, None, scaling=0.25)
    assert weights is None and out.shape == (B, 1, HK * G, D) and torch.equal(out[:, 0], marker)
    assert cache._layer_stores[0].asked == [("fused", (B, HK * G, D), 0.25)]

    # with a mask: dense keys = old (dequantised) + new (exact), through the library's SDPA call
    cache._layer_stores[0].asked.clear()
    mask = torch.zeros(B, 1, 1, S)
    mask[1, :, :, :2] = float("-inf")
    out, _ = hf.turboquant_attention_forward(mod, q, k_new, v_new, mask, scaling=0.25)
    k_all = torch.cat([old_k, k_new], 2).repeat_interleave(G, 1)
    v_all = torch.cat([old_v, v_new], 2).repeat_interleave(G, 1)
    want = torch.nn.functional.scaled_dot_product_attention(q, k_all, v_all, attn_mask=mask, scale=0.25).transpose(1, 2)
    assert torch.allclose(out, want, atol=1e-5)
    assert cache._layer_stores[0].asked == [("k", S - 1), ("v", S - 1)]

    # prefill (several query tokens) and a module without a cache never touch the store
    cache._layer_stores[0].asked.clear()
    q3 = torch.randn(B, HK * G, 3, D, generator=gen)
    k3, v3 = torch.randn(B, HK, 3, D, generator=gen), torch.randn(B, HK, 3, D, generator=gen)
    hf.turboquant_attention_forward(mod, q3, k3, v3, None, scaling=0.25)
    hf.turboquant_attention_forward(Module(), q, k_new, v_new, None, scaling=0.25)
    cache.fused_attention = False
    hf.turboquant_attention_forward(mod, q, k_new, v_new, None, scaling=0.25)
    assert cache._layer_stores[0].asked == []


def test_scan_gives_query_groups_full_waves_of_few_large_ctas():
    """The planning rule of the batched index scan: one group takes every SM; many groups take few CTAs each, the
    whole grid a whole number of waves or nearly so, never fewer than two CTAs per group."""
    lib = ctypes.CDLL(LIB)
    f = lib.tqb_scan_records_ctas_per_group
    f.restype, f.argtypes = ctypes.c_int, [ctypes.c_int, ctypes.c_int64, ctypes.c_int]
    sms = 148
    assert f(1, 10_000_000, sms) == sms                       # a call of up to eight queries
    assert f(2, 10_000_000, sms) == sms // 2                  # two groups side by side, one wave
    assert f(5, 4_000_000, sms) == 29                         # 145 CTAs: one wave
    assert f(64, 4_000_000, sms) == 2                         # 128 CTAs: one wave of large CTAs
    assert f(1250, 10_000_000, sms) == 2                      # 10,000 queries
    assert f(0, 1000, sms) == 0 and f(3, -1, sms) == 0
    # the rule itself: waves of CTAs x (a CTA's share of the 16-row records + a fixed part worth 14,000 records)
    def cost(groups, rows, x):
        return -(-groups * x // sms) * (14_000 + -(-(-(-rows // 16)) // x))

    for groups in range(1, 400, 7):
        for rows in (1_000, 1_000_000, 10_000_000):
            x = f(groups, rows, sms)
            assert 2 <= x <= sms
            assert cost(groups, rows, x) == min(cost(groups, rows, y) for y in range(2, sms + 1)), (groups, rows, x)
