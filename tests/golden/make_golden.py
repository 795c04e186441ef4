#!/usr/bin/env python3
"""Generate the golden fixtures in this folder by running the upstream Python package itself.

Run from a checkout of ansschh/turboquant-kv (the upstream project this repository is a
drop-in for), on CPU:

    python tests/golden/make_golden.py --reference /path/to/turboquant-kv

The script imports ``turboquant_kv`` from ``--reference`` (never from this repository), runs
its public functions on seeded inputs and stores inputs and outputs as compressed ``.npz``
files next to this script.  The fixtures pin (1) the CPU oracle under ``oracle/`` and (2) the
CUDA path, both of which are compared with these files by the test-suite.  Nothing here is
needed at run time; the fixtures travel with the repository, the upstream checkout does not.

Files written (all small):
  constants.npz   Lloyd-Max codebooks, rotation matrices, QJL matrices     (reference.py:26-183,375-389)
  pack.npz        bit-plane pack / unpack cases                            (reference.py:191-255)
  mse.npz         quantize_mse / dequantize_mse                            (reference.py:263-367)
  prod.npz        quantize_prod / dequantize_prod                          (reference.py:392-533)
  attention.npz   dequantise-then-attend through QuantizedKVCache          (cache.py:148-339)
                  (MSE mode only: in Prod mode the upstream cache allocates key_bits planes,
                  cache.py:84-85, but quantize_prod returns key_bits-1, so append raises)
  search.npz      TurboQuantIndex.add / search, MSE and Prod               (search.py:126-252)
  hf_prod.npz     TurboQuantCache(mode="prod").update over two calls       (hf_integration.py:82-236, 339-390)
  index_files.npz index files as upstream writes them: TurboQuantIndex.save() in MSE and Prod mode
                  (search.py:254-277) and -- when oracle/_ref/libtq_ref.so is built -- the C++ core's
                  save() (csrc/core/turboquant_core.cpp:559-581), each with the search results / rows
                  upstream holds for it
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of ansschh/turboquant-kv")
    args = ap.parse_args()
    sys.path.insert(0, os.path.abspath(args.reference))

    import torch

    torch.set_num_threads(1)  # fixed summation order inside torch's CPU matmul
    from turboquant_kv import reference as ref
    from turboquant_kv.cache import QuantizedKVCache
    from turboquant_kv.config import TurboQuantConfig
    from turboquant_kv.search import TurboQuantIndex

    here = os.path.dirname(os.path.abspath(__file__))

    def save(name, **arrays):
        path = os.path.join(here, name)
        np.savez_compressed(path, **{k: np.asarray(v) for k, v in arrays.items()})
        print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB, {len(arrays)} arrays")

    # ------------------------------------------------------------------ constants
    const = {}
    for bits in (1, 2, 3, 4):
        for dim in (64, 128):
            b, c = ref.lloyd_max_codebook(bits, dim)
            const[f"boundaries_b{bits}_d{dim}"] = b.numpy()
            const[f"centroids_b{bits}_d{dim}"] = c.numpy()
    for dim, seed in ((64, 42), (64, 43), (128, 42), (32, 7)):
        const[f"rotation_qr_d{dim}_s{seed}"] = ref.make_rotation_matrix(dim, seed=seed).numpy()
    const["rotation_rht_d64_s42"] = ref.make_rotation_matrix(64, seed=42, method="rht").numpy()
    const["rotation_rht_d48_s5"] = ref.make_rotation_matrix(48, seed=5, method="rht").numpy()
    for dim, seed in ((64, 42), (128, 42)):
        const[f"qjl_d{dim}_s{seed}"] = ref._make_qjl_matrix(dim, dim, seed, torch.device("cpu")).numpy()
    save("constants.npz", **const)

    # ------------------------------------------------------------------ pack / unpack
    pk = {}
    rng = np.random.default_rng(11)
    for bits in (1, 2, 3, 4):
        for dim in (8, 20, 32, 64, 100, 128, 256):
            codes = rng.integers(0, 1 << bits, size=(13, dim), dtype=np.uint8)
            packed = ref.pack_codes(torch.from_numpy(codes), bits)
            back = ref.unpack_codes(packed, bits, dim)
            assert np.array_equal(back.numpy(), codes)
            pk[f"codes_b{bits}_d{dim}"] = codes
            pk[f"packed_b{bits}_d{dim}"] = packed.numpy()
    save("pack.npz", **pk)

    # ------------------------------------------------------------------ MSE
    mse = {}
    g = torch.Generator().manual_seed(0)
    for dim, n in ((128, 384), (64, 257), (32, 33)):
        x = torch.randn(n, dim, generator=g)
        x[0] = 0.0  # the all-zero row exercises the clamp in reference.py:295
        x[1] *= 1e-3
        x[2] *= 1e3
        mse[f"x_d{dim}"] = x.numpy()
        rot = ref.make_rotation_matrix(dim, seed=42)
        for bits in (1, 2, 3, 4):
            cb = ref.lloyd_max_codebook(bits, dim)
            packed, norms = ref.quantize_mse(x, bits, rotation=rot, codebook=cb)
            recon = ref.dequantize_mse(packed, norms, bits, dim, rotation=rot, codebook=cb)
            mse[f"packed_b{bits}_d{dim}"] = packed.numpy()
            mse[f"norms_b{bits}_d{dim}"] = norms.numpy()
            mse[f"recon_b{bits}_d{dim}"] = recon[:64].numpy()  # first 64 rows keep the file small
    # unit-norm inputs of the 65,536 x 128 round-trip configuration, first 512 rows
    g = torch.Generator().manual_seed(0)
    x = torch.randn(65536, 128, generator=g)
    x /= x.norm(dim=-1, keepdim=True)
    rot = ref.make_rotation_matrix(128, seed=42)
    cb = ref.lloyd_max_codebook(4, 128)
    packed, norms = ref.quantize_mse(x, 4, rotation=rot, codebook=cb)
    recon = ref.dequantize_mse(packed, norms, 4, 128, rotation=rot, codebook=cb)
    mse["unit_rows"] = np.int64(65536)
    mse["unit_packed_head"] = packed[:512].numpy()
    mse["unit_norms_head"] = norms[:512].numpy()
    mse["unit_mse_per_vector"] = np.float64(((x - recon) ** 2).sum(-1).mean().item())
    # a checksum over all 65,536 packed rows: per-column byte sums
    mse["unit_packed_colsum"] = packed.to(torch.int64).sum(0).numpy()
    save("mse.npz", **mse)

    # ------------------------------------------------------------------ Prod
    prod = {}
    g = torch.Generator().manual_seed(2)
    for dim, n in ((128, 320), (64, 129)):
        sig = torch.exp(torch.empty(dim).uniform_(np.log(0.1), np.log(10.0), generator=g)).sqrt()
        x = torch.randn(n, dim, generator=g) * sig
        x = x / x.norm(dim=-1, keepdim=True)
        x[0] = 0.0
        x[3] *= 17.0
        prod[f"x_d{dim}"] = x.numpy()
        rot = ref.make_rotation_matrix(dim, seed=42)
        S = ref._make_qjl_matrix(dim, dim, 42, torch.device("cpu"))
        for bits in (2, 3, 4):
            cb = ref.lloyd_max_codebook(bits - 1, dim)
            mp, sg, rn, nm = ref.quantize_prod(x, bits, rotation=rot, codebook=cb, S_matrix=S)
            recon = ref.dequantize_prod(mp, sg, rn, nm, bits, dim, rotation=rot, codebook=cb, S_matrix=S)
            prod[f"mse_packed_b{bits}_d{dim}"] = mp.numpy()
            prod[f"signs_b{bits}_d{dim}"] = sg.numpy()
            prod[f"res_norms_b{bits}_d{dim}"] = rn.numpy()
            prod[f"norms_b{bits}_d{dim}"] = nm.numpy()
            prod[f"recon_b{bits}_d{dim}"] = recon[:64].numpy()
    save("prod.npz", **prod)

    # ------------------------------------------------------------------ attention via the cache
    att = {}
    for tag, (heads, dim, seq, kb, vb, mode) in {
        "k4v2_d64": (2, 64, 203, 4, 2, "mse"),
        "k4v3_d128": (2, 128, 77, 4, 3, "mse"),
        "k2v4_d64": (3, 64, 50, 2, 4, "mse"),
    }.items():
        g = torch.Generator().manual_seed(4000)
        cfg = TurboQuantConfig(key_bits=kb, value_bits=vb, mode=mode, seed=42)
        cache = QuantizedKVCache(cfg, num_layers=1, max_seq_len=256, num_heads=heads,
                                 head_dim=dim, device="cpu")
        k = torch.randn(heads, seq, dim, generator=g)
        v = torch.randn(heads, seq, dim, generator=g)
        for h in range(heads):
            ch = torch.randperm(dim, generator=g)[:4]
            k[h][:, ch] *= 20.0
        q = torch.randn(3, heads, 1, dim, generator=g)  # batch of 3 queries per head
        cache.append(0, k[:, :150], v[:, :150]) if seq > 150 else cache.append(0, k, v)
        if seq > 150:
            cache.append(0, k[:, 150:], v[:, 150:])
        logits = cache.attention_scores(0, q)            # (3, heads, 1, seq), scaled by 1/sqrt(d)
        weights = torch.softmax(logits, dim=-1)
        out = cache.attention_values(0, weights)         # (3, heads, 1, dim)
        att[f"{tag}_k"] = k.numpy()
        att[f"{tag}_v"] = v.numpy()
        att[f"{tag}_q"] = q.numpy()
        att[f"{tag}_key_packed"] = cache._key_packed[0][:, :seq].numpy()
        att[f"{tag}_key_norms"] = cache._key_norms[0][:, :seq].numpy()
        att[f"{tag}_val_packed"] = cache._val_packed[0][:, :seq].numpy()
        att[f"{tag}_val_norms"] = cache._val_norms[0][:, :seq].numpy()
        att[f"{tag}_logits"] = logits.numpy()
        att[f"{tag}_out"] = out.numpy()
        att[f"{tag}_memory_bytes"] = np.int64(cache.memory_bytes())
        att[f"{tag}_compression_ratio"] = np.float64(cache.compression_ratio)
    save("attention.npz", **att)

    # ------------------------------------------------------------------ search
    srch = {}
    rng = np.random.default_rng(1000)
    db = np.round(np.clip(rng.gamma(0.5, 40.0, size=(3000, 128)), 0, 255)).astype(np.float32)
    qs = np.round(np.clip(np.random.default_rng(999).gamma(0.5, 40.0, size=(16, 128)), 0, 255)).astype(np.float32)
    srch["db"] = db.astype(np.uint8)  # integer-valued, stored compactly
    srch["queries"] = qs.astype(np.uint8)
    for bits, mode in ((4, "mse"), (3, "mse"), (2, "mse"), (3, "prod")):
        idx = TurboQuantIndex(dim=128, bit_width=bits, mode=mode, seed=42)
        assert not idx._use_cpp
        idx.add(torch.from_numpy(db[:2000]))
        idx.add(torch.from_numpy(db[2000:]))  # incremental insertion
        scores, ids = idx.search(torch.from_numpy(qs), k=10)
        srch[f"scores_b{bits}_{mode}"] = scores.numpy()
        srch[f"ids_b{bits}_{mode}"] = ids.numpy()
        srch[f"packed_b{bits}_{mode}"] = idx._packed_codes.numpy()
        srch[f"norms_b{bits}_{mode}"] = idx._norms.numpy()
        if mode == "prod":
            srch[f"signs_b{bits}_{mode}"] = idx._qjl_signs.numpy()
            srch[f"res_norms_b{bits}_{mode}"] = idx._residual_norms.numpy()
    save("search.npz", **srch)

    # ------------------------------------------------------------------ HF cache, Prod mode
    from turboquant_kv.hf_integration import TurboQuantCache

    hf = {}
    g = torch.Generator().manual_seed(321)
    cache = TurboQuantCache(key_bits=3, value_bits=4, mode="prod", seed=42)
    for step, t in enumerate((7, 1)):
        k = torch.randn(2, 2, t, 64, generator=g)
        v = torch.randn(2, 2, t, 64, generator=g)
        ko, vo = cache.update(k, v, 0)
        hf[f"k{step}"], hf[f"v{step}"] = k.numpy(), v.numpy()
        hf[f"keys_out{step}"], hf[f"values_out{step}"] = ko.numpy(), vo.numpy()
    save("hf_prod.npz", **hf)

    # ------------------------------------------------------------------ index files written by upstream
    import tempfile

    files = {}
    small = db[:400]
    with tempfile.TemporaryDirectory() as tmp:
        for bits, mode in ((4, "mse"), (3, "prod")):
            idx = TurboQuantIndex(dim=128, bit_width=bits, mode=mode, seed=42)
            assert not idx._use_cpp
            idx.add(torch.from_numpy(small))
            path = os.path.join(tmp, f"{mode}.idx")
            idx.save(path)
            scores, ids = idx.search(torch.from_numpy(qs), k=10)
            files[f"file_{mode}"] = np.frombuffer(open(path, "rb").read(), dtype=np.uint8)
            files[f"scores_{mode}"], files[f"ids_{mode}"] = scores.numpy(), ids.numpy()
        try:
            sys.path.insert(0, os.path.dirname(os.path.dirname(here)))
            from oracle import oracle as orc

            if orc.ref_lib() is not None:
                path = os.path.join(tmp, "core.tqix")
                packed, norms = orc.ref_index_build_save(small, 4, 42, path)
                files["file_core"] = np.frombuffer(open(path, "rb").read(), dtype=np.uint8)
                files["core_packed"], files["core_norms"] = packed, norms
        except Exception as exc:  # the C++ core is optional
            print("C++ core file skipped:", exc)
    files["queries"] = qs.astype(np.uint8)
    save("index_files.npz", **files)


if __name__ == "__main__":
    main()
