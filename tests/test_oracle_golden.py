"""Pin the CPU checker (oracle/) against outputs of the upstream Python package.

The fixtures under tests/golden were produced by tests/golden/make_golden.py importing the
upstream ``turboquant_kv`` package.  Integer results (packed codes, sign bits, ids) must be
bit-exact except at decision-boundary ties, which are recognised from the oracle's own rotated
coordinates: a differing code is accepted only when the coordinate lies within 1e-6 of a
boundary (float32 summation order differs between torch's blocked matmul and a sequential sum).
"""
from __future__ import annotations

import numpy as np
import pytest

TIE_EPS = 1e-6        # |rotated coordinate - boundary| below which a differing code is a tie
MAX_TIE_RATE = 1e-5   # the parity bar for packed codes and signs


def _codes_match_up_to_ties(orc, packed, packed_ref, rotated, boundaries, bits, dim):
    a = orc.unpack_codes(packed, bits, dim)
    b = orc.unpack_codes(packed_ref, bits, dim)
    bad = np.argwhere(a != b)
    for r, j in bad:
        dist = np.min(np.abs(boundaries.astype(np.float64) - float(rotated[r, j])))
        assert dist < TIE_EPS, f"row {r} dim {j}: codes {a[r, j]} vs {b[r, j]}, {dist:.3e} from a boundary"
        assert abs(int(a[r, j]) - int(b[r, j])) == 1
    return len(bad) / a.size


def test_codebooks_match(orc, golden):
    g = golden("constants")
    for bits in (1, 2, 3, 4):
        for dim in (64, 128):
            bnd, cent = orc.lloyd_max_codebook(bits, dim)
            assert np.array_equal(bnd, g[f"boundaries_b{bits}_d{dim}"])
            assert np.array_equal(cent, g[f"centroids_b{bits}_d{dim}"])


def test_rotations_and_qjl_match(orc, golden):
    g = golden("constants")
    for dim, seed in ((64, 42), (64, 43), (128, 42), (32, 7)):
        assert np.array_equal(orc.make_rotation_matrix(dim, seed), g[f"rotation_qr_d{dim}_s{seed}"])
    assert np.allclose(orc.make_rotation_matrix(64, 42, "rht"), g["rotation_rht_d64_s42"], atol=1e-6)
    assert np.allclose(orc.make_rotation_matrix(48, 5, "rht"), g["rotation_rht_d48_s5"], atol=1e-6)
    for dim in (64, 128):
        assert np.array_equal(orc.make_qjl_matrix(dim, dim, 42), g[f"qjl_d{dim}_s42"])
    with pytest.raises(ValueError):
        orc.make_rotation_matrix(8, 1, "nope")


def test_pack_unpack_bit_exact(orc, golden):
    g = golden("pack")
    for bits in (1, 2, 3, 4):
        for dim in (8, 20, 32, 64, 100, 128, 256):
            codes, packed = g[f"codes_b{bits}_d{dim}"], g[f"packed_b{bits}_d{dim}"]
            assert np.array_equal(orc.pack_codes(codes, bits), packed)
            assert np.array_equal(orc.unpack_codes(packed, bits, dim), codes)
    assert orc.pack_codes(np.zeros((0, 64), np.uint8), 4).shape == (0, 32)


def test_quantize_mse_matches_upstream(orc, golden):
    g, c = golden("mse"), golden("constants")
    worst = 0.0
    for dim in (128, 64, 32):
        x = g[f"x_d{dim}"]
        rot = orc.make_rotation_matrix(dim, 42)
        for bits in (1, 2, 3, 4):
            bnd, cent = orc.lloyd_max_codebook(bits, dim)
            packed, norms, rotated = orc.quantize_mse(x, bits, rot, bnd, return_rotated=True)
            rate = _codes_match_up_to_ties(orc, packed, g[f"packed_b{bits}_d{dim}"], rotated, bnd, bits, dim)
            worst = max(worst, rate)
            np.testing.assert_allclose(norms, g[f"norms_b{bits}_d{dim}"], rtol=2e-6)
            recon = orc.dequantize_mse(g[f"packed_b{bits}_d{dim}"], g[f"norms_b{bits}_d{dim}"], bits, dim, rot, cent)
            ref = g[f"recon_b{bits}_d{dim}"]
            np.testing.assert_allclose(recon[:64], ref, rtol=1e-4, atol=1e-5 * np.abs(ref).max())
    assert worst <= 1e-3  # a few hundred rows: one tie is already 2e-5; the full-size rate is below


def test_quantize_mse_unit_sphere_config(orc, golden):
    """The 65,536 x 128 4-bit round trip: all packed rows (checksum), first 512 rows, and MSE."""
    import torch

    g = golden("mse")
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(65536, 128, generator=gen)
    x /= x.norm(dim=-1, keepdim=True)
    x = x.numpy()
    rot = orc.make_rotation_matrix(128, 42)
    bnd, cent = orc.lloyd_max_codebook(4, 128)
    packed, norms, rotated = orc.quantize_mse(x, 4, rot, bnd, return_rotated=True)
    rate = _codes_match_up_to_ties(orc, packed[:512], g["unit_packed_head"], rotated[:512], bnd, 4, 128)
    assert rate <= 1e-4
    np.testing.assert_allclose(norms[:512], g["unit_norms_head"], rtol=2e-6)
    # column checksums over all rows: a tie moves at most a couple of bits per column
    diff = np.abs(packed.astype(np.int64).sum(0) - g["unit_packed_colsum"])
    assert diff.max() <= 256 and (diff > 0).sum() <= 16
    recon = orc.dequantize_mse(packed, norms, 4, 128, rot, cent)
    mse = float(((x - recon) ** 2).sum(-1).mean())
    assert abs(mse - float(g["unit_mse_per_vector"])) < 1e-6


def test_quantize_prod_matches_upstream(orc, golden):
    g = golden("prod")
    for dim in (128, 64):
        x = g[f"x_d{dim}"]
        rot = orc.make_rotation_matrix(dim, 42)
        S = orc.make_qjl_matrix(dim, dim, 42)
        for bits in (2, 3, 4):
            bnd, cent = orc.lloyd_max_codebook(bits - 1, dim)
            mp, sg, rn, nm, proj = orc.quantize_prod(x, bits, rot, bnd, cent, S, return_projected=True)
            ref_codes = orc.unpack_codes(g[f"mse_packed_b{bits}_d{dim}"], bits - 1, dim)
            got_codes = orc.unpack_codes(mp, bits - 1, dim)
            rows_ok = (ref_codes == got_codes).all(axis=1)
            assert (~rows_ok).mean() <= 0.01  # MSE-code ties (checked precisely in the MSE test)
            a = orc.unpack_codes(sg, 1, dim)
            b = orc.unpack_codes(g[f"signs_b{bits}_d{dim}"], 1, dim)
            bad = np.argwhere((a != b) & rows_ok[:, None])
            scale = np.abs(proj).max()
            for r, j in bad:
                assert abs(proj[r, j]) < 1e-5 * scale, "sign differs away from a zero projection"
            assert len(bad) / a.size <= 1e-3
            np.testing.assert_allclose(nm, g[f"norms_b{bits}_d{dim}"], rtol=2e-6)
            np.testing.assert_allclose(rn[rows_ok], g[f"res_norms_b{bits}_d{dim}"][rows_ok], rtol=1e-4, atol=1e-6)
            recon = orc.dequantize_prod(g[f"mse_packed_b{bits}_d{dim}"], g[f"signs_b{bits}_d{dim}"],
                                        g[f"res_norms_b{bits}_d{dim}"], g[f"norms_b{bits}_d{dim}"],
                                        bits, dim, rot, cent, S)
            ref = g[f"recon_b{bits}_d{dim}"]
            np.testing.assert_allclose(recon[:64], ref, rtol=1e-4, atol=1e-5 * np.abs(ref).max())


@pytest.mark.parametrize("tag,dim,kb,vb", [("k4v2_d64", 64, 4, 2), ("k4v3_d128", 128, 4, 3), ("k2v4_d64", 64, 2, 4)])
def test_attention_matches_upstream_cache(orc, golden, tag, dim, kb, vb):
    g = golden("attention")
    k, v, q = g[f"{tag}_k"], g[f"{tag}_v"], g[f"{tag}_q"]          # (H,S,d), (H,S,d), (3,H,1,d)
    heads, seq, _ = k.shape
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    bk, ck = orc.lloyd_max_codebook(kb, dim)
    bv, cv = orc.lloyd_max_codebook(vb, dim)
    kp, kn = orc.quantize_mse(k.reshape(-1, dim), kb, rk, bk)
    vp, vn = orc.quantize_mse(v.reshape(-1, dim), vb, rv, bv)
    kp_ref, vp_ref = g[f"{tag}_key_packed"], g[f"{tag}_val_packed"]
    assert (kp.reshape(kp_ref.shape) != kp_ref).mean() < 1e-3
    assert (vp.reshape(vp_ref.shape) != vp_ref).mean() < 1e-3
    np.testing.assert_allclose(kn.reshape(heads, seq), g[f"{tag}_key_norms"], rtol=2e-6)
    # attend over the upstream cache contents: one "sequence" per query batch item
    nb = q.shape[0]
    rep = lambda a: np.broadcast_to(a[None], (nb,) + a.shape).copy()
    out = orc.decode_attention(q[:, :, 0, :], rep(kp_ref), rep(g[f"{tag}_key_norms"]), rep(vp_ref),
                               rep(g[f"{tag}_val_norms"]), np.full(nb, seq, np.int32), rk, ck, kb, rv, cv, vb)
    ref = g[f"{tag}_out"][:, :, 0, :]
    assert np.abs(out - ref).max() < 1e-4
    cos = (out * ref).sum() / np.sqrt((out * out).sum() * (ref * ref).sum())
    assert cos > 0.999999
    # operator-level scores (unscaled) against the cache logits (scaled by 1/sqrt(d))
    for h in range(heads):
        sc = orc.attention_scores_packed(q[:, h:h + 1, 0, :], kp_ref[h], g[f"{tag}_key_norms"][h], ck, rk, kb)
        ref_l = g[f"{tag}_logits"][:, h, 0, :] * np.sqrt(dim)
        np.testing.assert_allclose(sc[:, 0, :], ref_l, rtol=1e-4, atol=1e-4 * np.abs(ref_l).max())
        w = np.exp(g[f"{tag}_logits"][:, h, 0, :] - g[f"{tag}_logits"][:, h, 0, :].max(-1, keepdims=True))
        w = (w / w.sum(-1, keepdims=True)).astype(np.float32)
        o = orc.attention_values_packed(w[:, None, :], vp_ref[h], g[f"{tag}_val_norms"][h], cv, rv, vb)
        np.testing.assert_allclose(o[:, 0, :], ref[:, h, :], atol=1e-4)


@pytest.mark.parametrize("bits,mode", [(4, "mse"), (3, "mse"), (2, "mse"), (3, "prod")])
def test_search_matches_upstream_index(orc, golden, bits, mode):
    g = golden("search")
    db, qs = g["db"].astype(np.float32), g["queries"].astype(np.float32)
    rot = orc.make_rotation_matrix(128, 42)
    packed, norms = g[f"packed_b{bits}_{mode}"], g[f"norms_b{bits}_{mode}"]
    if mode == "mse":
        bnd, cent = orc.lloyd_max_codebook(bits, 128)
        got_p, got_n = orc.quantize_mse(db, bits, rot, bnd)
        assert (got_p != packed).mean() < 1e-4
        sc, ids, allsc = orc.search_mse(qs, packed, norms, rot, cent, bits, 10, return_all=True)
    else:
        bnd, cent = orc.lloyd_max_codebook(bits - 1, 128)
        S = orc.make_qjl_matrix(128, 128, 42)
        sc, ids, allsc = orc.search_prod(qs, packed, g[f"signs_b{bits}_{mode}"], g[f"res_norms_b{bits}_{mode}"],
                                         norms, rot, cent, S, bits, 10, return_all=True)
    ref_sc, ref_ids = g[f"scores_b{bits}_{mode}"], g[f"ids_b{bits}_{mode}"]
    np.testing.assert_allclose(sc, ref_sc, rtol=2e-5)
    for qi in range(qs.shape[0]):
        if np.array_equal(ids[qi], ref_ids[qi]):
            continue
        # any disagreement must be between scores closer than float32 summation noise
        for a, b in zip(ids[qi], ref_ids[qi]):
            if a != b:
                assert abs(allsc[qi, a] - allsc[qi, b]) <= 4e-6 * abs(allsc[qi, a])


def test_search_pads_when_k_exceeds_rows(orc, golden):
    g = golden("search")
    rot = orc.make_rotation_matrix(128, 42)
    _, cent = orc.lloyd_max_codebook(4, 128)
    sc, ids = orc.search_mse(g["queries"][:2].astype(np.float32), g["packed_b4_mse"][:3], g["norms_b4_mse"][:3],
                             rot, cent, 4, 5)
    assert np.all(ids[:, 3:] == -1) and np.all(np.isinf(sc[:, 3:]))
    assert set(ids[0, :3]) == {0, 1, 2}


def test_upstream_cpp_core_agrees_with_oracle(orc, golden):
    """The upstream C++ core (when built) and the restatement return the same top-10."""
    if orc.ref_lib() is None:
        pytest.skip("oracle/_ref/libtq_ref.so not built")
    g = golden("search")
    rot = orc.make_rotation_matrix(128, 42)
    bnd, cent = orc.lloyd_max_codebook(4, 128)
    qs = g["queries"].astype(np.float32)
    sc, ids = orc.search_mse(qs, g["packed_b4_mse"], g["norms_b4_mse"], rot, cent, 4, 10)
    rsc, rids = orc.ref_search_packed(qs, g["packed_b4_mse"], g["norms_b4_mse"], rot, cent, 4, 10)
    assert np.array_equal(ids, rids)
    np.testing.assert_allclose(sc, rsc, rtol=1e-6)
    p, n = orc.ref_quantize(g["db"].astype(np.float32), 4, rot, bnd, cent)
    assert (p != g["packed_b4_mse"]).mean() < 1e-4


def test_hf_prod_cache_fixture_is_algorithm_2_on_every_head(orc, golden):
    """The upstream HF cache in Prod mode (hf_integration.py:82-236): what update() returns for the OLD tokens
    is dequantize_prod(quantize_prod(.)) per head with the layer's constants (keys: seed, values: seed + 1),
    the NEW tokens come back exactly."""
    g = golden("hf_prod")
    for which, bits, seed in (("k", 3, 42), ("v", 4, 43)):
        rot = orc.make_rotation_matrix(64, seed)
        bnd, cent = orc.lloyd_max_codebook(bits - 1, 64)
        S = orc.make_qjl_matrix(64, 64, seed)
        first = g[f"{which}0"]                                        # (batch, heads, 7, 64)
        out1 = g["keys_out1" if which == "k" else "values_out1"]      # (batch, heads, 8, 64)
        assert np.array_equal(out1[:, :, 7:], g[f"{which}1"])
        mp, sg, rn, nr = orc.quantize_prod(first.reshape(-1, 64), bits, rot, bnd, cent, S)
        rec = orc.dequantize_prod(mp, sg, rn, nr, bits, 64, rot, cent, S).reshape(first.shape)
        np.testing.assert_allclose(out1[:, :, :7], rec, atol=3e-5)


def test_upstream_index_files_have_the_documented_layout(orc, golden):
    """Files written by upstream save() (search.py:254-277) and by the C++ core (turboquant_core.cpp:559-581):
    header fields and section sizes as the loader of this repository assumes them."""
    import struct

    g = golden("index_files")
    for mode, bits in (("mse", 4), ("prod", 3)):
        blob = g[f"file_{mode}"].tobytes()
        bw, dim, n = struct.unpack_from("<BII", blob, 0)               # bit width (u8), dim, rows; then a mode byte
        assert (bw, dim, n, blob[9]) == (bits, 128, 400, 0 if mode == "mse" else 1)
        per_row = (bits if mode == "mse" else bits - 1) * 16 + 4 + (16 + 4 if mode == "prod" else 0)
        assert len(blob) == 10 + 400 * per_row
    if "file_core" in g:
        blob = g["file_core"].tobytes()
        magic, version, dim, bits, seed, n = struct.unpack_from("<6I", blob, 0)
        assert (magic, version, dim, bits, seed, n) == (0x54514958, 1, 128, 4, 42, 400)
        assert len(blob) == 24 + 400 * (64 + 4)
        assert np.array_equal(np.frombuffer(blob, np.uint8, 400 * 64, 24).reshape(400, 64), g["core_packed"])
        assert np.array_equal(np.frombuffer(blob, np.float32, 400, 24 + 400 * 64), g["core_norms"])


def test_upstream_cpu_kernels_agree_with_oracle(orc):
    """The upstream OpenMP kernels (csrc/cpu/quant_cpu.cpp, compiled in place into oracle/_ref) on a small
    cache: their decode step equals the checker's dequantise-then-attend, and rotate_and_quantize_cpu yields
    the checker's codes (ties aside)."""
    if orc.ref_cpu_lib() is None:
        pytest.skip("oracle/_ref/libtq_ref_cpu.so is not built here")
    rng = np.random.default_rng(12)
    batch, kvh, group, dim, seq = 3, 2, 4, 64, 300
    rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
    bk, ck = orc.lloyd_max_codebook(4, dim)
    bv, cv = orc.lloyd_max_codebook(2, dim)
    k = rng.standard_normal((batch * kvh * seq, dim), dtype=np.float32)
    v = rng.standard_normal((batch * kvh * seq, dim), dtype=np.float32)
    kp, kn = orc.quantize_mse(k, 4, rk, bk)
    vp, vn = orc.quantize_mse(v, 2, rv, bv)
    r_kp, r_kn = orc.ref_cpu_quantize(k, 4, rk, bk)
    assert (r_kp != kp).mean() < 1e-4
    np.testing.assert_allclose(r_kn, kn, rtol=2e-6)
    q = rng.standard_normal((batch, kvh * group, dim), dtype=np.float32)
    lens = np.array([seq, 17, 0], np.int32)
    args = (q, kp.reshape(batch, kvh, seq, -1), kn.reshape(batch, kvh, seq), vp.reshape(batch, kvh, seq, -1),
            vn.reshape(batch, kvh, seq), lens, rk, ck, 4, rv, cv, 2)
    want = orc.decode_attention(*args)
    got = orc.ref_cpu_decode_attention(*args, threads=4)
    np.testing.assert_allclose(got, want, atol=2e-5, rtol=1e-4)
