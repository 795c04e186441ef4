"""GPU parity: TurboQuantIndex.add / search against the golden fixtures, the oracle and (when built) the
upstream C++ core.  Bar: top-k ids identical except between scores that float32 summation cannot separate;
scores bit-identical to the oracle because the merge kernel re-scores in the upstream order."""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

from util import topk_ids_match

pytestmark = pytest.mark.gpu


def _db(rows, seed):
    rng = np.random.default_rng(seed)
    return np.round(np.clip(rng.gamma(0.5, 40.0, size=(rows, 128)), 0, 255)).astype(np.float32)


@pytest.mark.parametrize("bits,mode", [(4, "mse"), (3, "mse"), (2, "mse"), (3, "prod")])
def test_index_matches_upstream_fixture(orc, golden, bits, mode):
    from turboquant_kv import TurboQuantIndex

    g = golden("search")
    db, qs = g["db"].astype(np.float32), g["queries"].astype(np.float32)
    idx = TurboQuantIndex(dim=128, bit_width=bits, mode=mode, seed=42)
    idx.add(torch.from_numpy(db[:2000]))           # host tensors: staged on the GPU
    idx.add(torch.from_numpy(db[2000:]).cuda())    # incremental insertion, device tensor
    assert idx.n_vectors == 3000
    assert (idx._packed_codes.cpu().numpy() != g[f"packed_b{bits}_{mode}"]).mean() < 1e-4
    np.testing.assert_allclose(idx._norms.cpu().numpy(), g[f"norms_b{bits}_{mode}"], rtol=2e-6)
    # search over the upstream index contents so that only the scan is under test
    if idx._use_records:          # the scan reads the records: load the upstream rows into them
        idx._import_rows(torch.from_numpy(g[f"packed_b{bits}_{mode}"]), torch.from_numpy(g[f"norms_b{bits}_{mode}"]))
        assert np.array_equal(idx._packed_codes.cpu().numpy(), g[f"packed_b{bits}_{mode}"])
    else:
        idx._packed_codes = torch.from_numpy(g[f"packed_b{bits}_{mode}"]).cuda()
        idx._norms = torch.from_numpy(g[f"norms_b{bits}_{mode}"]).cuda()
    rot = orc.make_rotation_matrix(128, 42)
    if mode == "prod":
        idx._qjl_signs = torch.from_numpy(g[f"signs_b{bits}_{mode}"]).cuda()
        idx._residual_norms = torch.from_numpy(g[f"res_norms_b{bits}_{mode}"]).cuda()
        _, cent = orc.lloyd_max_codebook(bits - 1, 128)
        S = orc.make_qjl_matrix(128, 128, 42)
        o_sc, o_ids, allsc = orc.search_prod(qs, g[f"packed_b{bits}_{mode}"], g[f"signs_b{bits}_{mode}"],
                                             g[f"res_norms_b{bits}_{mode}"], g[f"norms_b{bits}_{mode}"], rot, cent, S,
                                             bits, 10, return_all=True)
    else:
        _, cent = orc.lloyd_max_codebook(bits, 128)
        o_sc, o_ids, allsc = orc.search_mse(qs, g[f"packed_b{bits}_{mode}"], g[f"norms_b{bits}_{mode}"], rot, cent,
                                            bits, 10, return_all=True)
    sc, ids = idx.search(torch.from_numpy(qs), k=10)
    assert sc.device.type == "cpu" and ids.dtype == torch.int64
    topk_ids_match(ids.numpy(), g[f"ids_b{bits}_{mode}"], allsc)
    np.testing.assert_allclose(sc.numpy(), g[f"scores_b{bits}_{mode}"], rtol=2e-5)
    if mode == "mse":
        assert np.array_equal(ids.numpy(), o_ids)
        assert np.array_equal(sc.numpy(), o_sc), "re-scored results must equal the upstream-order float32 sums"


@pytest.mark.parametrize("rows", [1, 5, 15, 16, 17, 1000, 50001])
def test_scan_row_counts_and_padding(orc, rows):
    from turboquant_kv import TurboQuantIndex

    db = _db(rows, 5)
    qs = _db(9, 6)
    idx = TurboQuantIndex(dim=128, bit_width=4, seed=42)
    idx.add(torch.from_numpy(db).cuda())
    rot = orc.make_rotation_matrix(128, 42)
    _, cent = orc.lloyd_max_codebook(4, 128)
    k = 10
    sc, ids = idx.search(torch.from_numpy(qs).cuda(), k=k)
    kk = min(k, rows)
    assert sc.shape == (9, kk)                      # k is clipped like the upstream Python path
    o_sc, o_ids = orc.search_mse(qs, idx._packed_codes.cpu().numpy(), idx._norms.cpu().numpy(), rot, cent, 4, kk)
    assert np.array_equal(ids.cpu().numpy(), o_ids)
    assert np.array_equal(sc.cpu().numpy(), o_sc)


@pytest.mark.parametrize("dim,bits", [(64, 4), (64, 2), (128, 3), (32, 4), (200, 3), (256, 1), (96, 2)])
def test_scan_shapes_tensor_core_and_generic_paths(orc, dim, bits):
    from turboquant_kv import TurboQuantIndex

    rng = np.random.default_rng(dim * 10 + bits)
    db = rng.normal(size=(4099, dim)).astype(np.float32)
    qs = rng.normal(size=(7, dim)).astype(np.float32)
    idx = TurboQuantIndex(dim=dim, bit_width=bits, seed=7)
    idx.add(torch.from_numpy(db).cuda())
    rot = orc.make_rotation_matrix(dim, 7)
    _, cent = orc.lloyd_max_codebook(bits, dim)
    sc, ids = idx.search(torch.from_numpy(qs).cuda(), k=25)
    o_sc, o_ids, allsc = orc.search_mse(qs, idx._packed_codes.cpu().numpy(), idx._norms.cpu().numpy(), rot, cent,
                                        bits, 25, return_all=True)
    topk_ids_match(ids.cpu().numpy(), o_ids, allsc, rel_tie=1e-6)
    np.testing.assert_allclose(sc.cpu().numpy(), o_sc, rtol=1e-6)


def test_scan_duplicate_rows_order_by_id(orc):
    from turboquant_kv import TurboQuantIndex

    base = _db(64, 1)
    db = np.concatenate([base] * 40)                # every row 40 times: massive exact ties
    idx = TurboQuantIndex(dim=128, bit_width=4, seed=42)
    idx.add(torch.from_numpy(db).cuda())
    qs = _db(4, 2)
    sc, ids = idx.search(torch.from_numpy(qs).cuda(), k=10)
    rot = orc.make_rotation_matrix(128, 42)
    _, cent = orc.lloyd_max_codebook(4, 128)
    o_sc, o_ids = orc.search_mse(qs, idx._packed_codes.cpu().numpy(), idx._norms.cpu().numpy(), rot, cent, 4, 10)
    assert np.array_equal(ids.cpu().numpy(), o_ids)
    assert np.array_equal(sc.cpu().numpy(), o_sc)


def test_scan_against_upstream_cpp_core(orc):
    if orc.ref_lib() is None:
        pytest.skip("oracle/_ref/libtq_ref.so not built")
    from turboquant_kv import TurboQuantIndex

    db, qs = _db(200_000, 1000), _db(16, 999)
    idx = TurboQuantIndex(dim=128, bit_width=4, seed=42)
    idx.add(torch.from_numpy(db).cuda())
    sc, ids = idx.search(torch.from_numpy(qs).cuda(), k=10)
    rot = orc.make_rotation_matrix(128, 42)
    _, cent = orc.lloyd_max_codebook(4, 128)
    r_sc, r_ids = orc.ref_search_packed(qs, idx._packed_codes.cpu().numpy(), idx._norms.cpu().numpy(), rot, cent, 4, 10)
    assert np.array_equal(ids.cpu().numpy(), r_ids)
    assert np.array_equal(sc.cpu().numpy(), r_sc)


def _scan_rows_call(packed, norms, qs, dim, bits, rot, cent, k):
    """tqb_scan_topk through the C ABI on upstream-layout rows (the drop-in for search_packed)."""
    from turboquant_kv import _native as N

    L = N.lib()
    n, nq = packed.shape[0], qs.shape[0]
    d = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dt)
    q_d, p_d, n_d, r_d, c_d = d(qs, torch.float32), d(packed, torch.uint8), d(norms, torch.float32), \
        d(rot, torch.float32), d(cent, torch.float32)
    need = L.tqb_scan_topk_workspace_bytes(nq, n, dim, bits, k)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    sc = torch.full((nq, k), float("nan"), device="cuda")
    ids = torch.full((nq, k), -7, dtype=torch.int64, device="cuda")
    N.check(L.tqb_scan_topk(q_d.data_ptr(), nq, p_d.data_ptr(), n_d.data_ptr(), n, dim, bits, r_d.data_ptr(),
                            c_d.data_ptr(), k, 0, ws.data_ptr(), need, sc.data_ptr(), ids.data_ptr(),
                            torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(ws[:4].view(torch.int32).item()) == 0, "a bounded device-side wait expired"
    return sc.cpu().numpy(), ids.cpu().numpy()


@pytest.mark.parametrize("dim,bits", [(64, 2), (64, 3), (64, 4), (128, 2), (128, 3), (128, 4)])
def test_scan_topk_on_upstream_rows_matches_oracle_and_upstream_core(orc, dim, bits):
    """The tensor-core scan over upstream-layout rows (dims 64 / 128, 2-4 bits) behind tqb_scan_topk,
    checked against the CPU checker and the upstream C++ core (csrc/core/turboquant_core.cpp:407-514):
    ids and scores identical, at row counts around the 16-row tile and with a ragged last tile."""
    rng = np.random.default_rng(100 * dim + bits)
    rot = orc.make_rotation_matrix(dim, 42)
    bnd, cent = orc.lloyd_max_codebook(bits, dim)
    k = 10
    for rows in (1, 15, 16, 17, 50_021):
        db = np.round(np.clip(rng.gamma(0.5, 40.0, size=(rows, dim)), 0, 255)).astype(np.float32)
        packed, norms = orc.quantize_mse(db, bits, rot, bnd)
        for nq in (1, 5, 8):
            qs = np.round(np.clip(rng.gamma(0.5, 40.0, size=(nq, dim)), 0, 255)).astype(np.float32)
            sc, ids = _scan_rows_call(packed, norms, qs, dim, bits, rot, cent, k)
            kk = min(k, rows)
            o_sc, o_ids = orc.search_mse(qs, packed, norms, rot, cent, bits, kk)
            assert np.array_equal(ids[:, :kk], o_ids), (rows, nq)
            assert np.array_equal(sc[:, :kk], o_sc), (rows, nq)
            assert (ids[:, kk:] == -1).all() and np.isneginf(sc[:, kk:]).all()   # padded like upstream
            if orc.ref_lib() is not None:
                r_sc, r_ids = orc.ref_search_packed(qs, packed, norms, rot, cent, bits, k)
                assert np.array_equal(ids, r_ids), (rows, nq)
                assert np.array_equal(sc, r_sc), (rows, nq)


def test_many_queries_and_large_k(orc):
    from turboquant_kv import TurboQuantIndex

    db, qs = _db(30_000, 3), _db(700, 4)            # more queries than one scan call takes
    idx = TurboQuantIndex(dim=128, bit_width=4, seed=42)
    idx.add(torch.from_numpy(db).cuda())
    sc, ids = idx.search(torch.from_numpy(qs).cuda(), k=100)
    rot = orc.make_rotation_matrix(128, 42)
    _, cent = orc.lloyd_max_codebook(4, 128)
    o_sc, o_ids, allsc = orc.search_mse(qs, idx._packed_codes.cpu().numpy(), idx._norms.cpu().numpy(), rot, cent, 4, 100,
                                        return_all=True)
    topk_ids_match(ids.cpu().numpy(), o_ids, allsc, rel_tie=1e-6)
    with pytest.raises(RuntimeError):
        idx.search(torch.from_numpy(qs[:2]).cuda(), k=1000)


def test_save_load_both_layouts(tmp_path, golden):
    from turboquant_kv import TurboQuantIndex

    g = golden("search")
    db = torch.from_numpy(g["db"].astype(np.float32))
    qs = torch.from_numpy(g["queries"].astype(np.float32)).cuda()
    for mode, bits in (("mse", 4), ("prod", 3)):
        idx = TurboQuantIndex.from_vectors(db, bit_width=bits, mode=mode, seed=42)
        want = idx.search(qs, 10)
        p = str(tmp_path / f"{mode}.idx")
        idx.save(p)
        back = TurboQuantIndex.load(p, seed=42)
        assert back.mode == mode and back.n_vectors == 3000
        got = back.search(qs, 10)
        assert torch.equal(want[1], got[1]) and torch.equal(want[0], got[0])
        size = os.path.getsize(p)
        per_row = (bits if mode == "mse" else bits - 1) * 16 + 4 + (16 + 4 if mode == "prod" else 0)
        assert size == 9 + 1 + 3000 * per_row
    idx = TurboQuantIndex.from_vectors(db, bit_width=4, seed=42)
    p = str(tmp_path / "core.tqix")
    idx.save(p, format="tqix")
    assert os.path.getsize(p) == 24 + 3000 * 68
    back = TurboQuantIndex.load(p)
    assert torch.equal(back.search(qs, 10)[1], idx.search(qs, 10)[1])


def test_row_sharded_search_merges_to_the_global_answer(orc):
    """Two shards on one GPU, merged with the merge kernel: same top-k as the unsharded index."""
    from turboquant_kv import TurboQuantIndex
    from turboquant_kv.distributed import shard_rows
    from turboquant_kv.search import merge_topk

    db, qs = _db(20_001, 8), torch.from_numpy(_db(33, 9)).cuda()
    whole = TurboQuantIndex.from_vectors(torch.from_numpy(db).cuda(), bit_width=4, seed=42)
    want_s, want_i = whole.search(qs, 10)
    parts_s, parts_i = [], []
    for r in range(3):
        lo, hi = shard_rows(db.shape[0], 3, r)
        shard = TurboQuantIndex(dim=128, bit_width=4, seed=42)
        shard.id_offset = lo
        shard.add(torch.from_numpy(db[lo:hi]).cuda())
        s, i = shard.search(qs, 10)
        parts_s.append(s)
        parts_i.append(i)
    got_s, got_i = merge_topk(torch.stack(parts_s, 1), torch.stack(parts_i, 1), 10)
    assert torch.equal(got_i, want_i) and torch.equal(got_s, want_s)


@pytest.mark.parametrize("dim,bits", [(64, 2), (64, 3), (64, 4), (128, 2), (128, 3), (128, 4)])
def test_index_records_hold_exactly_the_upstream_rows(dim, bits):
    """The index stores key-only 16-row records; exported, they are the rows quantize_mse produces, and
    rows imported into records come back unchanged (any row count, including a partial last record)."""
    from turboquant_kv import TurboQuantIndex, _native as N, quantize_mse

    rng = np.random.default_rng(dim + bits)
    n = 1000 + 7
    x = torch.from_numpy(rng.standard_normal((n, dim)).astype(np.float32)).cuda()
    idx = TurboQuantIndex(dim=dim, bit_width=bits, seed=7, device="cuda")
    idx.add(x[:333])
    idx.add(x[333:])                                   # a second add starts in the middle of a record
    assert idx._use_records and idx.n_vectors == n
    packed, norms = quantize_mse(x, bits, rotation=idx._rotation, codebook=idx._codebook)
    assert torch.equal(idx._packed_codes, packed)
    assert torch.equal(idx._norms, norms)
    # import -> export round trip through the C ABI on random codes
    L = N.lib()
    rec_bytes = L.tqb_kv_record_bytes(dim, bits, 0)
    assert rec_bytes == 2 * dim * bits + 64
    codes = torch.from_numpy(rng.integers(0, 256, size=(n, bits * dim // 8), dtype=np.uint8)).cuda()
    nrm = torch.from_numpy(rng.random(n).astype(np.float32)).cuda()
    store = torch.zeros(((n + 15) // 16) * rec_bytes, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    N.check(L.tqb_kv_import(store.data_ptr(), n, dim, bits, 0, None, codes.data_ptr(), nrm.data_ptr(), None, None, st))
    back_c, back_n = torch.empty_like(codes), torch.empty_like(nrm)
    N.check(L.tqb_kv_export(store.data_ptr(), n, dim, bits, 0, None, back_c.data_ptr(), back_n.data_ptr(), None, None, st))
    torch.cuda.synchronize()
    assert torch.equal(back_c, codes) and torch.equal(back_n, nrm)
    # key-only records have no value rows
    rc = L.tqb_kv_export(store.data_ptr(), n, dim, bits, 0, None, back_c.data_ptr(), back_n.data_ptr(),
                         back_c.data_ptr(), None, st)
    assert rc != 0 and "key-only" in L.tqb_last_error().decode()


@pytest.mark.parametrize("mode,bits", [("mse", 4), ("prod", 3)])
def test_load_reads_files_written_by_upstream_save(tmp_path, golden, orc, mode, bits):
    """An index file written by the upstream Python ``TurboQuantIndex.save()`` (search.py:254-277; the bytes
    are part of the fixture) loads here and searches like the upstream index it came from."""
    from turboquant_kv import TurboQuantIndex

    g = golden("index_files")
    p = str(tmp_path / f"upstream_{mode}.idx")
    g[f"file_{mode}"].tofile(p)
    idx = TurboQuantIndex.load(p, seed=42)
    assert (idx.mode, idx.bit_width, idx.dim, idx.n_vectors) == (mode, bits, 128, 400)
    qs = g["queries"].astype(np.float32)
    sc, ids = idx.search(torch.from_numpy(qs), k=10)
    # all scores of the upstream index's rows, for the tie rule
    rot = orc.make_rotation_matrix(128, 42)
    packed, norms = idx._packed_codes.cpu().numpy(), idx._norms.cpu().numpy()
    if mode == "prod":
        _, cent = orc.lloyd_max_codebook(bits - 1, 128)
        _, _, allsc = orc.search_prod(qs, packed, idx._qjl_signs.cpu().numpy(), idx._residual_norms.cpu().numpy(), norms,
                                      rot, cent, orc.make_qjl_matrix(128, 128, 42), bits, 10, return_all=True)
    else:
        _, cent = orc.lloyd_max_codebook(bits, 128)
        _, _, allsc = orc.search_mse(qs, packed, norms, rot, cent, bits, 10, return_all=True)
    topk_ids_match(ids.numpy(), g[f"ids_{mode}"], allsc)
    np.testing.assert_allclose(sc.numpy(), g[f"scores_{mode}"], rtol=2e-5)
    # and a file written here is byte-identical to upstream's for the same index
    q = str(tmp_path / f"again_{mode}.idx")
    idx.save(q)
    assert np.array_equal(np.fromfile(q, dtype=np.uint8), g[f"file_{mode}"])


def test_load_reads_a_file_written_by_the_upstream_cpp_core(tmp_path, golden):
    """A file written by the upstream C++ core's ``save()`` (csrc/core/turboquant_core.cpp:559-581): header and
    rows are read as the core holds them, and writing them back reproduces the file.  (The core draws its
    rotation and codebook from its own generators, so searching such rows needs the core's constants; the
    layout is what is checked here.)"""
    from turboquant_kv import TurboQuantIndex

    g = golden("index_files")
    if "file_core" not in g:
        pytest.skip("the fixture was generated without the C++ core")
    p = str(tmp_path / "core.tqix")
    g["file_core"].tofile(p)
    idx = TurboQuantIndex.load(p)
    assert (idx.mode, idx.bit_width, idx.dim, idx.n_vectors, idx.seed) == ("mse", 4, 128, 400, 42)
    assert np.array_equal(idx._packed_codes.cpu().numpy(), g["core_packed"])
    assert np.array_equal(idx._norms.cpu().numpy(), g["core_norms"])
    q = str(tmp_path / "again.tqix")
    idx.save(q, format="tqix")
    assert np.array_equal(np.fromfile(q, dtype=np.uint8), g["file_core"])


@pytest.mark.parametrize("dim,bits,rows", [(128, 3, 30_011), (64, 2, 1000), (96, 4, 5000), (128, 5, 777)])
def test_prod_search_runs_the_packed_scan_and_matches_dequantise_then_multiply(orc, dim, bits, rows):
    """Prod-mode search (upstream search.py:229-252) through tqb_scan_topk_prod: ids against the CPU checker's
    dequantise-then-multiply except between scores closer than float32 summation noise, scores to rounding;
    several dims and bit widths (1 to 4 MSE bits), a ragged row count, more queries than a pass."""
    from turboquant_kv import TurboQuantIndex

    rng = np.random.default_rng(dim + bits)
    db = rng.standard_normal((rows, dim)).astype(np.float32) * rng.uniform(0.3, 3.0, size=(1, dim)).astype(np.float32)
    qs = rng.standard_normal((21, dim)).astype(np.float32)
    idx = TurboQuantIndex(dim=dim, bit_width=bits, mode="prod", seed=42)
    idx.add(torch.from_numpy(db).cuda())
    k = 10
    sc, ids = idx.search(torch.from_numpy(qs).cuda(), k=k)
    rot = orc.make_rotation_matrix(dim, 42)
    _, cent = orc.lloyd_max_codebook(bits - 1, dim)
    S = orc.make_qjl_matrix(dim, dim, 42)
    o_sc, o_ids, allsc = orc.search_prod(qs, idx._packed_codes.cpu().numpy(), idx._qjl_signs.cpu().numpy(),
                                         idx._residual_norms.cpu().numpy(), idx._norms.cpu().numpy(), rot, cent, S,
                                         bits, k, return_all=True)
    topk_ids_match(ids.cpu().numpy(), o_ids, allsc, rel_tie=2e-5)
    np.testing.assert_allclose(sc.cpu().numpy(), o_sc, rtol=3e-5, atol=1e-5)
    # k larger than the rows of a tiny index is clipped like upstream
    tiny = TurboQuantIndex(dim=dim, bit_width=bits, mode="prod", seed=42)
    tiny.add(torch.from_numpy(db[:5]).cuda())
    s5, i5 = tiny.search(torch.from_numpy(qs[:2]).cuda(), k=10)
    assert s5.shape == (2, 5) and sorted(i5[0].tolist()) == [0, 1, 2, 3, 4]
