"""GPU test of tqb_scan_topk_static, the scan entry point that uses scratch memory built into the library.

Collected last on purpose (the file name sorts after every other test file): it must pass both on its
own and after the rest of the suite has used the device.  It talks to the C ABI directly."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

c_void_p, c_int, c_int64, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t


def _lib():
    from turboquant_kv import _native

    L = _native.lib()
    L.tqb_scan_topk_static.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                       c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]
    L.tqb_scan_topk_static_capacity.restype = c_size_t
    L.tqb_scan_topk_static_capacity.argtypes = []
    return L, _native


def _index(n, dim, bits, seed):
    from turboquant_kv import TurboQuantIndex

    rng = np.random.default_rng(seed)
    db = np.round(np.clip(rng.gamma(0.5, 40.0, size=(n, dim)), 0, 255)).astype(np.float32)
    idx = TurboQuantIndex(dim=dim, bit_width=bits, seed=42, device="cuda")
    idx.add(torch.from_numpy(db))
    return idx


def _both(L, N, idx, queries, k):
    """(scores, ids) from the regular entry point with a caller workspace, and from the static one."""
    q = queries.cuda().contiguous()
    nq, dim = q.shape
    n = idx.n_vectors
    rot = idx._rotation.to("cuda", torch.float32).contiguous()
    cent = idx._codebook[1].to("cuda", torch.float32).contiguous()
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for static in (False, True):
        sc = torch.full((nq, k), float("nan"), device="cuda")
        ids = torch.full((nq, k), -7, dtype=torch.int64, device="cuda")
        if static:
            rc = L.tqb_scan_topk_static(q.data_ptr(), nq, idx._packed_codes.data_ptr(), idx._norms.data_ptr(), n, dim,
                                        idx.bit_width, rot.data_ptr(), cent.data_ptr(), k, 0, sc.data_ptr(),
                                        ids.data_ptr(), stream)
        else:
            need = L.tqb_scan_topk_workspace_bytes(nq, n, dim, idx.bit_width, k)
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            rc = L.tqb_scan_topk(q.data_ptr(), nq, idx._packed_codes.data_ptr(), idx._norms.data_ptr(), n, dim,
                                 idx.bit_width, rot.data_ptr(), cent.data_ptr(), k, 0, ws.data_ptr(), need,
                                 sc.data_ptr(), ids.data_ptr(), stream)
        N.check(rc)
        outs.append((sc, ids))
    torch.cuda.synchronize()
    return outs


def test_static_scratch_scan_equals_workspace_scan_twice_in_a_row():
    L, N = _lib()
    assert L.tqb_scan_topk_static_capacity() == 4 << 20
    idx = _index(50_021, 128, 4, seed=5)
    gen = torch.Generator().manual_seed(9)
    for call, (nq, k) in enumerate([(8, 10), (3, 25)]):          # two calls in a row share the scratch
        queries = torch.rand(nq, 128, generator=gen) * 60.0
        (sc_ws, id_ws), (sc_st, id_st) = _both(L, N, idx, queries, k)
        assert torch.equal(id_st, id_ws), f"call {call}: ids differ"
        assert torch.equal(sc_st, sc_ws), f"call {call}: scores differ"
        assert not torch.isnan(sc_st).any() and (id_st >= 0).all()


def test_static_scratch_scan_rejects_what_does_not_fit():
    L, N = _lib()
    idx = _index(4_096, 64, 3, seed=6)
    q = torch.rand(200, 64).cuda()
    sc = torch.empty(200, 200, device="cuda")
    ids = torch.empty(200, 200, dtype=torch.int64, device="cuda")
    rot = idx._rotation.to("cuda", torch.float32).contiguous()
    cent = idx._codebook[1].to("cuda", torch.float32).contiguous()
    rc = L.tqb_scan_topk_static(q.data_ptr(), 200, idx._packed_codes.data_ptr(), idx._norms.data_ptr(), 4_096, 64, 3,
                                rot.data_ptr(), cent.data_ptr(), 200, 0, sc.data_ptr(), ids.data_ptr(),
                                torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    with pytest.raises(RuntimeError, match="built-in scratch holds"):
        N.check(rc)
