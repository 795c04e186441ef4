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


def _oracle_answer(orc, idx, queries, k):
    rot = orc.make_rotation_matrix(idx.dim, 42)
    _, cent = orc.lloyd_max_codebook(idx.bit_width, idx.dim)
    return orc.search_mse(queries.numpy(), idx._packed_codes.cpu().numpy(), idx._norms.cpu().numpy(), rot, cent,
                          idx.bit_width, k)


@pytest.mark.parametrize("dim,bits", [(128, 4), (96, 2)])     # the tensor-core path and the generic path
def test_static_scratch_scan_equals_workspace_scan_twice_in_a_row(orc, dim, bits):
    """Two calls in a row (they share the built-in scratch) give what the workspace entry point gives
    and what the CPU checker computes, and the call leaves the device's memory untouched."""
    L, N = _lib()
    assert L.tqb_scan_topk_static_capacity() == 4 << 20
    idx = _index(50_021, dim, bits, seed=5)
    gen = torch.Generator().manual_seed(9)
    for call, (nq, k) in enumerate([(8, 10), (3, 25)]):          # two calls in a row share the scratch
        queries = torch.rand(nq, dim, generator=gen) * 60.0
        (sc_ws, id_ws), (sc_st, id_st) = _both(L, N, idx, queries, k)
        assert torch.equal(id_st, id_ws), f"call {call}: ids differ"
        assert torch.equal(sc_st, sc_ws), f"call {call}: scores differ"
        assert not torch.isnan(sc_st).any() and (id_st >= 0).all()
        o_sc, o_ids = _oracle_answer(orc, idx, queries, k)
        assert np.array_equal(id_st.cpu().numpy(), o_ids), f"call {call}: ids differ from the CPU checker"
        assert np.array_equal(sc_st.cpu().numpy(), o_sc), f"call {call}: scores differ from the CPU checker"


def test_static_scratch_scan_allocates_nothing():
    """The property the entry point exists for: neither the driver nor torch's allocator hands out a
    single byte during a call (the set-up call that resolves the array's address comes first)."""
    L, N = _lib()
    idx = _index(20_000, 128, 4, seed=7)
    q = (torch.rand(4, 128) * 60.0).cuda()
    rot = idx._rotation.to("cuda", torch.float32).contiguous()
    cent = idx._codebook[1].to("cuda", torch.float32).contiguous()
    packed, norms = idx._packed_codes, idx._norms
    sc = torch.empty(4, 10, device="cuda")
    ids = torch.empty(4, 10, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        N.check(L.tqb_scan_topk_static(q.data_ptr(), 4, packed.data_ptr(), norms.data_ptr(), idx.n_vectors, 128, 4,
                                       rot.data_ptr(), cent.data_ptr(), 10, 0, sc.data_ptr(), ids.data_ptr(), stream))

    call()                                   # set-up: first call on this device
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, "device memory changed hands during tqb_scan_topk_static"
    assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0


def test_static_scratch_scan_rejects_what_does_not_fit():
    L, N = _lib()
    idx = _index(4_096, 64, 3, seed=6)
    rot = idx._rotation.to("cuda", torch.float32).contiguous()
    cent = idx._codebook[1].to("cuda", torch.float32).contiguous()
    cap = L.tqb_scan_topk_static_capacity()
    stream = torch.cuda.current_stream().cuda_stream

    def call(nq, k):
        q = torch.rand(nq, 64).cuda()
        sc = torch.empty(nq, k, device="cuda")
        ids = torch.empty(nq, k, dtype=torch.int64, device="cuda")
        rc = L.tqb_scan_topk_static(q.data_ptr(), nq, idx._packed_codes.data_ptr(), idx._norms.data_ptr(), 4_096, 64,
                                    3, rot.data_ptr(), cent.data_ptr(), k, 0, sc.data_ptr(), ids.data_ptr(), stream)
        torch.cuda.synchronize()
        return rc

    rc = call(200, 200)
    assert rc != 0
    with pytest.raises(RuntimeError, match="built-in scratch holds"):
        N.check(rc)
    # the boundary: the largest query count whose workspace still fits is accepted, one more is refused
    need = lambda nq: L.tqb_scan_topk_workspace_bytes(nq, 4_096, 64, 3, 10)
    fit = max(nq for nq in range(1, 200) if need(nq) <= cap)
    assert need(fit + 1) > cap
    assert call(fit, 10) == 0
    assert call(fit + 1, 10) == -4                       # TQB_ERR_WORKSPACE
    # same error code as tqb_scan_topk for a k beyond the scan's limit
    assert call(1, 257) == -2                            # TQB_ERR_UNSUPPORTED
