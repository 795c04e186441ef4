"""Host replay of the tensor-core fragment maps used by the decode-attention and scan kernels.

csrc/decode_bits.cuh holds the bit-plane -> fragment index arithmetic as host/device functions.
tests/fragment_harness.cpp replays a full 32-lane warp tile with them on the CPU; here the result
is compared with a direct evaluation on unpacked codes.  This pins the index maps, table entry
builders and dimension permutations without a GPU.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "turboquant-kv_b200", "csrc")


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("frag") / "libfrag.so")
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-x", "c++", "-shared", "-fPIC", "-I", CSRC,
                           os.path.join(ROOT, "tests", "fragment_harness.cpp"), "-o", out])
    return ctypes.CDLL(out)


def _ptr(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("bits", [2, 3, 4])
def test_key_tile_scores(harness, orc, dim, bits):
    rng = np.random.default_rng(dim + bits)
    codes = rng.integers(0, 1 << bits, size=(16, dim), dtype=np.uint8)
    tile = orc.pack_codes(codes, bits)
    cent = np.sort(rng.normal(size=1 << bits)).astype(np.float32)
    q = rng.normal(size=(8, dim)).astype(np.float32)
    out = np.zeros((16, 8), np.float32)
    rc = harness.replay_key_tile(dim, bits, _ptr(tile, ctypes.c_uint8), _ptr(cent, ctypes.c_float),
                                 _ptr(q, ctypes.c_float), _ptr(out, ctypes.c_float))
    assert rc == 0
    want = cent[codes] @ q.T
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("bits", [2, 3, 4])
def test_value_tile_accumulate(harness, orc, dim, bits):
    rng = np.random.default_rng(7 * dim + bits)
    codes = rng.integers(0, 1 << bits, size=(16, dim), dtype=np.uint8)
    tile = orc.pack_codes(codes, bits)
    cent = np.sort(rng.normal(size=1 << bits)).astype(np.float32)
    pw = rng.random(size=(16, 8)).astype(np.float32)
    out = np.zeros((dim, 8), np.float32)
    rc = harness.replay_value_tile(dim, bits, _ptr(tile, ctypes.c_uint8), _ptr(cent, ctypes.c_float),
                                   _ptr(pw, ctypes.c_float), _ptr(out, ctypes.c_float))
    assert rc == 0
    want = cent[codes].T @ pw
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("kb,vb", [(4, 2), (4, 3), (4, 4), (3, 3), (2, 2), (3, 4), (2, 3)])
def test_tiled_layout_roundtrip(harness, dim, kb, vb):
    """Fragment-major cache layout: the writer-side slots and the reader-side fields agree."""
    rng = np.random.default_rng(dim + 10 * kb + vb)
    kc = rng.integers(0, 1 << kb, size=(16, dim), dtype=np.uint8)
    vc = rng.integers(0, 1 << vb, size=(16, dim), dtype=np.uint8)
    ck = np.sort(rng.normal(size=1 << kb)).astype(np.float32)
    cv = np.sort(rng.normal(size=1 << vb)).astype(np.float32)
    q = rng.normal(size=(8, dim)).astype(np.float32)
    pw = rng.random(size=(16, 8)).astype(np.float32)
    scores = np.zeros((16, 8), np.float32)
    outv = np.zeros((dim, 8), np.float32)
    nbytes = harness.tiled_record_bytes(dim, kb, vb)
    assert nbytes == 2 * dim * (kb + vb) + 128
    rec = np.zeros(nbytes, np.uint8)
    rc = harness.replay_tiled(dim, kb, vb, _ptr(kc, ctypes.c_uint8), _ptr(vc, ctypes.c_uint8), _ptr(ck, ctypes.c_float),
                              _ptr(cv, ctypes.c_float), _ptr(q, ctypes.c_float), _ptr(pw, ctypes.c_float),
                              _ptr(scores, ctypes.c_float), _ptr(outv, ctypes.c_float), _ptr(rec, ctypes.c_uint8))
    assert rc == 0
    np.testing.assert_allclose(scores, ck[kc] @ q.T, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(outv, cv[vc].T @ pw, rtol=1e-4, atol=1e-4)
    # every code bit is stored exactly once: the code sections are fully used
    used = 2 * dim * (kb + vb)
    assert rec[used:].sum() == 0
