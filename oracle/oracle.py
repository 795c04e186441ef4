"""numpy front-end of the CPU checker.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module.  It is loaded by the test-suite, by the
smoke test and by the CPU-baseline legs of bench.py, and only to *check* or to be *timed beside*
the CUDA kernels -- never as a compute path of the product.

It wraps ``libtq_oracle.so`` (the C restatement in ``tq_oracle.c``) and, when present,
``_ref/libtq_ref.so`` (the upstream C++ core compiled from an upstream checkout), and restates the
three host-side constant generators of upstream ``turboquant_kv/reference.py``:

  lloyd_max_codebook     reference.py:26-73
  make_rotation_matrix   reference.py:81-183
  make_qjl_matrix        reference.py:375-389

Parity is pinned: ``tests/test_oracle_golden.py`` compares every function here with outputs of
the upstream Python package stored under ``tests/golden``.
"""
from __future__ import annotations

import ctypes
import math
import os
from functools import lru_cache

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

_f32p = ctypes.POINTER(ctypes.c_float)
_u8p = ctypes.POINTER(ctypes.c_uint8)
_i64p = ctypes.POINTER(ctypes.c_int64)
_i32p = ctypes.POINTER(ctypes.c_int32)


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libtq_oracle.so")
        if not os.path.exists(path):
            from . import build as _b  # type: ignore

            _b.build_oracle()
        _LIB = ctypes.CDLL(path)
        _LIB.tqo_num_threads.restype = ctypes.c_int
    return _LIB


def ref_lib():
    """The upstream C++ core behind the C shim, or None when it was never built."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libtq_ref.so")
        if not os.path.exists(path):
            return None
        _REF = ctypes.CDLL(path)
        _REF.tqr_num_threads.restype = ctypes.c_int
    return _REF


_REF_CPU = None


def ref_cpu_lib():
    """The upstream CPU kernels (csrc/cpu/quant_cpu.cpp) behind ref_cpu_shim.cpp, or None when never built.
    The library links against torch: torch is imported first so that its shared objects are loaded."""
    global _REF_CPU
    if _REF_CPU is None:
        path = os.path.join(_HERE, "_ref", "libtq_ref_cpu.so")
        if not os.path.exists(path):
            return None
        import torch  # noqa: F401  (loads libtorch_cpu / libc10 into the process)

        try:
            _REF_CPU = ctypes.CDLL(path)
        except OSError:
            return None
        _REF_CPU.tqc_num_threads.restype = ctypes.c_int
    return _REF_CPU


def num_threads() -> int:
    return int(_lib().tqo_num_threads())


def set_num_threads(n: int) -> None:
    _lib().tqo_set_num_threads(int(n))
    r = ref_lib()
    if r is not None:
        r.tqr_set_num_threads(int(n))
    if _REF_CPU is not None:
        _REF_CPU.tqc_set_num_threads(int(n))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def _p(a, t):
    return a.ctypes.data_as(t)


def packed_dim(dim: int, bits: int) -> int:
    return bits * ((dim + 7) // 8)


# --------------------------------------------------------------------------- host constants


@lru_cache(maxsize=32)
def _lloyd_max_unit(bits: int, max_iter: int = 200, tol: float = 1e-12):
    """Lloyd-Max levels of N(0,1) (reference.py:26-55): start from linspace(-3,3), iterate
    boundary = midpoint, centroid = conditional mean, stop when the largest move is < tol."""
    from scipy.stats import norm

    levels = 1 << bits
    cent = np.linspace(-3.0, 3.0, levels)
    for _ in range(max_iter):
        edges = np.concatenate(([-np.inf], 0.5 * (cent[:-1] + cent[1:]), [np.inf]))
        new = np.zeros(levels, dtype=np.float64)
        for i in range(levels):
            lo, hi = edges[i], edges[i + 1]
            mass = norm.cdf(hi) - norm.cdf(lo)
            new[i] = cent[i] if mass < 1e-15 else (norm.pdf(lo) - norm.pdf(hi)) / mass
        if np.max(np.abs(new - cent)) < tol:
            break  # upstream keeps the previous centroids when it stops here
        cent = new
    return 0.5 * (cent[:-1] + cent[1:]), cent


def lloyd_max_codebook(bits: int, dim: int):
    """(boundaries[2^b-1], centroids[2^b]) float32, N(0,1) levels scaled by 1/sqrt(dim)
    (reference.py:58-73)."""
    import torch

    bnd, cent = _lloyd_max_unit(bits)
    scale = 1.0 / math.sqrt(dim)
    return (torch.tensor(bnd * scale, dtype=torch.float32).numpy(),
            torch.tensor(cent * scale, dtype=torch.float32).numpy())


def make_rotation_matrix(dim: int, seed: int = 42, method: str = "dense_qr") -> np.ndarray:
    """Random orthogonal matrix, float32 (reference.py:81-183)."""
    if method == "dense_qr":
        g = np.random.RandomState(seed).randn(dim, dim).astype(np.float32)
        q, r = np.linalg.qr(g)
        sgn = np.sign(np.diag(r))
        sgn[sgn == 0] = 1.0
        return np.ascontiguousarray(q * sgn[None, :], dtype=np.float32)
    if method == "rht":
        import torch

        gen = torch.Generator().manual_seed(seed)
        padded = 1
        while padded < dim:
            padded <<= 1
        flips = torch.where(torch.randint(0, 2, (padded,), generator=gen).bool(),
                            torch.ones(padded), -torch.ones(padded))
        had = torch.ones(1, 1)
        while had.shape[0] < padded:
            had = torch.cat([torch.cat([had, had], 1), torch.cat([had, -had], 1)], 0)
        had = had / math.sqrt(padded)
        m = (had @ torch.diag(flips))[:dim, :dim]
        q, r = torch.linalg.qr(m)
        sgn = torch.sign(torch.diag(r))
        sgn[sgn == 0] = 1.0
        return (q * sgn.unsqueeze(0)).float().numpy().copy()
    raise ValueError(f"Unknown rotation method: {method}")


def make_qjl_matrix(dim: int, n_sign_bits: int, seed: int) -> np.ndarray:
    """Gaussian QJL projection, torch CPU generator seeded with seed+12345 (reference.py:375-389)."""
    import torch

    gen = torch.Generator(device="cpu").manual_seed(seed + 12345)
    return torch.randn(n_sign_bits, dim, generator=gen, dtype=torch.float32).numpy().copy()


# --------------------------------------------------------------------------- wrappers


def pack_codes(codes, bits: int) -> np.ndarray:
    codes = _u8(codes)
    n, dim = codes.shape
    out = np.empty((n, packed_dim(dim, bits)), dtype=np.uint8)
    _lib().tqo_pack_codes(_p(codes, _u8p), ctypes.c_int64(n), dim, bits, _p(out, _u8p))
    return out


def unpack_codes(packed, bits: int, dim: int) -> np.ndarray:
    packed = _u8(packed)
    n = packed.shape[0]
    assert packed.shape[1] == packed_dim(dim, bits)
    out = np.empty((n, dim), dtype=np.uint8)
    _lib().tqo_unpack_codes(_p(packed, _u8p), ctypes.c_int64(n), dim, bits, _p(out, _u8p))
    return out


def quantize_mse(x, bits: int, rotation, boundaries, return_rotated: bool = False):
    x = _f32(x).reshape(-1, np.shape(x)[-1])
    n, dim = x.shape
    rot, bnd = _f32(rotation), _f32(boundaries)
    assert bnd.shape[0] == (1 << bits) - 1
    packed = np.empty((n, packed_dim(dim, bits)), dtype=np.uint8)
    norms = np.empty((n,), dtype=np.float32)
    rotated = np.empty((n, dim), dtype=np.float32) if return_rotated else None
    _lib().tqo_quantize_mse(_p(x, _f32p), ctypes.c_int64(n), dim, _p(rot, _f32p), _p(bnd, _f32p),
                            bits, _p(packed, _u8p), _p(norms, _f32p),
                            _p(rotated, _f32p) if return_rotated else None)
    return (packed, norms, rotated) if return_rotated else (packed, norms)


def dequantize_mse(packed, norms, bits: int, dim: int, rotation, centroids) -> np.ndarray:
    packed, norms = _u8(packed), _f32(norms)
    n = packed.shape[0]
    rot, cent = _f32(rotation), _f32(centroids)
    out = np.empty((n, dim), dtype=np.float32)
    _lib().tqo_dequantize_mse(_p(packed, _u8p), _p(norms, _f32p), ctypes.c_int64(n), dim,
                              _p(rot, _f32p), _p(cent, _f32p), bits, _p(out, _f32p))
    return out


def quantize_prod(x, bits: int, rotation, boundaries, centroids, S, return_projected: bool = False):
    x = _f32(x).reshape(-1, np.shape(x)[-1])
    n, dim = x.shape
    rot, bnd, cent, S = _f32(rotation), _f32(boundaries), _f32(centroids), _f32(S)
    assert bits >= 2 and bnd.shape[0] == (1 << (bits - 1)) - 1
    mp = np.empty((n, packed_dim(dim, bits - 1)), dtype=np.uint8)
    sg = np.empty((n, packed_dim(dim, 1)), dtype=np.uint8)
    rn = np.empty((n,), dtype=np.float32)
    nm = np.empty((n,), dtype=np.float32)
    proj = np.empty((n, dim), dtype=np.float32) if return_projected else None
    _lib().tqo_quantize_prod(_p(x, _f32p), ctypes.c_int64(n), dim, _p(rot, _f32p), _p(bnd, _f32p),
                             _p(cent, _f32p), _p(S, _f32p), bits, _p(mp, _u8p), _p(sg, _u8p),
                             _p(rn, _f32p), _p(nm, _f32p),
                             _p(proj, _f32p) if return_projected else None)
    return (mp, sg, rn, nm, proj) if return_projected else (mp, sg, rn, nm)


def dequantize_prod(mse_packed, signs, res_norms, norms, bits: int, dim: int, rotation, centroids,
                    S) -> np.ndarray:
    mp, sg, rn, nm = _u8(mse_packed), _u8(signs), _f32(res_norms), _f32(norms)
    n = mp.shape[0]
    rot, cent, S = _f32(rotation), _f32(centroids), _f32(S)
    out = np.empty((n, dim), dtype=np.float32)
    _lib().tqo_dequantize_prod(_p(mp, _u8p), _p(sg, _u8p), _p(rn, _f32p), _p(nm, _f32p),
                               ctypes.c_int64(n), dim, _p(rot, _f32p), _p(cent, _f32p),
                               _p(S, _f32p), bits, _p(out, _f32p))
    return out


def attention_scores_packed(query, packed_keys, key_norms, centroids, rotation, bits: int):
    """ops.py:131-194 -- unscaled scores (batch, heads, seq)."""
    q = _f32(query)
    b, h, dim = q.shape
    pk, kn = _u8(packed_keys), _f32(key_norms)
    seq = pk.shape[0]
    out = np.empty((b, h, seq), dtype=np.float32)
    _lib().tqo_attention_scores_packed(_p(q, _f32p), ctypes.c_int64(b * h), dim, _p(pk, _u8p),
                                       _p(kn, _f32p), ctypes.c_int64(seq),
                                       _p(_f32(centroids), _f32p), _p(_f32(rotation), _f32p), bits,
                                       _p(out, _f32p))
    return out


def attention_values_packed(weights, packed_values, value_norms, centroids, rotation_T, bits: int):
    """ops.py:202-246 -- (batch, heads, dim)."""
    w = _f32(weights)
    b, h, seq = w.shape
    rt = _f32(rotation_T)
    dim = rt.shape[0]
    out = np.empty((b, h, dim), dtype=np.float32)
    _lib().tqo_attention_values_packed(_p(w, _f32p), ctypes.c_int64(b * h), ctypes.c_int64(seq),
                                       dim, _p(_u8(packed_values), _u8p),
                                       _p(_f32(value_norms), _f32p), _p(_f32(centroids), _f32p),
                                       _p(rt, _f32p), bits, _p(out, _f32p))
    return out


def decode_attention(query, k_packed, k_norms, v_packed, v_norms, seq_lens, rot_k, cent_k, kbits,
                     rot_v, cent_v, vbits, scale=None):
    """Dequantise-then-attend for one new token per sequence (cache.py:216-339).

    query (batch, q_heads, dim); k_packed (batch, kv_heads, max_seq, pk); k_norms
    (batch, kv_heads, max_seq); same for v; seq_lens (batch,).  Returns (batch, q_heads, dim).
    """
    q = _f32(query)
    batch, q_heads, dim = q.shape
    kp, kn, vp, vn = _u8(k_packed), _f32(k_norms), _u8(v_packed), _f32(v_norms)
    kv_heads, max_seq = kp.shape[1], kp.shape[2]
    sl = np.ascontiguousarray(seq_lens, dtype=np.int32)
    if scale is None:
        scale = 1.0 / math.sqrt(dim)
    out = np.empty((batch, q_heads, dim), dtype=np.float32)
    _lib().tqo_decode_attention(_p(q, _f32p), batch, q_heads, kv_heads, dim, _p(kp, _u8p),
                                _p(kn, _f32p), _p(vp, _u8p), _p(vn, _f32p),
                                ctypes.c_int64(max_seq), _p(sl, _i32p), _p(_f32(rot_k), _f32p),
                                _p(_f32(cent_k), _f32p), kbits, _p(_f32(rot_v), _f32p),
                                _p(_f32(cent_v), _f32p), vbits, ctypes.c_float(scale),
                                _p(out, _f32p))
    return out


def ref_cpu_decode_attention(query, k_packed, k_norms, v_packed, v_norms, seq_lens, rot_k, cent_k, kbits,
                             rot_v, cent_v, vbits, scale=None, threads: int = 0):
    """The same decode step with the UPSTREAM CPU kernels (csrc/cpu/quant_cpu.cpp:125-266): per (sequence, KV
    head) attention_scores_packed_cpu, softmax, attention_values_packed_cpu.  Arguments as decode_attention."""
    lib = ref_cpu_lib()
    if lib is None:
        raise RuntimeError("oracle/_ref/libtq_ref_cpu.so was not built (no upstream checkout)")
    q = _f32(query)
    batch, q_heads, dim = q.shape
    kp, kn, vp, vn = _u8(k_packed), _f32(k_norms), _u8(v_packed), _f32(v_norms)
    kv_heads, max_seq = kp.shape[1], kp.shape[2]
    sl = np.ascontiguousarray(seq_lens, dtype=np.int32)
    if scale is None:
        scale = 1.0 / math.sqrt(dim)
    lib.tqc_set_num_threads(int(threads) if threads else (os.cpu_count() or 1))
    out = np.empty((batch, q_heads, dim), dtype=np.float32)
    # attention_values_packed_cpu ends with out = rotated @ M; the inverse of y = R x is x = y @ R
    rc = lib.tqc_decode_attention(_p(q, _f32p), _p(kp, _u8p), _p(kn, _f32p), _p(vp, _u8p), _p(vn, _f32p),
                                  _p(sl, _i32p), batch, q_heads, kv_heads, max_seq, dim, kbits, vbits,
                                  _p(_f32(rot_k), _f32p), _p(_f32(cent_k), _f32p), _p(_f32(rot_v), _f32p),
                                  _p(_f32(cent_v), _f32p), ctypes.c_float(scale), _p(out, _f32p))
    if rc != 0:
        raise RuntimeError("the upstream CPU kernels raised")
    return out


def ref_cpu_quantize(x, bits: int, rotation, boundaries):
    """Upstream rotate_and_quantize_cpu (csrc/cpu/quant_cpu.cpp:44-119)."""
    lib = ref_cpu_lib()
    if lib is None:
        raise RuntimeError("oracle/_ref/libtq_ref_cpu.so was not built (no upstream checkout)")
    v = _f32(x)
    n, dim = v.shape
    packed = np.empty((n, packed_dim(dim, bits)), dtype=np.uint8)
    norms = np.empty(n, dtype=np.float32)
    rc = lib.tqc_rotate_and_quantize(_p(v, _f32p), n, dim, _p(_f32(rotation), _f32p), _p(_f32(boundaries), _f32p), bits,
                                     _p(packed, _u8p), _p(norms, _f32p))
    if rc != 0:
        raise RuntimeError("the upstream CPU kernels raised")
    return packed, norms


def search_mse(queries, packed, norms, rotation, centroids, bits: int, k: int,
               return_all: bool = False):
    q = _f32(queries)
    nq, dim = q.shape
    pk, nm = _u8(packed), _f32(norms)
    n = pk.shape[0]
    sc = np.empty((nq, k), dtype=np.float32)
    ids = np.empty((nq, k), dtype=np.int64)
    allsc = np.empty((nq, n), dtype=np.float32) if return_all else None
    _lib().tqo_search_mse(_p(q, _f32p), ctypes.c_int64(nq), dim, _p(pk, _u8p), _p(nm, _f32p),
                          ctypes.c_int64(n), _p(_f32(rotation), _f32p), _p(_f32(centroids), _f32p),
                          bits, k, _p(sc, _f32p), _p(ids, _i64p),
                          _p(allsc, _f32p) if return_all else None)
    return (sc, ids, allsc) if return_all else (sc, ids)


def search_prod(queries, mse_packed, signs, res_norms, norms, rotation, centroids, S, bits: int,
                k: int, return_all: bool = False):
    q = _f32(queries)
    nq, dim = q.shape
    mp = _u8(mse_packed)
    n = mp.shape[0]
    sc = np.empty((nq, k), dtype=np.float32)
    ids = np.empty((nq, k), dtype=np.int64)
    allsc = np.empty((nq, n), dtype=np.float32) if return_all else None
    _lib().tqo_search_prod(_p(q, _f32p), ctypes.c_int64(nq), dim, _p(mp, _u8p),
                           _p(_u8(signs), _u8p), _p(_f32(res_norms), _f32p),
                           _p(_f32(norms), _f32p), ctypes.c_int64(n), _p(_f32(rotation), _f32p),
                           _p(_f32(centroids), _f32p), _p(_f32(S), _f32p), bits, k,
                           _p(sc, _f32p), _p(ids, _i64p), _p(allsc, _f32p) if return_all else None)
    return (sc, ids, allsc) if return_all else (sc, ids)


# --------------------------------------------------------------------------- upstream C++ core


def ref_search_packed(queries, packed, norms, rotation, centroids, bits: int, k: int):
    """Upstream ``turboquant::search_packed`` (csrc/core/turboquant_core.cpp:407-514)."""
    lib = ref_lib()
    if lib is None:
        raise RuntimeError("oracle/_ref/libtq_ref.so was not built (no upstream checkout)")
    q = _f32(queries)
    nq, dim = q.shape
    pk, nm = _u8(packed), _f32(norms)
    sc = np.empty((nq, k), dtype=np.float32)
    ids = np.empty((nq, k), dtype=np.int64)
    lib.tqr_search_packed(_p(q, _f32p), nq, _p(pk, _u8p), _p(nm, _f32p), pk.shape[0], dim, bits,
                          _p(_f32(rotation), _f32p), _p(_f32(centroids), _f32p), k, _p(sc, _f32p),
                          _p(ids, _i64p))
    return sc, ids


def ref_index_build_save(vectors, bits: int, seed: int, path: str):
    """Upstream C++ ``TurboQuantIndex``: add the vectors, ``save(path)`` (csrc/core/turboquant_core.cpp:523-581).
    Returns the rows the core holds: (packed (n, bits * ceil(dim / 8)), norms (n,))."""
    lib = ref_lib()
    if lib is None:
        raise RuntimeError("oracle/_ref/libtq_ref.so was not built (no upstream checkout)")
    x = _f32(vectors)
    n, dim = x.shape
    packed = np.empty((n, packed_dim(dim, bits)), dtype=np.uint8)
    norms = np.empty(n, dtype=np.float32)
    lib.tqr_index_build_save.restype = ctypes.c_int
    got = lib.tqr_index_build_save(_p(x, _f32p), n, dim, bits, seed, path.encode(), _p(packed, _u8p), _p(norms, _f32p))
    if got != n:
        raise RuntimeError("the upstream core failed to build or save the index")
    return packed, norms


def ref_quantize(x, bits: int, rotation, boundaries, centroids):
    """Upstream ``turboquant::quantize_vectors`` (csrc/core/turboquant_core.cpp:277-343)."""
    lib = ref_lib()
    if lib is None:
        raise RuntimeError("oracle/_ref/libtq_ref.so was not built (no upstream checkout)")
    x = _f32(x)
    n, dim = x.shape
    packed = np.empty((n, packed_dim(dim, bits)), dtype=np.uint8)
    norms = np.empty((n,), dtype=np.float32)
    lib.tqr_quantize(_p(x, _f32p), n, dim, _p(_f32(rotation), _f32p), _p(_f32(boundaries), _f32p),
                     _p(_f32(centroids), _f32p), bits, _p(packed, _u8p), _p(norms, _f32p))
    return packed, norms
