"""TurboQuant Algorithm 1 (MSE) and Algorithm 2 (Prod), arXiv:2504.19874 -- B200 build.

Same public functions and argument meaning as upstream ``turboquant_kv/reference.py``
(``quantize_mse`` :263, ``dequantize_mse`` :320, ``quantize_prod`` :392, ``dequantize_prod`` :472,
``pack_codes`` :191, ``unpack_codes`` :227, ``lloyd_max_codebook`` :58, ``make_rotation_matrix`` :81),
but the tensor work runs in hand-written sm_100a kernels behind ``libtqb200.so``.

What stays in Python are the three one-off constant generators (codebook, rotation, QJL matrix):
they run once per configuration on the host and their results are *inputs* of the kernels.

Differences from upstream, all deliberate:
  * computation always happens on a CUDA device.  Host tensors are copied to the current device,
    processed there and the results copied back; without CUDA the call raises (no CPU fallback);
  * arithmetic is float32 whatever the input dtype (upstream rotates fp16/bf16 inputs in half
    precision, reference.py:300,307); norms are returned as float32;
  * supported head/vector dims: multiples of 8 up to 256.
"""
from __future__ import annotations

import math
from functools import lru_cache
from typing import Optional, Tuple

import numpy as np
import torch

from . import _native as N

__all__ = [
    "lloyd_max_codebook", "make_rotation_matrix", "make_rht_rotation", "pack_codes", "unpack_codes",
    "quantize_mse", "dequantize_mse", "quantize_prod", "dequantize_prod",
]


# --------------------------------------------------------------------------------------------
# host-side constants
# --------------------------------------------------------------------------------------------

def _lloyd_max_codebook_unscaled(bits: int, max_iter: int = 200, tol: float = 1e-12):
    """Lloyd-Max quantiser of the standard normal: float64 (boundaries, centroids).

    Fixed-point iteration from 2^bits levels spread evenly over [-3, 3]: decision boundaries are
    midpoints, every level moves to the conditional mean of its cell,
    E[X | lo < X < hi] = (pdf(lo) - pdf(hi)) / (cdf(hi) - cdf(lo)); cells of mass < 1e-15 stay put.
    The loop ends once no level would move by `tol` any more (that last move is not applied).
    """
    from scipy.stats import norm as gaussian

    levels = 1 << bits
    cent = np.linspace(-3.0, 3.0, levels)
    for _ in range(max_iter):
        cuts = np.concatenate(([-np.inf], (cent[1:] + cent[:-1]) / 2.0, [np.inf]))
        lo, hi = cuts[:-1], cuts[1:]
        moved = cent.copy()
        for i in range(levels):
            mass = gaussian.cdf(hi[i]) - gaussian.cdf(lo[i])
            if mass >= 1e-15:
                moved[i] = (gaussian.pdf(lo[i]) - gaussian.pdf(hi[i])) / mass
        if np.max(np.abs(moved - cent)) < tol:
            break
        cent = moved
    return (cent[1:] + cent[:-1]) / 2.0, cent


@lru_cache(maxsize=16)
def lloyd_max_codebook(bits: int, dim: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(boundaries (2^bits - 1,), centroids (2^bits,)) float32 for coordinates ~ N(0, 1/dim)."""
    bnd, cent = _lloyd_max_codebook_unscaled(bits)
    s = 1.0 / math.sqrt(dim)
    return torch.tensor(bnd * s, dtype=torch.float32), torch.tensor(cent * s, dtype=torch.float32)


def make_rotation_matrix(dim: int, seed: int = 42, method: str = "dense_qr") -> torch.Tensor:
    """Random orthogonal (dim, dim) float32 matrix: "dense_qr" (paper) or "rht" (Hadamard based)."""
    if method == "dense_qr":
        gauss = np.random.RandomState(seed).randn(dim, dim).astype(np.float32)
        q, r = np.linalg.qr(gauss)
        flip = np.sign(np.diag(r))
        flip[flip == 0] = 1.0  # keeps Q unique: diag(R) > 0
        return torch.from_numpy(np.ascontiguousarray(q * flip[None, :]))
    if method == "rht":
        return make_rht_rotation(dim, seed)
    raise ValueError(f"Unknown rotation method: {method}")


def make_rht_rotation(dim: int, seed: int = 42) -> torch.Tensor:
    """Randomised Hadamard rotation as an explicit matrix: H D cropped to (dim, dim), then QR."""
    gen = torch.Generator().manual_seed(seed)
    size = 1 << max(0, (dim - 1).bit_length())
    coin = torch.randint(0, 2, (size,), generator=gen).bool()
    diag = torch.where(coin, torch.ones(size), -torch.ones(size))
    had = torch.ones(1, 1)
    while had.shape[0] < size:
        had = torch.cat([torch.cat([had, had], dim=1), torch.cat([had, -had], dim=1)], dim=0)
    mat = ((had / math.sqrt(size)) @ torch.diag(diag))[:dim, :dim]
    q, r = torch.linalg.qr(mat)
    flip = torch.sign(torch.diag(r))
    flip[flip == 0] = 1.0
    return (q * flip.unsqueeze(0)).float()


def _make_qjl_matrix(dim: int, n_sign_bits: int, seed: int, device) -> torch.Tensor:
    """Gaussian QJL projection S (n_sign_bits, dim); torch CPU generator seeded with seed + 12345."""
    gen = torch.Generator(device="cpu").manual_seed(seed + 12345)
    return torch.randn(n_sign_bits, dim, generator=gen, dtype=torch.float32).to(device)


def _packed_dim(dim: int, bits: int) -> int:
    return bits * ((dim + 7) // 8)


# --------------------------------------------------------------------------------------------
# pack / unpack
# --------------------------------------------------------------------------------------------

def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """(N, d) codes in [0, 2^bits) -> (N, bits * ceil(d/8)) uint8 bit planes."""
    home = codes.device
    c = N.to_device(codes).to(torch.uint8).contiguous()
    n, d = c.shape
    out = torch.empty((n, _packed_dim(d, bits)), dtype=torch.uint8, device=c.device)
    with torch.cuda.device(c.device):
        N.check(N.lib().tqb_pack_codes(N.ptr(c), n, d, bits, N.ptr(out), N.stream_of(c)))
    return out.to(home)


def unpack_codes(packed: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    """(N, bits * ceil(dim/8)) uint8 -> (N, dim) uint8 codes."""
    home = packed.device
    p = N.to_device(packed).contiguous()
    if p.dim() != 2 or p.shape[1] != _packed_dim(dim, bits):
        raise RuntimeError(f"packed dim mismatch: expected {_packed_dim(dim, bits)} got {tuple(p.shape)}")
    n = p.shape[0]
    out = torch.empty((n, dim), dtype=torch.uint8, device=p.device)
    with torch.cuda.device(p.device):
        N.check(N.lib().tqb_unpack_codes(N.ptr(p), n, dim, bits, N.ptr(out), N.stream_of(p)))
    return out.to(home)


# --------------------------------------------------------------------------------------------
# Algorithm 1
# --------------------------------------------------------------------------------------------

def _rows(vectors: torch.Tensor, d: int) -> torch.Tensor:
    flat = vectors.reshape(-1, d)
    if flat.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        flat = flat.float()
    if flat.stride(-1) != 1 or (flat.shape[0] > 1 and flat.stride(0) < d):
        flat = flat.contiguous()
    return flat


def quantize_mse(
    vectors: torch.Tensor,
    bits: int,
    dim: Optional[int] = None,
    rotation: Optional[torch.Tensor] = None,
    codebook: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    seed: int = 42,
    rotation_method: str = "dense_qr",
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Algorithm 1: (packed codes (N, bits*ceil(d/8)) uint8, norms (N,) float32)."""
    d = dim if dim is not None else vectors.shape[-1]
    home = vectors.device
    x = _rows(N.to_device(vectors), d)
    dev = x.device
    if rotation is None:
        rotation = make_rotation_matrix(d, seed=seed, method=rotation_method)
    if codebook is None:
        codebook = lloyd_max_codebook(bits, d)
    rot = N.f32c(rotation, dev)
    bnd = N.f32c(codebook[0], dev)
    if bnd.numel() != (1 << bits) - 1:
        raise RuntimeError("boundaries length must be 2^bit_width - 1")
    n = x.shape[0]
    packed = torch.empty((n, _packed_dim(d, bits)), dtype=torch.uint8, device=dev)
    norms = torch.empty((n,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        N.check(N.lib().tqb_quantize_mse(N.ptr(x), N.dtype_code(x.dtype), n, d, x.stride(0) if n > 1 else d,
                                         N.ptr(rot), N.ptr(bnd), bits, N.ptr(packed), N.ptr(norms), None,
                                         N.stream_of(x)))
    return packed.to(home), norms.to(home)


def dequantize_mse(
    packed_codes: torch.Tensor,
    norms: torch.Tensor,
    bits: int,
    dim: int,
    rotation: Optional[torch.Tensor] = None,
    codebook: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    seed: int = 42,
    rotation_method: str = "dense_qr",
) -> torch.Tensor:
    """Inverse of Algorithm 1: (N, dim) reconstruction in the dtype of `norms`."""
    home = packed_codes.device
    p = N.to_device(packed_codes).contiguous()
    dev = p.device
    out_dtype = norms.dtype if norms.dtype in (torch.float16, torch.bfloat16) else torch.float32
    nr = N.f32c(N.to_device(norms, dev), dev)
    if rotation is None:
        rotation = make_rotation_matrix(dim, seed=seed, method=rotation_method)
    if codebook is None:
        codebook = lloyd_max_codebook(bits, dim)
    rot, cent = N.f32c(rotation, dev), N.f32c(codebook[1], dev)
    if p.dim() != 2 or p.shape[1] != _packed_dim(dim, bits):
        raise RuntimeError(f"packed dim mismatch: expected {_packed_dim(dim, bits)} got {tuple(p.shape)}")
    n = p.shape[0]
    out = torch.empty((n, dim), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        N.check(N.lib().tqb_dequantize_mse(N.ptr(p), N.ptr(nr), n, dim, N.ptr(rot), N.ptr(cent), bits,
                                           N.ptr(out), N.dtype_code(out_dtype), N.stream_of(p)))
    return out.to(home)


# --------------------------------------------------------------------------------------------
# Algorithm 2
# --------------------------------------------------------------------------------------------

_QJL_ROT_CACHE: dict = {}


def _qjl_rot(S: torch.Tensor, rot: torch.Tensor) -> torch.Tensor:
    """S @ R^T (float64 product, rounded once): lets the kernel project the residual in rotated space."""
    key = (S.data_ptr(), rot.data_ptr(), S._version, rot._version, str(S.device))
    hit = _QJL_ROT_CACHE.get(key)
    if hit is None:
        if len(_QJL_ROT_CACHE) > 64:
            _QJL_ROT_CACHE.clear()
        hit = (S.double() @ rot.double().t()).float().contiguous()
        _QJL_ROT_CACHE[key] = hit
    return hit


def quantize_prod(
    vectors: torch.Tensor,
    bits: int,
    dim: Optional[int] = None,
    rotation: Optional[torch.Tensor] = None,
    codebook: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    S_matrix: Optional[torch.Tensor] = None,
    seed: int = 42,
    rotation_method: str = "dense_qr",
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Algorithm 2: (mse_packed at bits-1, qjl_signs (N, ceil(d/8)), residual_norms (N,), norms (N,))."""
    d = dim if dim is not None else vectors.shape[-1]
    mse_bits = bits - 1
    if mse_bits < 1:
        raise ValueError(f"Prod mode requires bits >= 2, got {bits}")
    home = vectors.device
    x = _rows(N.to_device(vectors), d)
    dev = x.device
    if codebook is None:
        codebook = lloyd_max_codebook(mse_bits, d)
    if rotation is None:
        rotation = make_rotation_matrix(d, seed=seed, method=rotation_method)
    if S_matrix is None:
        S_matrix = _make_qjl_matrix(d, d, seed, dev)
    rot, S = N.f32c(rotation, dev), N.f32c(S_matrix, dev)
    bnd, cent = N.f32c(codebook[0], dev), N.f32c(codebook[1], dev)
    srt = _qjl_rot(S, rot)
    n = x.shape[0]
    mp = torch.empty((n, _packed_dim(d, mse_bits)), dtype=torch.uint8, device=dev)
    sg = torch.empty((n, _packed_dim(d, 1)), dtype=torch.uint8, device=dev)
    rn = torch.empty((n,), dtype=torch.float32, device=dev)
    nm = torch.empty((n,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        N.check(N.lib().tqb_quantize_prod(N.ptr(x), N.dtype_code(x.dtype), n, d, x.stride(0) if n > 1 else d,
                                          N.ptr(rot), N.ptr(bnd), N.ptr(cent), N.ptr(srt), bits, N.ptr(mp),
                                          N.ptr(sg), N.ptr(rn), N.ptr(nm), N.stream_of(x)))
    return mp.to(home), sg.to(home), rn.to(home), nm.to(home)


def dequantize_prod(
    mse_packed: torch.Tensor,
    qjl_signs: torch.Tensor,
    residual_norms: torch.Tensor,
    norms: torch.Tensor,
    bits: int,
    dim: int,
    rotation: Optional[torch.Tensor] = None,
    codebook: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    S_matrix: Optional[torch.Tensor] = None,
    seed: int = 42,
    rotation_method: str = "dense_qr",
) -> torch.Tensor:
    """Inverse of Algorithm 2: mse part + sqrt(pi/2)/dim * ||r|| * (signs @ S), times the norm."""
    home = mse_packed.device
    mp = N.to_device(mse_packed).contiguous()
    dev = mp.device
    out_dtype = norms.dtype if norms.dtype in (torch.float16, torch.bfloat16) else torch.float32
    sg = N.to_device(qjl_signs, dev).contiguous()
    rn = N.f32c(N.to_device(residual_norms, dev), dev)
    nm = N.f32c(N.to_device(norms, dev), dev)
    mse_bits = bits - 1
    if codebook is None:
        codebook = lloyd_max_codebook(mse_bits, dim)
    if rotation is None:
        rotation = make_rotation_matrix(dim, seed=seed, method=rotation_method)
    if S_matrix is None:
        S_matrix = _make_qjl_matrix(dim, dim, seed, dev)
    rot, S, cent = N.f32c(rotation, dev), N.f32c(S_matrix, dev), N.f32c(codebook[1], dev)
    n = mp.shape[0]
    out = torch.empty((n, dim), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        N.check(N.lib().tqb_dequantize_prod(N.ptr(mp), N.ptr(sg), N.ptr(rn), N.ptr(nm), n, dim, N.ptr(rot),
                                            N.ptr(cent), N.ptr(S), bits, N.ptr(out), N.dtype_code(out_dtype),
                                            N.stream_of(mp)))
    return out.to(home)
