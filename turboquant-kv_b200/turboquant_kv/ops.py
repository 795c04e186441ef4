"""Operator-level entry points (upstream turboquant_kv/ops.py:49-246) and the ``turboquant::*`` torch
operator library (upstream csrc/registration.cpp:84-99).

Upstream tries Triton, then a compiled extension, then a pure-torch fallback.  Here every function is
one call into libtqb200.so: no Triton, no dispatch chain, no CPU path.  The five operator schemas are
registered through ``torch.library`` for CUDA tensors only, so existing
``torch.ops.turboquant.<op>(...)`` call sites keep working.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _native as N
from .reference import pack_codes as _pack, unpack_codes as _unpack

__all__ = ["pack_codes", "unpack_codes", "rotate_and_quantize", "attention_scores_packed",
           "attention_values_packed"]


def _check_bits(bit_width: int) -> None:
    if not 1 <= bit_width <= 4:
        raise RuntimeError("bit_width must be 1-4")


def pack_codes(codes: torch.Tensor, bit_width: int) -> torch.Tensor:
    if codes.dtype != torch.uint8:
        raise RuntimeError("codes must be uint8")
    if codes.dim() != 2:
        raise RuntimeError("codes must be 2D [N, d]")
    _check_bits(bit_width)
    return _pack(codes, bit_width)


def unpack_codes(packed: torch.Tensor, bit_width: int, dim: int) -> torch.Tensor:
    if packed.dtype != torch.uint8:
        raise RuntimeError("packed must be uint8")
    if packed.dim() != 2:
        raise RuntimeError("packed must be 2D")
    _check_bits(bit_width)
    return _unpack(packed, bit_width, dim)


def rotate_and_quantize(vectors: torch.Tensor, rotation: torch.Tensor, boundaries: torch.Tensor,
                        bit_width: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Fused norm + rotation + code selection + packing: (packed (N, packed_dim) uint8, norms (N,) f32)."""
    _check_bits(bit_width)
    if vectors.dim() != 2:
        raise RuntimeError("vectors must be [N, d]")
    d = vectors.shape[1]
    if rotation.shape != (d, d):
        raise RuntimeError("Rotation matrix must be [d, d]")
    if boundaries.numel() != (1 << bit_width) - 1:
        raise RuntimeError("boundaries length must be 2^bit_width - 1")
    from .reference import quantize_mse
    return quantize_mse(vectors, bit_width, dim=d, rotation=rotation, codebook=(boundaries, None))


def attention_scores_packed(query: torch.Tensor, packed_keys: torch.Tensor, key_norms: torch.Tensor,
                            centroids: torch.Tensor, rotation: torch.Tensor, bit_width: int) -> torch.Tensor:
    """Unscaled scores (batch, heads, seq) of every (batch, head) query against ONE packed key stream."""
    _check_bits(bit_width)
    if query.dim() != 3:
        raise RuntimeError("query must be [batch, heads, head_dim]")
    if packed_keys.dim() != 2:
        raise RuntimeError("packed_keys must be [seq_len, packed_dim]")
    home = query.device
    q = N.f32c(N.to_device(query), None)
    dev = q.device
    b, h, d = q.shape
    if packed_keys.shape[1] != bit_width * ((d + 7) // 8):
        raise RuntimeError("packed_keys dim mismatch")
    if centroids.numel() != (1 << bit_width):
        raise RuntimeError("centroids length must be 2^bit_width")
    if rotation.shape != (d, d):
        raise RuntimeError("Rotation matrix must be [d, d]")
    pk = N.to_device(packed_keys, dev).contiguous()
    kn, ce, ro = N.f32c(N.to_device(key_norms, dev), dev), N.f32c(centroids, dev), N.f32c(rotation, dev)
    seq = pk.shape[0]
    out = torch.empty((b, h, seq), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        N.check(N.lib().tqb_attention_scores_packed(N.ptr(q), b * h, d, N.ptr(pk), N.ptr(kn), seq, N.ptr(ce),
                                                    N.ptr(ro), bit_width, N.ptr(out), N.stream_of(q)))
    return out.to(home)


def attention_values_packed(attn_weights: torch.Tensor, packed_values: torch.Tensor, value_norms: torch.Tensor,
                            centroids: torch.Tensor, rotation_T: torch.Tensor, bit_width: int) -> torch.Tensor:
    """(batch, heads, head_dim) = (sum_s w_s * norm_s * centroids[code_s]) @ rotation_T.

    To undo the forward rotation of ``quantize_mse`` pass the rotation matrix itself as ``rotation_T``
    (x = y @ R), as upstream's own fallback does.
    """
    _check_bits(bit_width)
    if attn_weights.dim() != 3:
        raise RuntimeError("attn_weights must be [batch, heads, seq_len]")
    if packed_values.dim() != 2:
        raise RuntimeError("packed_values must be [seq_len, packed_dim]")
    home = attn_weights.device
    w = N.f32c(N.to_device(attn_weights), None)
    dev = w.device
    b, h, seq = w.shape
    d = rotation_T.shape[0]
    if packed_values.shape[0] != seq or packed_values.shape[1] != bit_width * ((d + 7) // 8):
        raise RuntimeError("packed_values shape mismatch")
    if centroids.numel() != (1 << bit_width):
        raise RuntimeError("centroids length must be 2^bit_width")
    pv = N.to_device(packed_values, dev).contiguous()
    vn, ce, rt = N.f32c(N.to_device(value_norms, dev), dev), N.f32c(centroids, dev), N.f32c(rotation_T, dev)
    out = torch.empty((b, h, d), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        N.check(N.lib().tqb_attention_values_packed(N.ptr(w), b * h, seq, d, N.ptr(pv), N.ptr(vn), N.ptr(ce),
                                                    N.ptr(rt), bit_width, N.ptr(out), N.stream_of(w)))
    return out.to(home)


# ---- torch operator library: same five schemas as upstream, CUDA implementations only ----------
_LIBRARY = None


def register_torch_ops() -> None:
    """Define ``torch.ops.turboquant.*`` (idempotent).  Raises if another build already owns the namespace."""
    global _LIBRARY
    if _LIBRARY is not None:
        return
    lib = torch.library.Library("turboquant", "DEF")
    lib.define("rotate_and_quantize(Tensor vectors, Tensor rotation, Tensor boundaries, int bit_width)"
               " -> (Tensor, Tensor)")
    lib.define("attention_scores_packed(Tensor query, Tensor packed_keys, Tensor key_norms,"
               " Tensor centroids, Tensor rotation, int bit_width) -> Tensor")
    lib.define("attention_values_packed(Tensor attn_weights, Tensor packed_values, Tensor value_norms,"
               " Tensor centroids, Tensor rotation_T, int bit_width) -> Tensor")
    lib.define("pack_codes(Tensor codes, int bit_width) -> Tensor")
    lib.define("unpack_codes(Tensor packed, int bit_width, int dim) -> Tensor")
    lib.impl("rotate_and_quantize", rotate_and_quantize, "CUDA")
    lib.impl("attention_scores_packed", attention_scores_packed, "CUDA")
    lib.impl("attention_values_packed", attention_values_packed, "CUDA")
    lib.impl("pack_codes", pack_codes, "CUDA")
    lib.impl("unpack_codes", unpack_codes, "CUDA")
    _LIBRARY = lib
