"""The packed KV store shared by QuantizedKVCache, TurboQuantCache and the paged vLLM cache.

Keys and values live in 16-token RECORDS laid out for the decode kernel (include/tqb200.h describes
the layout; it holds the same codes and bytes per token as upstream's bit-plane rows).  A token SLOT
is the flat index ``unit * pitch + position``; ``unit`` is (sequence, head) for contiguous caches and
(block, head) for paged pools, ``pitch`` a multiple of 16.  This class owns the rotation matrices and
codebooks of one cache configuration and wraps the four C entry points that touch records: append,
export (records -> upstream rows), import (upstream rows -> records) and the fused decode attention.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _native as N
from .reference import lloyd_max_codebook, make_rotation_matrix


STATUS_WAIT_EXPIRED, STATUS_NO_SMEM, STATUS_UNIT_FULL, STATUS_LEN_CLAMPED = 1, 2, 4, 8   # TQB_DECODE_* of tqb200.h


def pad16(n: int) -> int:
    return (n + 15) // 16 * 16


class PackedKVStore:
    def __init__(self, head_dim: int, key_bits: int, value_bits: int, seed: int, rotation: str, device):
        self.head_dim, self.key_bits, self.value_bits = head_dim, key_bits, value_bits
        self.device = torch.device(device)
        self.record_bytes = int(N.lib().tqb_kv_record_bytes(head_dim, key_bits, value_bits))
        if self.record_bytes == 0:
            raise RuntimeError(f"packed KV store: head_dim must be 64 or 128 and bits 2..4 "
                               f"(got head_dim={head_dim}, K{key_bits}/V{value_bits})")
        dev = self.device
        self.key_rotation = make_rotation_matrix(head_dim, seed=seed, method=rotation).to(dev)
        self.val_rotation = make_rotation_matrix(head_dim, seed=seed + 1, method=rotation).to(dev)
        self.key_codebook = tuple(t.to(dev) for t in lloyd_max_codebook(key_bits, head_dim))
        self.val_codebook = tuple(t.to(dev) for t in lloyd_max_codebook(value_bits, head_dim))
        bpp = head_dim // 8
        self.pk, self.pv = key_bits * bpp, value_bits * bpp
        self._workspace: Optional[torch.Tensor] = None

    def alloc(self, units: int, pitch: int) -> torch.Tensor:
        """Zeroed records for `units` units of `pitch` token slots each."""
        assert pitch % 16 == 0
        return torch.zeros(units, pitch // 16, self.record_bytes, dtype=torch.uint8, device=self.device)

    # ---- append -----------------------------------------------------------------------------
    def append(self, store: torch.Tensor, key: torch.Tensor, value: torch.Tensor, rowmap: N.RowMap) -> None:
        """key / value: (..., head_dim) contiguous, same shape; input row r goes to slot rowmap(r)."""
        k = key.to(self.device)
        if k.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            k = k.float()
        k = k.contiguous()
        v = value.to(self.device, k.dtype).contiguous()
        n = k.numel() // self.head_dim
        with torch.cuda.device(self.device):
            N.check(N.lib().tqb_kv_append(
                N.ptr(k), N.ptr(v), N.dtype_code(k.dtype), n, self.head_dim, self.head_dim,
                N.ptr(self.key_rotation), N.ptr(self.key_codebook[0]), self.key_bits,
                N.ptr(self.val_rotation), N.ptr(self.val_codebook[0]), self.value_bits,
                N.ptr(store), rowmap, N.stream_of(k)))

    # ---- upstream-layout views ------------------------------------------------------------------
    def export_rows(self, store: torch.Tensor, n: int, rowmap: N.RowMap, keys: bool = True, values: bool = True):
        """(k_packed (n, pk) u8, k_norms (n,), v_packed (n, pv) u8, v_norms (n,)) of slots rowmap(0..n-1)."""
        dev = self.device
        kp = torch.empty(n, self.pk, dtype=torch.uint8, device=dev) if keys else None
        kn = torch.empty(n, dtype=torch.float32, device=dev) if keys else None
        vp = torch.empty(n, self.pv, dtype=torch.uint8, device=dev) if values else None
        vn = torch.empty(n, dtype=torch.float32, device=dev) if values else None
        with torch.cuda.device(dev):
            N.check(N.lib().tqb_kv_export(N.ptr(store), n, self.head_dim, self.key_bits, self.value_bits, rowmap,
                                          N.ptr(kp), N.ptr(kn), N.ptr(vp), N.ptr(vn), N.stream_of(store)))
        return kp, kn, vp, vn

    def import_rows(self, store: torch.Tensor, rowmap: N.RowMap, k_packed=None, k_norms=None, v_packed=None,
                    v_norms=None) -> None:
        """Write upstream-layout rows (any subset) into slots rowmap(0..n-1)."""
        dev = self.device
        prep = lambda t, dt: None if t is None else t.to(dev, dt).contiguous()
        kp, vp = prep(k_packed, torch.uint8), prep(v_packed, torch.uint8)
        kn, vn = prep(k_norms, torch.float32), prep(v_norms, torch.float32)
        n = next(t for t in (kp, vp, kn, vn) if t is not None).shape[0]
        with torch.cuda.device(dev):
            N.check(N.lib().tqb_kv_import(N.ptr(store), n, self.head_dim, self.key_bits, self.value_bits, rowmap,
                                          N.ptr(kp), N.ptr(kn), N.ptr(vp), N.ptr(vn), N.stream_of(store)))

    def dequantize(self, packed: torch.Tensor, norms: torch.Tensor, which: str, dtype=torch.float32) -> torch.Tensor:
        """Dense (n, head_dim) reconstruction of exported rows; which = "key" | "value"."""
        n = packed.shape[0]
        rot = self.key_rotation if which == "key" else self.val_rotation
        cent = (self.key_codebook if which == "key" else self.val_codebook)[1]
        bits = self.key_bits if which == "key" else self.value_bits
        out = torch.empty(n, self.head_dim, dtype=dtype, device=self.device)
        with torch.cuda.device(self.device):
            N.check(N.lib().tqb_dequantize_mse(N.ptr(packed), N.ptr(norms), n, self.head_dim, N.ptr(rot), N.ptr(cent),
                                               bits, N.ptr(out), N.dtype_code(dtype), N.stream_of(packed)))
        return out

    # ---- fused decode attention -------------------------------------------------------------------
    def decode_attention(self, store: torch.Tensor, query: torch.Tensor, kv_heads: int, seq_lens: torch.Tensor,
                         max_len: int, pitch: int = 0, block_tables: Optional[torch.Tensor] = None,
                         block_size: int = 0, scale: Optional[float] = None,
                         out: Optional[torch.Tensor] = None, reserve_len: int = 0) -> torch.Tensor:
        """query (batch, q_heads, head_dim) -> (batch, q_heads, head_dim) in the query's dtype."""
        q = query.to(self.device)
        if q.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            q = q.float()
        q = q.contiguous()
        B, HQ, D = q.shape
        L = N.lib()
        need = max(L.tqb_decode_attention_workspace_bytes(B, HQ, kv_heads, D, max_len),
                   L.tqb_decode_attention_workspace_bytes(B, HQ, kv_heads, D, max(reserve_len, max_len)))
        if need == 0:
            raise RuntimeError(f"decode_attention: {HQ} query heads do not fit {kv_heads} KV heads")
        self._reserve_workspace(need)
        res = out if out is not None else torch.empty_like(q)
        paged = block_tables is not None
        with torch.cuda.device(self.device):
            N.check(L.tqb_decode_attention(
                N.ptr(q), N.dtype_code(q.dtype), B, HQ, kv_heads, D, N.ptr(store), pitch, N.ptr(seq_lens), max_len,
                N.ptr(block_tables) if paged else None, block_tables.shape[1] if paged else 0, block_size,
                N.ptr(self.key_rotation), N.ptr(self.key_codebook[1]), self.key_bits,
                N.ptr(self.val_rotation), N.ptr(self.val_codebook[1]), self.value_bits,
                float(scale if scale is not None else 1.0 / math.sqrt(D)),
                N.ptr(self._workspace), self._workspace.numel(), N.ptr(res), N.dtype_code(res.dtype), N.stream_of(q)))
        return res

    def decode_step(self, store: torch.Tensor, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                    kv_heads: int, seq_lens: torch.Tensor, max_len: int, pitch: int, scale: Optional[float] = None,
                    out: Optional[torch.Tensor] = None, reserve_len: int = 0) -> torch.Tensor:
        """Append one token per sequence and attend to it and everything before it, in one launch.

        query (batch, q_heads, head_dim); key / value (batch, kv_heads, head_dim), same dtype as the query.
        ``seq_lens`` (device int32) gives the write position and is advanced by one on the device;
        ``max_len`` bounds the new lengths."""
        q = query.to(self.device)
        if q.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            q = q.float()
        q = q.contiguous()
        k = key.to(device=self.device, dtype=q.dtype).contiguous()
        v = value.to(device=self.device, dtype=q.dtype).contiguous()
        B, HQ, D = q.shape
        if k.shape != (B, kv_heads, D) or v.shape != k.shape:
            raise RuntimeError(f"decode_step: key/value must be ({B}, {kv_heads}, {D}), got {tuple(k.shape)}")
        L = N.lib()
        need = max(L.tqb_decode_attention_workspace_bytes(B, HQ, kv_heads, D, max_len),
                   L.tqb_decode_attention_workspace_bytes(B, HQ, kv_heads, D, max(reserve_len, max_len)))
        if need == 0:
            raise RuntimeError(f"decode_step: {HQ} query heads do not fit {kv_heads} KV heads")
        self._reserve_workspace(need)
        res = out if out is not None else torch.empty_like(q)
        with torch.cuda.device(self.device):
            N.check(L.tqb_decode_step(
                N.ptr(q), N.ptr(k), N.ptr(v), N.dtype_code(q.dtype), D, B, HQ, kv_heads, D, N.ptr(store), pitch,
                N.ptr(seq_lens), max_len,
                N.ptr(self.key_rotation), N.ptr(self.key_codebook[0]), N.ptr(self.key_codebook[1]), self.key_bits,
                N.ptr(self.val_rotation), N.ptr(self.val_codebook[0]), N.ptr(self.val_codebook[1]), self.value_bits,
                float(scale if scale is not None else 1.0 / math.sqrt(D)),
                N.ptr(self._workspace), self._workspace.numel(), N.ptr(res), N.dtype_code(res.dtype), N.stream_of(q)))
        return res

    def _reserve_workspace(self, need: int) -> None:
        """The decode workspace starts zeroed (status word, arrival counters); the kernel keeps it clean."""
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.zeros(need, dtype=torch.uint8, device=self.device)

    def status(self) -> int:
        """Status bits raised by the decode calls since the last status() (synchronises, then clears them):
        0 = all good; STATUS_WAIT_EXPIRED / STATUS_NO_SMEM = results invalid (the workspace is re-zeroed here);
        STATUS_UNIT_FULL = a fused step found a full unit and dropped its token; STATUS_LEN_CLAMPED = a
        sequence length outside the announced bounds was clamped."""
        if self._workspace is None:
            return 0
        word = self._workspace[:4].view(torch.int32)
        value = int(word.item())
        if value & (STATUS_WAIT_EXPIRED | STATUS_NO_SMEM):
            self._workspace.zero_()
        elif value:
            word.zero_()
        return value
