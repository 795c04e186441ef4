"""QuantizedKVCache -- packed TurboQuant KV cache, B200 build.

Same constructor and methods as upstream ``turboquant_kv/cache.py:29-381`` (``append``,
``attention_scores``, ``attention_values``, ``_dequantize_keys/_values``, ``memory_bytes``,
``compression_ratio``).  Storage is written by the fused quantise kernels and read by kernels that
work on the packed codes; nothing is dequantised to attend.

Storage layout: quantised layers live in the 16-token record layout of ``kvstore.PackedKVStore``
(same codes, same bytes per token as upstream, ordered for the decode kernel).  The upstream
attributes ``_key_packed / _key_norms / _val_packed / _val_norms`` are still there, as read-only
upstream-layout COPIES produced on access; ``load_packed`` writes upstream-layout rows back.

Additions for serving (none changes upstream behaviour):
  * ``batch_size=B`` gives every sequence of a batch its own cache rows (upstream keeps a single
    sequence and silently drops ``key[1:]``, cache.py:157-160 -- still the behaviour when
    ``batch_size`` is left at None);
  * ``decode_attention(layer, query)``: the fused one-token decode step (scores, softmax, values,
    grouped-query heads) in one kernel launch;
  * per-layer sequence lengths also live on the device so the decode path never synchronises.

Prod mode: upstream allocates ``key_bits`` planes per token but ``quantize_prod`` returns
``key_bits - 1`` (cache.py:84-85 vs reference.py:441), so its ``append`` raises in that mode.  This
build raises the same kind of error, with a message that says why.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _native as N
from .config import TurboQuantConfig
from .kvstore import PackedKVStore, pad16 as _pad16
from .reference import _make_qjl_matrix, lloyd_max_codebook, make_rotation_matrix


class QuantizedKVCache:
    """Pre-allocated packed keys/values for all layers of one model (or one tensor-parallel shard)."""

    def __init__(self, config: TurboQuantConfig, num_layers: int, max_seq_len: int, num_heads: int,
                 head_dim: int, device: str = "cuda", batch_size: Optional[int] = None):
        N.require_cuda()
        self.config = config
        self.num_layers = num_layers
        self.max_seq_len = max_seq_len
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("QuantizedKVCache (B200 build) lives on a CUDA device; there is no CPU path")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        if config.mode not in ("mse", "prod"):
            raise ValueError(f"Unknown mode: {config.mode}")
        self.batch_size = batch_size
        self._batch = 1 if batch_size is None else int(batch_size)
        self._pitch = _pad16(max_seq_len)  # rows per (sequence, head); tiles of 16 never straddle units

        self.seq_lens = torch.zeros(num_layers, dtype=torch.long)  # host copy, as upstream
        self._seq_lens_dev = torch.zeros(num_layers, self._batch, dtype=torch.int32, device=self.device)

        dev = self.device
        self._key_rotation = make_rotation_matrix(head_dim, seed=config.seed, method=config.rotation).to(dev)
        self._val_rotation = make_rotation_matrix(head_dim, seed=config.seed + 1, method=config.rotation).to(dev)
        self._key_codebook = lloyd_max_codebook(config.key_bits, head_dim)
        self._val_codebook = lloyd_max_codebook(config.value_bits, head_dim)
        self._kb_dev = tuple(t.to(dev) for t in self._key_codebook)
        self._vb_dev = tuple(t.to(dev) for t in self._val_codebook)

        self._has_outliers = config.outlier_channels > 0
        if self._has_outliers:  # built and unused, exactly like upstream
            self._key_codebook_outlier = lloyd_max_codebook(config.key_bits + 1, head_dim)
            self._val_codebook_outlier = lloyd_max_codebook(config.value_bits + 1, head_dim)

        self._is_prod = config.mode == "prod"
        if self._is_prod:
            self._key_S = _make_qjl_matrix(head_dim, head_dim, config.seed, dev)
            self._val_S = _make_qjl_matrix(head_dim, head_dim, config.seed + 1, dev)
            self._key_codebook_prod = lloyd_max_codebook(config.key_bits - 1, head_dim)
            self._val_codebook_prod = lloyd_max_codebook(config.value_bits - 1, head_dim)

        bpp = (head_dim + 7) // 8
        self._pk, self._pv = config.key_bits * bpp, config.value_bits * bpp
        B, H = self._batch, num_heads
        self._kv: Optional[PackedKVStore] = None
        self._store = []
        if not self._is_prod:
            self._kv = PackedKVStore(head_dim, config.key_bits, config.value_bits, config.seed, config.rotation, dev)
            self._store = [self._kv.alloc(B * H, self._pitch) for _ in range(num_layers)]

        self._protected = config.protected_layers > 0
        if self._protected:
            self._key_fp = [torch.zeros(B, H, max_seq_len, head_dim, dtype=torch.float16, device=dev)
                            for _ in range(config.protected_layers)]
            self._val_fp = [torch.zeros(B, H, max_seq_len, head_dim, dtype=torch.float16, device=dev)
                            for _ in range(config.protected_layers)]

    # ---- upstream-shaped copies of the storage: (num_heads, max_seq_len, ...) when batch_size is None
    def _export(self, layer_id: int, seq: int, keys: bool = True, values: bool = True):
        """Upstream-layout rows of the first `seq` tokens of every (sequence, head): each (B*H*seq, ...)."""
        rm = N.RowMap(max(seq, 1), self._pitch, 1, 0, None, 1, None, 1)
        return self._kv.export_rows(self._store[layer_id], self._batch * self.num_heads * seq, rm, keys, values)

    def _upstream_view(self, which: int):
        B, H, S = self._batch, self.num_heads, self.max_seq_len
        out = []
        for layer in range(self.num_layers):
            t = self._export(layer, S, keys=which < 2, values=which >= 2)[which]
            t = t.view(B, H, S, -1) if t.dim() == 2 else t.view(B, H, S)
            out.append(t[0] if self.batch_size is None else t)
        return out

    @property
    def _key_packed(self):
        return self._upstream_view(0)

    @property
    def _key_norms(self):
        return self._upstream_view(1)

    @property
    def _val_packed(self):
        return self._upstream_view(2)

    @property
    def _val_norms(self):
        return self._upstream_view(3)

    def load_packed(self, layer_id: int, k_packed=None, k_norms=None, v_packed=None, v_norms=None) -> None:
        """Write upstream-layout rows into the cache: tensors shaped ([batch,] heads, seq, ...), the first
        `seq` tokens of every (sequence, head).  Sets the layer's length to `seq`."""
        first = next(t for t in (k_norms, v_norms, k_packed, v_packed) if t is not None)
        seq = first.shape[-1] if first.dtype != torch.uint8 else first.shape[-2]
        flat = lambda t, last: None if t is None else (t.reshape(-1, t.shape[-1]) if last else t.reshape(-1))
        rm = N.RowMap(max(seq, 1), self._pitch, 1, 0, None, 1, None, 1)
        self._kv.import_rows(self._store[layer_id], rm, flat(k_packed, True), flat(k_norms, False),
                             flat(v_packed, True), flat(v_norms, False))
        self.seq_lens[layer_id] = seq
        self._seq_lens_dev[layer_id] = seq

    def _is_protected_layer(self, layer_id: int) -> bool:
        return self._protected and layer_id < self.config.protected_layers

    # ------------------------------------------------------------------------------------------
    def append(self, layer_id: int, key: torch.Tensor, value: torch.Tensor):
        """Quantise and store new tokens.

        key / value: (num_heads, new, head_dim), or (batch, num_heads, new, head_dim).  Without
        ``batch_size`` only batch item 0 is kept (upstream behaviour); with it, ``batch`` must match.
        """
        if key.dim() == 4:
            if self.batch_size is None:
                key, value = key[:1], value[:1]
            elif key.shape[0] != self._batch:
                raise RuntimeError(f"expected batch {self._batch}, got {key.shape[0]}")
        else:
            assert key.dim() == 3, f"Expected 3D key, got {key.dim()}D"
            if self._batch != 1:
                raise RuntimeError("a batched cache needs (batch, heads, new, head_dim) inputs")
            key, value = key.unsqueeze(0), value.unsqueeze(0)
        B, H, T, D = key.shape
        if H != self.num_heads or D != self.head_dim:
            raise RuntimeError(f"expected (*, {self.num_heads}, new, {self.head_dim}), got {tuple(key.shape)}")
        pos = int(self.seq_lens[layer_id])
        if pos + T > self.max_seq_len:
            raise RuntimeError(f"cache overflow: {pos} + {T} > max_seq_len {self.max_seq_len}")

        if self._is_protected_layer(layer_id):
            self._key_fp[layer_id][:, :, pos:pos + T] = key.to(self.device).half()
            self._val_fp[layer_id][:, :, pos:pos + T] = value.to(self.device).half()
        elif self._is_prod:
            raise RuntimeError(
                "QuantizedKVCache in prod mode: upstream stores key_bits planes per token but quantize_prod "
                "yields key_bits - 1, so upstream append() fails with a shape error; not supported here either")
        else:
            # rows are (batch*head, token); the write position is read on the device so that a captured
            # CUDA graph of a decode step keeps appending at the right place when replayed
            rm = N.RowMap(T, self._pitch, 1, 0, N.ptr(self._seq_lens_dev[layer_id]), H, None, 1)
            self._kv.append(self._store[layer_id], self._as_rows(key), self._as_rows(value), rm)
        self.seq_lens[layer_id] += T
        self._seq_lens_dev[layer_id] += T

    def _as_rows(self, x: torch.Tensor) -> torch.Tensor:
        x = x.to(self.device)
        if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            x = x.float()
        return x.contiguous()

    # ------------------------------------------------------------------------------------------
    def _dequantize(self, layer_id: int, which: str, fp_store):
        seq = int(self.seq_lens[layer_id])
        B, H, D = self._batch, self.num_heads, self.head_dim
        if seq == 0:
            out = torch.zeros(B, H, 0, D, dtype=torch.float32, device=self.device)
        elif self._is_protected_layer(layer_id):
            out = fp_store[layer_id][:, :, :seq].float()
        else:
            kp, kn, vp, vn = self._export(layer_id, seq, keys=which == "key", values=which == "value")
            out = self._kv.dequantize(kp if which == "key" else vp, kn if which == "key" else vn, which)
            out = out.view(B, H, seq, D)
        return out[0] if self.batch_size is None else out

    def _dequantize_keys(self, layer_id: int) -> torch.Tensor:
        """Dense keys (num_heads, seq, head_dim) float32 (with a leading batch dim for batched caches)."""
        return self._dequantize(layer_id, "key", getattr(self, "_key_fp", None))

    def _dequantize_values(self, layer_id: int) -> torch.Tensor:
        return self._dequantize(layer_id, "value", getattr(self, "_val_fp", None))

    # ------------------------------------------------------------------------------------------
    def attention_scores(self, layer_id: int, query: torch.Tensor) -> torch.Tensor:
        """Logits q.k / sqrt(head_dim) straight from the packed keys.

        query: (batch, num_heads, seq_q, head_dim) or (num_heads, seq_q, head_dim); every batch item
        attends to the same cached sequence (upstream semantics).  Returns (..., seq_q, seq_kv).
        """
        if self._batch != 1:
            raise RuntimeError("attention_scores follows upstream's single-sequence semantics; "
                               "use decode_attention on a batched cache")
        has_batch = query.dim() == 4
        q = query if has_batch else query.unsqueeze(0)
        q = q.reshape(q.shape[0], self.num_heads, -1, self.head_dim).to(self.device).float()
        nb, H, sq, D = q.shape
        seq = int(self.seq_lens[layer_id])
        scale = 1.0 / math.sqrt(D)
        if self._is_protected_layer(layer_id) or seq == 0:
            keys = self._dequantize_keys(layer_id)
            keys = keys if keys.dim() == 3 else keys[0]
            logits = torch.matmul(q, keys.transpose(-2, -1).unsqueeze(0)) * scale
        else:
            logits = torch.empty(nb, H, sq, seq, dtype=torch.float32, device=self.device)
            kp, kn, _, _ = self._export(layer_id, seq, values=False)
            kp, kn = kp.view(H, seq, -1), kn.view(H, seq)
            with torch.cuda.device(self.device):
                for h in range(H):
                    qh = q[:, h].reshape(nb * sq, D).contiguous()
                    out = torch.empty(nb * sq, seq, dtype=torch.float32, device=self.device)
                    N.check(N.lib().tqb_attention_scores_packed(
                        N.ptr(qh), nb * sq, D, N.ptr(kp[h]), N.ptr(kn[h]), seq, N.ptr(self._kb_dev[1]),
                        N.ptr(self._key_rotation), self.config.key_bits, N.ptr(out), N.stream_of(qh)))
                    logits[:, h] = out.view(nb, sq, seq)
            logits *= scale
        return logits if has_batch else logits.squeeze(0)

    def attention_values(self, layer_id: int, attn_weights: torch.Tensor) -> torch.Tensor:
        """Weighted sum of the cached values: (..., seq_q, seq_kv) -> (..., seq_q, head_dim)."""
        if self._batch != 1:
            raise RuntimeError("attention_values follows upstream's single-sequence semantics; "
                               "use decode_attention on a batched cache")
        has_batch = attn_weights.dim() == 4
        w = (attn_weights if has_batch else attn_weights.unsqueeze(0)).to(self.device).float()
        nb, H, sq, seq = w.shape
        D = self.head_dim
        if self._is_protected_layer(layer_id) or seq == 0:
            vals = self._dequantize_values(layer_id)
            vals = vals if vals.dim() == 3 else vals[0]
            out = torch.matmul(w, vals.unsqueeze(0))
        else:
            out = torch.empty(nb, H, sq, D, dtype=torch.float32, device=self.device)
            _, _, vp, vn = self._export(layer_id, seq, keys=False)
            vp, vn = vp.view(H, seq, -1), vn.view(H, seq)
            with torch.cuda.device(self.device):
                for h in range(H):
                    wh = w[:, h].reshape(nb * sq, seq).contiguous()
                    oh = torch.empty(nb * sq, D, dtype=torch.float32, device=self.device)
                    N.check(N.lib().tqb_attention_values_packed(
                        N.ptr(wh), nb * sq, seq, D, N.ptr(vp[h]), N.ptr(vn[h]), N.ptr(self._vb_dev[1]),
                        N.ptr(self._val_rotation), self.config.value_bits, N.ptr(oh), N.stream_of(wh)))
                    out[:, h] = oh.view(nb, sq, D)
        return out if has_batch else out.squeeze(0)

    # ------------------------------------------------------------------------------------------
    def decode_attention(self, layer_id: int, query: torch.Tensor, scale: Optional[float] = None,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """softmax(scale * q K^T) V for ONE new token per sequence, fused, over the packed cache.

        query: (batch, q_heads, head_dim) or (batch, q_heads, 1, head_dim); q_heads must be a multiple of
        the cache's (KV) heads -- query head h reads KV head h // group.  Returns the query's shape, in
        the query's dtype.  Stream-ordered, no host synchronisation.
        """
        if self._is_protected_layer(layer_id) or self._is_prod:
            raise RuntimeError("decode_attention covers MSE-quantised layers")
        squeeze = query.dim() == 4
        q = query[:, :, 0] if squeeze else query
        B, HQ, D = q.shape
        if B != self._batch or D != self.head_dim or HQ % self.num_heads:
            raise RuntimeError(f"query {tuple(query.shape)} does not fit cache (batch {self._batch}, "
                               f"kv heads {self.num_heads}, head_dim {self.head_dim})")
        max_len = self._pitch if torch.cuda.is_current_stream_capturing() else int(self.seq_lens[layer_id])
        res = self._kv.decode_attention(self._store[layer_id], q, self.num_heads, self._seq_lens_dev[layer_id],
                                        max_len, pitch=self._pitch, scale=scale, out=out, reserve_len=self._pitch)
        return res.unsqueeze(2) if squeeze else res

    def decode_step(self, layer_id: int, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                    scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``append`` of one token per sequence followed by ``decode_attention``, in one launch.

        query: (batch, q_heads, head_dim); key / value: (batch, num_heads, head_dim) or
        (batch, num_heads, 1, head_dim).  Same result as the two separate calls."""
        if self._is_protected_layer(layer_id) or self._is_prod:
            raise RuntimeError("decode_step covers MSE-quantised layers")
        if key.dim() == 4:
            key, value = key[:, :, 0], value[:, :, 0]
        squeeze = query.dim() == 4
        q = query[:, :, 0] if squeeze else query
        B, HQ, D = q.shape
        if B != self._batch or D != self.head_dim or HQ % self.num_heads:
            raise RuntimeError(f"query {tuple(query.shape)} does not fit cache (batch {self._batch}, "
                               f"kv heads {self.num_heads}, head_dim {self.head_dim})")
        pos = int(self.seq_lens[layer_id])
        if pos + 1 > self.max_seq_len:
            raise RuntimeError(f"cache overflow: {pos} + 1 > max_seq_len {self.max_seq_len}")
        max_len = self._pitch if torch.cuda.is_current_stream_capturing() else pos + 1
        res = self._kv.decode_step(self._store[layer_id], q, key, value, self.num_heads,
                                   self._seq_lens_dev[layer_id], max_len, self._pitch, scale=scale, out=out,
                                   reserve_len=self._pitch)
        self.seq_lens[layer_id] += 1
        return res.unsqueeze(2) if squeeze else res

    def decode_status(self) -> int:
        """Status bits raised by decode calls since the last query (kvstore.PackedKVStore.status); 0 = all good."""
        return 0 if self._kv is None else self._kv.status()

    # ------------------------------------------------------------------------------------------
    def memory_bytes(self) -> int:
        """Bytes of packed codes + norms in use (upstream formula, cache.py:341-365), per stored sequence."""
        total = 0
        for layer_id in range(self.num_layers):
            seq = int(self.seq_lens[layer_id])
            if seq == 0:
                continue
            if self._is_protected_layer(layer_id):
                total += 2 * self.num_heads * seq * self.head_dim * 2
                continue
            per_token = self._pk + self._pv + 8
            if self._is_prod:
                per_token += 2 * ((self.head_dim + 7) // 8) + 8
            total += self.num_heads * seq * per_token
        return total * self._batch

    @property
    def compression_ratio(self) -> float:
        """fp16 bytes of the same tokens divided by memory_bytes()."""
        fp16 = sum(2 * self.num_heads * int(s) * self.head_dim * 2 for s in self.seq_lens) * self._batch
        used = self.memory_bytes()
        return fp16 / used if used else 0.0
