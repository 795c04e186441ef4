"""vLLM-facing classes -- B200 build of upstream ``turboquant_kv/vllm_plugin/__init__.py``.

Same names and method signatures (``TurboQuantKVCacheConfig`` :67, ``TurboQuantPagedKVCache`` :114,
``TurboQuantAttentionImpl`` :312, ``TurboQuantAttentionBackend`` :420, ``register`` :469).  Upstream's
cache is paged in name only (it wraps one contiguous single-sequence cache and never uses block
tables or slot mappings, :114-304).  Here the pool really is paged:

    (num_blocks * kv_heads, block_size / 16, record_bytes) uint8: 16-token records of key codes, value
    codes and both norms per (block, head), in the layout of ``kvstore.PackedKVStore``

``append_slots`` scatters freshly quantised tokens through a vLLM slot mapping in one launch and
``paged_decode_attention`` runs the fused decode kernel through block tables (grouped-query heads,
per-sequence lengths).  The upstream-style methods (``append`` / ``attention_scores`` /
``attention_values`` / ``get_keys`` ...) keep their single-sequence meaning: tokens fill the pool in
block order.

vLLM itself is not imported at module import (it takes several seconds and the classes work
without it); ``register()`` looks for a backend registry when called.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Type

import torch

from .. import _native as N
from ..config import TurboQuantConfig
from ..kvstore import PackedKVStore


class AttentionBackend:  # stand-ins for vLLM's abstract bases (duck-typed by the engine)
    pass


class AttentionImpl:
    pass


class AttentionMetadata:
    pass


@dataclass
class TurboQuantKVCacheConfig:
    """TurboQuant settings plus vLLM's paging parameters."""

    key_bits: int = 4
    value_bits: int = 2
    mode: str = "mse"
    rotation: str = "dense_qr"
    block_size: int = 16
    num_gpu_blocks: int = 0
    num_cpu_blocks: int = 0
    protected_layers: int = 0
    seed: int = 42

    def to_turboquant_config(self) -> TurboQuantConfig:
        return TurboQuantConfig(key_bits=self.key_bits, value_bits=self.value_bits, mode=self.mode,
                                rotation=self.rotation, protected_layers=self.protected_layers,
                                quantize_on_append=True, seed=self.seed)


class TurboQuantPagedKVCache:
    """Paged pools of packed K/V codes for all layers."""

    def __init__(self, config: TurboQuantKVCacheConfig, num_layers: int, num_heads: int, head_dim: int,
                 dtype: torch.dtype = torch.float16, device: str = "cuda") -> None:
        N.require_cuda()
        if config.mode != "mse":
            raise RuntimeError("TurboQuantPagedKVCache (B200 build) implements mode='mse'")
        if config.block_size % 16:
            raise ValueError("block_size must be a multiple of 16")
        self.config, self.num_layers, self.num_heads, self.head_dim = config, num_layers, num_heads, head_dim
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.block_size = config.block_size
        self.tq_config = config.to_turboquant_config()
        self.kv = PackedKVStore(head_dim, config.key_bits, config.value_bits, config.seed, config.rotation, self.device)
        self._key_rotation, self._val_rotation = self.kv.key_rotation, self.kv.val_rotation
        self._kb, self._vb = self.kv.key_codebook, self.kv.val_codebook
        self._pk, self._pv = self.kv.pk, self.kv.pv
        self._total_blocks = 0
        self._max_tokens = 0
        self._pools: List[torch.Tensor] = []
        self._seq_len = [0] * num_layers          # upstream-style single-sequence fill level per layer
        if config.num_gpu_blocks > 0:
            self.allocate(config.num_gpu_blocks, config.num_cpu_blocks)

    def allocate(self, num_gpu_blocks: int, num_cpu_blocks: int = 0) -> None:
        """(Re)allocate the pools for `num_gpu_blocks` pages."""
        self._total_blocks, self._max_tokens = num_gpu_blocks, num_gpu_blocks * self.block_size
        self._pools = [self.kv.alloc(num_gpu_blocks * self.num_heads, self.block_size) for _ in range(self.num_layers)]
        self._seq_len = [0] * self.num_layers

    def _need_pool(self):
        if not self._pools:
            raise RuntimeError("KV cache not allocated: call allocate(num_gpu_blocks) first")

    # ---- paged API ---------------------------------------------------------------------------
    def append_slots(self, layer_id: int, key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor) -> None:
        """key / value: (num_tokens, kv_heads, head_dim); slot_mapping: (num_tokens,) int64, slot =
        block * block_size + offset, negative = skip (vLLM padding)."""
        self._need_pool()
        T, H, D = key.shape
        slots = slot_mapping.to(self.device, torch.int64).contiguous()
        rm = N.RowMap(H, 0, 0, 0, None, 1, N.ptr(slots), self.block_size)
        self.kv.append(self._pools[layer_id], key, value, rm)

    def paged_decode_attention(self, layer_id: int, query: torch.Tensor, block_tables: torch.Tensor,
                               seq_lens: torch.Tensor, max_seq_len: Optional[int] = None,
                               scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """query (batch, q_heads, head_dim); block_tables (batch, max_blocks) int32; seq_lens (batch,) int32.
        `max_seq_len` is a host upper bound on seq_lens (defaults to the table capacity: no sync)."""
        self._need_pool()
        bt = block_tables.to(self.device, torch.int32).contiguous()
        sl = seq_lens.to(self.device, torch.int32).contiguous()
        max_len = int(max_seq_len) if max_seq_len is not None else bt.shape[1] * self.block_size
        return self.kv.decode_attention(self._pools[layer_id], query, self.num_heads, sl, max_len, block_tables=bt,
                                        block_size=self.block_size, scale=scale, out=out)

    # ---- upstream-style single-sequence API ------------------------------------------------------
    def append(self, layer_id: int, key: torch.Tensor, value: torch.Tensor) -> None:
        """key / value: (kv_heads, new, head_dim) (or with a leading batch dim, item 0 is used)."""
        self._need_pool()
        if key.dim() == 4:
            key, value = key[0], value[0]
        T = key.shape[1]
        pos = self._seq_len[layer_id]
        if pos + T > self._max_tokens:
            raise RuntimeError("paged KV cache is full")
        slots = torch.arange(pos, pos + T, dtype=torch.int64, device=self.device)
        self.append_slots(layer_id, key.transpose(0, 1), value.transpose(0, 1), slots)
        self._seq_len[layer_id] += T

    def _rows(self, layer_id: int, keys: bool = True, values: bool = True):
        """Upstream-layout rows of the single sequence, head-major: each (heads * seq, ...)."""
        seq, H, bs = self._seq_len[layer_id], self.num_heads, self.block_size
        tok = torch.arange(seq, device=self.device, dtype=torch.int64)
        # row (h, t) lives at slot ((t // bs) * H + h) * bs + t % bs
        slots = ((tok // bs)[None, :] * H + torch.arange(H, device=self.device)[:, None]) * bs + (tok % bs)[None, :]
        flat = slots.reshape(-1).contiguous()
        # a dense map over explicit slots: inner = 1 and block_size = 1 make slot -> slot
        rm = N.RowMap(1, 0, 0, 0, None, 1, N.ptr(flat), 1)
        out = self.kv.export_rows(self._pools[layer_id], H * seq, rm, keys, values)
        del flat
        return out

    def _dense(self, layer_id: int, which: str) -> torch.Tensor:
        seq, H, D = (self._seq_len[layer_id] if self._pools else 0), self.num_heads, self.head_dim
        if seq == 0:
            return torch.zeros(H, 0, D, dtype=torch.float32, device=self.device)
        kp, kn, vp, vn = self._rows(layer_id, keys=which == "key", values=which == "value")
        return self.kv.dequantize(kp if which == "key" else vp, kn if which == "key" else vn, which).view(H, seq, D)

    def get_keys(self, layer_id: int) -> torch.Tensor:
        return self._dense(layer_id, "key")

    def get_values(self, layer_id: int) -> torch.Tensor:
        return self._dense(layer_id, "value")

    def attention_scores(self, layer_id: int, query: torch.Tensor) -> torch.Tensor:
        """(heads, seq_q, head_dim) -> (heads, seq_q, seq_kv) logits scaled by 1/sqrt(head_dim)."""
        self._need_pool()
        from ..ops import attention_scores_packed

        q = query.to(self.device).float()
        H, sq, D = q.shape
        seq = self._seq_len[layer_id]
        kp, kn, _, _ = self._rows(layer_id, values=False)
        kp, kn = kp.view(H, seq, -1), kn.view(H, seq)
        out = torch.empty(H, sq, seq, dtype=torch.float32, device=self.device)
        for h in range(H):
            out[h] = attention_scores_packed(q[h].unsqueeze(0), kp[h], kn[h], self._kb[1], self._key_rotation,
                                             self.config.key_bits)[0]
        return out * (1.0 / math.sqrt(D))

    def attention_values(self, layer_id: int, attn_weights: torch.Tensor) -> torch.Tensor:
        self._need_pool()
        from ..ops import attention_values_packed

        w = attn_weights.to(self.device).float()
        H, sq, seq = w.shape
        _, _, vp, vn = self._rows(layer_id, keys=False)
        vp, vn = vp.view(H, seq, -1), vn.view(H, seq)
        out = torch.empty(H, sq, self.head_dim, dtype=torch.float32, device=self.device)
        for h in range(H):
            out[h] = attention_values_packed(w[h].unsqueeze(0), vp[h], vn[h], self._vb[1], self._val_rotation,
                                             self.config.value_bits)[0]
        return out

    def get_seq_length(self, layer_id: int) -> int:
        return self._seq_len[layer_id]

    def memory_bytes(self) -> int:
        per_token = self._pk + self._pv + 8
        return sum(self.num_heads * s * per_token for s in self._seq_len)

    @property
    def compression_ratio(self) -> float:
        used = self.memory_bytes()
        fp16 = sum(2 * self.num_heads * s * self.head_dim * 2 for s in self._seq_len)
        return fp16 / used if used else 0.0


class TurboQuantAttentionImpl(AttentionImpl):
    """Attention over a ``TurboQuantPagedKVCache``.

    ``forward`` takes the paged decode path when the metadata carries ``slot_mapping``,
    ``block_tables`` and ``seq_lens`` (one new token per sequence, grouped-query heads, ``self.scale``
    applied); otherwise it reproduces upstream's single-sequence sequence of calls (append, scores,
    softmax without mask, values; vllm_plugin/__init__.py:391-403).
    """

    def __init__(self, num_heads: int, head_dim: int, scale: float, num_kv_heads: int,
                 alibi_slopes: Optional[List[float]] = None, sliding_window: Optional[int] = None,
                 kv_cache_dtype: str = "turboquant", blocksparse_params: Optional[Dict[str, Any]] = None,
                 logits_soft_cap: Optional[float] = None, **kwargs: Any) -> None:
        self.num_heads, self.head_dim, self.scale, self.num_kv_heads = num_heads, head_dim, scale, num_kv_heads
        self.alibi_slopes, self.sliding_window, self.logits_soft_cap = alibi_slopes, sliding_window, logits_soft_cap

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, kv_cache: TurboQuantPagedKVCache,
                attn_metadata: Any, k_scale: float = 1.0, v_scale: float = 1.0, attn_type: Any = None,
                output: Optional[torch.Tensor] = None, **kwargs: Any) -> torch.Tensor:
        """query (num_tokens, num_heads, head_dim); key / value (num_tokens, num_kv_heads, head_dim)."""
        layer_id: int = getattr(attn_metadata, "layer_id", 0)
        slots = getattr(attn_metadata, "slot_mapping", None)
        tables = getattr(attn_metadata, "block_tables", None)
        lens = getattr(attn_metadata, "seq_lens", None)
        if slots is not None and tables is not None and lens is not None:
            kv_cache.append_slots(layer_id, key, value, slots)
            lens_t = lens if torch.is_tensor(lens) else torch.tensor(lens, dtype=torch.int32)
            res = kv_cache.paged_decode_attention(layer_id, query, tables, lens_t,
                                                  max_seq_len=getattr(attn_metadata, "max_seq_len", None),
                                                  scale=self.scale)
        else:
            kv_cache.append(layer_id, key.transpose(0, 1), value.transpose(0, 1))
            logits = kv_cache.attention_scores(layer_id, query.transpose(0, 1))
            res = kv_cache.attention_values(layer_id, torch.softmax(logits, dim=-1)).transpose(0, 1)
        res = res.to(query.dtype)
        if output is not None:
            output.copy_(res)
            return output
        return res


class TurboQuantAttentionBackend(AttentionBackend):
    """Backend descriptor vLLM queries for names, classes and cache shapes."""

    @staticmethod
    def get_name() -> str:
        return "turboquant"

    @staticmethod
    def get_impl_cls() -> Type[TurboQuantAttentionImpl]:
        return TurboQuantAttentionImpl

    @staticmethod
    def get_metadata_cls() -> Type[AttentionMetadata]:
        return AttentionMetadata

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int) -> Tuple[int, ...]:
        """Logical shape used by vLLM's bookkeeping (the packed pools are owned by the cache object)."""
        return (2, num_blocks, block_size, num_kv_heads, head_size)

    @staticmethod
    def get_supported_head_sizes() -> List[int]:
        return [64, 128]


_REGISTERED = False


def register() -> None:
    """Hook for vLLM's ``vllm.general_plugins`` entry point; idempotent, silent without vLLM."""
    global _REGISTERED
    if _REGISTERED:
        return
    try:
        from vllm.attention import selector as _selector  # type: ignore

        if hasattr(_selector, "register_backend"):
            _selector.register_backend("turboquant", TurboQuantAttentionBackend)
    except Exception:
        pass
    _REGISTERED = True


__all__ = ["TurboQuantKVCacheConfig", "TurboQuantPagedKVCache", "TurboQuantAttentionBackend",
           "TurboQuantAttentionImpl", "register"]
