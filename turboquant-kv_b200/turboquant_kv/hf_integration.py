"""HuggingFace Transformers integration -- ``TurboQuantCache``, B200 build.

Same constructor and ``DynamicCache`` surface as upstream ``turboquant_kv/hf_integration.py:267-555``
(``update``, ``get_seq_length``, ``get_max_length``, ``get_usable_length``, ``reorder_cache``,
``from_config``, ``seen_tokens``, ``memory_bytes``, ``__len__/__getitem__/__iter__``).

``update`` keeps upstream's contract -- it returns dense tensors: every OLD token dequantised, the NEW
tokens exact (hf_integration.py:383-390) -- but all sequences of a batch share one record store
(batch * heads units of 16-token records, see csrc/tiled_layout.cuh) that the fused kernels write and
read; the per-head, per-batch Python loops of upstream are gone.  ``decode_attention`` is the fast path that skips the dense
round trip altogether for one-token steps; ``TurboQuantCache.attach(model)`` routes a stock
``transformers`` model there through the attention-function registry (``attn_implementation="turboquant"``),
so that ``model(...)`` / ``generate`` never rebuild the dense history in a decode step -- the step upstream
pays O(context) dequantisation for at hf_integration.py:373-390.
"""
from __future__ import annotations

import math
import warnings
import weakref
from typing import Any, Dict, List, Optional, Tuple

import torch

from . import _native as N
from .config import TurboQuantConfig
from .kvstore import PackedKVStore

_TRANSFORMERS_AVAILABLE = False
_DynamicCache: type = object
try:
    from transformers import DynamicCache as _HFDynamicCache

    _DynamicCache = _HFDynamicCache  # type: ignore[misc]
    _TRANSFORMERS_AVAILABLE = True
except ImportError:  # pragma: no cover
    pass


class _LayerQuantStore:
    """Packed keys and values of one layer for a whole batch; capacity doubles as tokens arrive."""

    def __init__(self, tq_config: TurboQuantConfig, batch: int, num_heads: int, head_dim: int, device):
        self.tq_config, self.batch, self.num_heads, self.head_dim = tq_config, batch, num_heads, head_dim
        self.device = torch.device(device)
        self.seq_len = 0
        self.capacity = 0
        self.kv = PackedKVStore(head_dim, tq_config.key_bits, tq_config.value_bits, tq_config.seed,
                                tq_config.rotation, device)
        self._store: Optional[torch.Tensor] = None
        self._len_dev = torch.zeros(batch, dtype=torch.int32, device=device)

    def _reserve(self, need: int) -> None:
        if need <= self.capacity:
            return
        cap = max(256, self.capacity)
        while cap < need:
            cap *= 2
        new = self.kv.alloc(self.batch * self.num_heads, cap)
        if self._store is not None:
            new[:, : self._store.shape[1]] = self._store
        self._store, self.capacity = new, cap

    def append(self, key: torch.Tensor, value: torch.Tensor) -> None:
        """key / value: (batch, heads, new, head_dim)."""
        T = key.shape[2]
        self._reserve(self.seq_len + T)
        rm = N.RowMap(T, self.capacity, 1, self.seq_len, None, 1, None, 1)
        self.kv.append(self._store, key, value, rm)
        self.seq_len += T
        self._len_dev += T

    def _dense(self, which: str, dtype, upto: Optional[int] = None) -> torch.Tensor:
        B, H, D = self.batch, self.num_heads, self.head_dim
        S = self.seq_len if upto is None else upto
        if S == 0:
            return torch.zeros(B, H, 0, D, dtype=dtype, device=self.device)
        rm = N.RowMap(S, self.capacity, 1, 0, None, 1, None, 1)
        kp, kn, vp, vn = self.kv.export_rows(self._store, B * H * S, rm, keys=which == "key", values=which == "value")
        out = self.kv.dequantize(kp if which == "key" else vp, kn if which == "key" else vn, which, dtype)
        return out.view(B, H, S, D)

    def get_keys(self, dtype=torch.float32, upto: Optional[int] = None) -> torch.Tensor:
        return self._dense("key", dtype, upto)

    def get_values(self, dtype=torch.float32, upto: Optional[int] = None) -> torch.Tensor:
        return self._dense("value", dtype, upto)

    def export(self):
        """Upstream-layout rows of everything stored: k_packed (B, H, S, pk), k_norms (B, H, S), v_packed, v_norms."""
        B, H, S = self.batch, self.num_heads, self.seq_len
        rm = N.RowMap(max(S, 1), self.capacity, 1, 0, None, 1, None, 1)
        kp, kn, vp, vn = self.kv.export_rows(self._store, B * H * S, rm)
        return kp.view(B, H, S, -1), kn.view(B, H, S), vp.view(B, H, S, -1), vn.view(B, H, S)

    def decode_attention(self, query: torch.Tensor, scale: Optional[float]) -> torch.Tensor:
        return self.kv.decode_attention(self._store, query, self.num_heads, self._len_dev, self.seq_len,
                                        pitch=self.capacity, scale=scale, reserve_len=self.capacity)

    def packed_bytes(self) -> int:
        per_token = self.kv.pk + self.kv.pv + 8
        return self.batch * self.num_heads * self.seq_len * per_token


class _LayerProdStore:
    """Prod-mode keys and values of one layer for a whole batch (upstream hf_integration.py:82-143, 210-236):
    both are quantised with Algorithm 2 (MSE codes at bits - 1, one QJL residual sign per dimension, the
    residual norm, the norm) and kept as upstream-layout rows -- (batch, heads, capacity, ...) tensors that
    double as tokens arrive, instead of upstream's per-append chunk lists.  One ``tqb_quantize_prod`` /
    ``tqb_dequantize_prod`` launch serves all heads and sequences (they share rotation, codebook and S)."""

    FIELDS = ("packed", "signs", "res", "norms")

    def __init__(self, tq_config: TurboQuantConfig, batch: int, num_heads: int, head_dim: int, device):
        from .reference import _make_qjl_matrix, lloyd_max_codebook, make_rotation_matrix

        if min(tq_config.key_bits, tq_config.value_bits) < 2:
            raise ValueError("mode='prod' needs at least 2 bits (1 MSE bit + 1 sign bit)")
        self.tq_config, self.batch, self.num_heads, self.head_dim = tq_config, batch, num_heads, head_dim
        self.device = torch.device(device)
        self.seq_len = 0
        self.capacity = 0
        self._side = {}
        for name, bits, seed in (("key", tq_config.key_bits, tq_config.seed), ("value", tq_config.value_bits, tq_config.seed + 1)):
            self._side[name] = {
                "bits": bits,
                "rotation": make_rotation_matrix(head_dim, seed=seed, method=tq_config.rotation).to(self.device),
                "codebook": tuple(t.to(self.device) for t in lloyd_max_codebook(bits - 1, head_dim)),
                "S": _make_qjl_matrix(head_dim, head_dim, seed, self.device),
                "packed": None, "signs": None, "res": None, "norms": None,
            }

    def _reserve(self, need: int) -> None:
        if need <= self.capacity:
            return
        cap = max(256, self.capacity)
        while cap < need:
            cap *= 2
        B, H, D = self.batch, self.num_heads, self.head_dim
        for side in self._side.values():
            shapes = {"packed": ((side["bits"] - 1) * ((D + 7) // 8), torch.uint8), "signs": ((D + 7) // 8, torch.uint8),
                      "res": (None, torch.float32), "norms": (None, torch.float32)}
            for f, (last, dt) in shapes.items():
                new = torch.zeros((B, H, cap) + ((last,) if last else ()), dtype=dt, device=self.device)
                if side[f] is not None:
                    new[:, :, : self.seq_len] = side[f][:, :, : self.seq_len]
                side[f] = new
        self.capacity = cap

    def append(self, key: torch.Tensor, value: torch.Tensor) -> None:
        """key / value: (batch, heads, new, head_dim)."""
        from .reference import quantize_prod

        B, H, T, D = key.shape
        self._reserve(self.seq_len + T)
        lo, hi = self.seq_len, self.seq_len + T
        for name, x in (("key", key), ("value", value)):
            side = self._side[name]
            mp, sg, rn, nr = quantize_prod(x.reshape(B * H * T, D), side["bits"], dim=D, rotation=side["rotation"],
                                           codebook=side["codebook"], S_matrix=side["S"])
            side["packed"][:, :, lo:hi] = mp.view(B, H, T, -1)
            side["signs"][:, :, lo:hi] = sg.view(B, H, T, -1)
            side["res"][:, :, lo:hi] = rn.view(B, H, T)
            side["norms"][:, :, lo:hi] = nr.view(B, H, T)
        self.seq_len = hi

    def _dense(self, which: str, dtype) -> torch.Tensor:
        from .reference import dequantize_prod

        B, H, S, D = self.batch, self.num_heads, self.seq_len, self.head_dim
        if S == 0:
            return torch.zeros(B, H, 0, D, dtype=dtype, device=self.device)
        side = self._side[which]
        rows = [side[f][:, :, :S].reshape((B * H * S,) + tuple(side[f].shape[3:])) for f in self.FIELDS]
        out = dequantize_prod(rows[0], rows[1], rows[2], rows[3], side["bits"], D, rotation=side["rotation"],
                              codebook=side["codebook"], S_matrix=side["S"])
        return out.view(B, H, S, D).to(dtype)

    def get_keys(self, dtype=torch.float32) -> torch.Tensor:
        return self._dense("key", dtype)

    def get_values(self, dtype=torch.float32) -> torch.Tensor:
        return self._dense("value", dtype)

    def export(self, which: str = "key"):
        """Upstream-layout rows of one side: mse_packed (B, H, S, .), signs (B, H, S, .), residual norms, norms."""
        S = self.seq_len
        return tuple(self._side[which][f][:, :, :S] for f in self.FIELDS)

    def decode_attention(self, query: torch.Tensor, scale: Optional[float]) -> torch.Tensor:
        raise RuntimeError("TurboQuantCache(mode='prod') has no fused decode kernel in this build: use update(), "
                           "which returns the dequantised history as upstream does")

    def packed_bytes(self) -> int:
        D = self.head_dim
        per_token = sum((s["bits"] - 1) * ((D + 7) // 8) + (D + 7) // 8 + 8 for s in self._side.values())
        return self.batch * self.num_heads * self.seq_len * per_token


class TurboQuantCache(_DynamicCache):  # type: ignore[misc]
    """``DynamicCache`` whose layers hold TurboQuant codes instead of fp16 tensors."""

    def __init__(self, key_bits: int = 4, value_bits: int = 2, mode: str = "mse", rotation: str = "dense_qr",
                 protected_layers: int = 0, seed: int = 42, **kwargs: Any) -> None:
        if _TRANSFORMERS_AVAILABLE:
            super().__init__(**kwargs)
        self.tq_config = TurboQuantConfig(key_bits=key_bits, value_bits=value_bits, mode=mode, rotation=rotation,
                                          protected_layers=protected_layers, quantize_on_append=True, seed=seed)
        self._protected_layers = protected_layers
        self._layer_stores: Dict[int, _LayerQuantStore] = {}
        self._fp_key_cache: Dict[int, List[torch.Tensor]] = {}
        self._fp_value_cache: Dict[int, List[torch.Tensor]] = {}
        self.fused_attention = False     # set by attach(): one-token updates return the new token only

    def _store(self, layer_idx: int, like: torch.Tensor) -> _LayerQuantStore:
        st = self._layer_stores.get(layer_idx)
        if st is None:
            if not like.is_cuda:
                raise RuntimeError("TurboQuantCache (B200 build) needs CUDA key/value states; there is no CPU path")
            B, H, _, D = like.shape
            cls = _LayerProdStore if self.tq_config.mode == "prod" else _LayerQuantStore
            st = cls(self.tq_config, B, H, D, like.device)
            self._layer_stores[layer_idx] = st
        return st

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[Dict[str, Any]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Quantise and store the new tokens; return (all_keys, all_values), each
        (batch, kv_heads, total, head_dim): old tokens dequantised, new tokens exact."""
        if layer_idx < self._protected_layers:
            self._fp_key_cache.setdefault(layer_idx, []).append(key_states)
            self._fp_value_cache.setdefault(layer_idx, []).append(value_states)
            return torch.cat(self._fp_key_cache[layer_idx], dim=2), torch.cat(self._fp_value_cache[layer_idx], dim=2)
        st = self._store(layer_idx, key_states)
        if self.fused_attention and key_states.shape[2] == 1 and isinstance(st, _LayerQuantStore):
            # the attention function registered by attach() reads the packed records itself
            st.append(key_states, value_states)
            return key_states, value_states
        dt = key_states.dtype if key_states.dtype in (torch.float16, torch.bfloat16) else torch.float32
        k_old, v_old = st.get_keys(dt), st.get_values(dt)
        st.append(key_states, value_states)
        return (torch.cat([k_old.to(key_states.dtype), key_states], dim=2),
                torch.cat([v_old.to(value_states.dtype), value_states], dim=2))

    def append_only(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int) -> None:
        """Store new tokens without building the dense history (pair with ``decode_attention``)."""
        self._store(layer_idx, key_states).append(key_states, value_states)

    def decode_attention(self, query: torch.Tensor, layer_idx: int, scale: Optional[float] = None) -> torch.Tensor:
        """Fused attention of one new query token per sequence over the packed layer.

        query: (batch, q_heads, head_dim) or (batch, q_heads, 1, head_dim)."""
        st = self._layer_stores[layer_idx]
        squeeze = query.dim() == 4
        out = st.decode_attention(query[:, :, 0] if squeeze else query, scale)
        return out.unsqueeze(2) if squeeze else out

    def attach(self, model) -> "TurboQuantCache":
        """Route `model`'s attention through the packed cache: registers the ``"turboquant"`` attention
        function with ``transformers``, selects it on the model and ties this cache to every attention module
        (the registry's functions receive the module, not the cache).  Afterwards a one-token ``update`` stores
        the token and returns it alone, and the attention function runs the fused kernel over the packed
        records; longer updates, protected and Prod-mode layers and padded batches keep the dense contract of
        ``update``.  The new token is attended in its quantised form (as ``QuantizedKVCache.decode_attention``
        does, cache.py:200-263), where the dense contract keeps it exact."""
        register_turboquant_attention()
        for mod in model.modules():
            if hasattr(mod, "layer_idx") and hasattr(mod, "q_proj"):
                mod._turboquant_cache = weakref.ref(self)
        if hasattr(model, "set_attn_implementation"):
            model.set_attn_implementation(ATTENTION_NAME)
        else:  # pragma: no cover
            model.config._attn_implementation = ATTENTION_NAME
        self.fused_attention = True
        return self

    def get_mask_sizes(self, query_length, layer_idx: int = 0) -> Tuple[int, int]:
        """(kv_length, kv_offset) of the mask a layer call needs: everything stored plus the new tokens."""
        new = int(query_length.shape[0]) if isinstance(query_length, torch.Tensor) else int(query_length)
        return self.get_seq_length(layer_idx) + new, 0

    def get_seq_length(self, layer_idx: int = 0) -> int:
        if layer_idx < self._protected_layers:
            return sum(c.shape[2] for c in self._fp_key_cache.get(layer_idx, []))
        st = self._layer_stores.get(layer_idx)
        return 0 if st is None else st.seq_len

    def get_max_length(self) -> Optional[int]:
        return None

    def get_usable_length(self, new_seq_length: int, layer_idx: int = 0) -> int:
        return self.get_seq_length(layer_idx)

    def reorder_cache(self, beam_idx: torch.LongTensor) -> None:
        """Beam reordering: exact for protected layers; packed rows of quantised layers are gathered."""
        for li in list(self._fp_key_cache.keys()):
            self._fp_key_cache[li] = [c.index_select(0, beam_idx.to(c.device)) for c in self._fp_key_cache[li]]
            self._fp_value_cache[li] = [c.index_select(0, beam_idx.to(c.device)) for c in self._fp_value_cache[li]]
        if self._layer_stores:
            warnings.warn("TurboQuantCache.reorder_cache: beam search reordering is not fully supported for "
                          "quantised layers. Results may be incorrect. Use greedy or sampling decoding instead.",
                          stacklevel=2)

    @classmethod
    def from_config(cls, key_bits: int = 4, value_bits: int = 2, mode: str = "mse", rotation: str = "dense_qr",
                    protected_layers: int = 0, seed: int = 42) -> "TurboQuantCache":
        return cls(key_bits=key_bits, value_bits=value_bits, mode=mode, rotation=rotation,
                   protected_layers=protected_layers, seed=seed)

    @property
    def seen_tokens(self) -> int:
        lengths = [self.get_seq_length(i) for i in range(max(len(self._layer_stores), 1))]
        lengths.extend(self.get_seq_length(i) for i in self._fp_key_cache)
        return max(lengths) if lengths else 0

    def memory_bytes(self) -> int:
        """Bytes of packed codes and norms (protected fp16 layers not counted, as upstream)."""
        return sum(st.packed_bytes() for st in self._layer_stores.values())

    def __len__(self) -> int:
        return len(self._layer_stores) + len(self._fp_key_cache)

    def __getitem__(self, layer_idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if layer_idx < self._protected_layers and layer_idx in self._fp_key_cache:
            return torch.cat(self._fp_key_cache[layer_idx], dim=2), torch.cat(self._fp_value_cache[layer_idx], dim=2)
        st = self._layer_stores.get(layer_idx)
        if st is None:
            raise IndexError(f"No cached data for layer {layer_idx}")
        return st.get_keys(), st.get_values()

    def __iter__(self):
        for idx in sorted(set(self._layer_stores) | set(self._fp_key_cache)):
            yield self[idx]


ATTENTION_NAME = "turboquant"


def turboquant_attention_forward(module, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                                 attention_mask: Optional[torch.Tensor] = None, dropout: float = 0.0,
                                 scaling: Optional[float] = None, **kwargs):
    """Attention function for ``transformers``' registry (same signature and return as its
    ``sdpa_attention_forward``: output (batch, q_len, q_heads, head_dim), no weights).

    query (batch, q_heads, q_len, head_dim).  For a one-token step on a layer whose cache was attached with
    ``TurboQuantCache.attach`` the fused kernel attends over the packed records; `key` / `value` then hold the
    new token only.  With an attention mask (padded batches) the old tokens are dequantised here instead and the
    call, like every other one, goes to the library's SDPA function."""
    from transformers.integrations.sdpa_attention import sdpa_attention_forward

    ref = getattr(module, "_turboquant_cache", None)
    cache = ref() if ref is not None else None
    layer_idx = getattr(module, "layer_idx", None)
    st = cache._layer_stores.get(layer_idx) if cache is not None and cache.fused_attention else None
    if isinstance(st, _LayerQuantStore) and query.shape[2] == 1 and key.shape[2] != st.seq_len:
        # update() returned the new token alone
        if attention_mask is None and dropout == 0.0:
            out = st.decode_attention(query[:, :, 0], scaling)
            return out.unsqueeze(1).to(query.dtype), None
        dt = key.dtype if key.dtype in (torch.float16, torch.bfloat16) else torch.float32
        key = torch.cat([st.get_keys(dt, st.seq_len - 1).to(key.dtype), key], dim=2)
        value = torch.cat([st.get_values(dt, st.seq_len - 1).to(value.dtype), value], dim=2)
    return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling, **kwargs)


def register_turboquant_attention() -> str:
    """Register ``turboquant_attention_forward`` (and SDPA-style masks for it) with ``transformers``; returns the
    name to pass as ``attn_implementation``."""
    if not _TRANSFORMERS_AVAILABLE:
        raise ImportError("transformers is required for register_turboquant_attention")
    from transformers import AttentionInterface
    from transformers.masking_utils import AttentionMaskInterface, sdpa_mask

    AttentionInterface.register(ATTENTION_NAME, turboquant_attention_forward)
    AttentionMaskInterface.register(ATTENTION_NAME, sdpa_mask)
    return ATTENTION_NAME


__all__ = ["TurboQuantCache", "turboquant_attention_forward", "register_turboquant_attention", "ATTENTION_NAME"]
