"""Multi-GPU semantics on one node: one process per GPU, ``torch.distributed`` for the plumbing.

``DistributedQuantizedKVCache`` mirrors upstream ``turboquant_kv/distributed.py:32-216``: KV heads are
split evenly over ``tp_size`` ranks, each rank owns a ``QuantizedKVCache`` for its heads, and because
attention heads are independent no collective is needed on the attention path.

``ShardedTurboQuantIndex`` is the row-sharded search: rank r holds a contiguous slice of the database
(global id = local row + ``id_offset``); a search runs the local scan on every rank, all-gathers the
(Q, k) scores and ids (12 bytes per candidate) and merges them with the scan's ordering rule (score
descending, id ascending), so every rank returns the same global top-k.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .cache import QuantizedKVCache
from .config import TurboQuantConfig
from .search import TurboQuantIndex, merge_topk


class DistributedQuantizedKVCache:
    """Tensor-parallel packed KV cache: this rank stores ``num_heads // tp_size`` heads."""

    def __init__(self, config: TurboQuantConfig, num_layers: int, max_seq_len: int, num_heads: int,
                 head_dim: int, tp_size: int = 1, tp_rank: int = 0, device: str = "cuda",
                 batch_size: Optional[int] = None):
        if num_heads % tp_size != 0:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by tp_size ({tp_size})")
        if not (0 <= tp_rank < tp_size):
            raise ValueError(f"tp_rank ({tp_rank}) must be in [0, {tp_size})")
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self.num_heads = num_heads
        self.local_num_heads = num_heads // tp_size
        self.head_dim, self.num_layers, self.max_seq_len, self.device = head_dim, num_layers, max_seq_len, device
        self.cache = QuantizedKVCache(config, num_layers, max_seq_len, self.local_num_heads, head_dim, device,
                                      batch_size=batch_size)

    @classmethod
    def from_config(cls, config: TurboQuantConfig, tp_size: int, tp_rank: int, num_layers: int,
                    max_seq_len: int, num_heads: int, head_dim: int, device: Optional[str] = None,
                    batch_size: Optional[int] = None) -> "DistributedQuantizedKVCache":
        """``device`` defaults to ``cuda:{tp_rank}`` (one process per GPU of a node)."""
        return cls(config, num_layers, max_seq_len, num_heads, head_dim, tp_size=tp_size, tp_rank=tp_rank,
                   device=device if device is not None else f"cuda:{tp_rank}", batch_size=batch_size)

    def head_slice(self) -> slice:
        """The global KV-head range owned by this rank."""
        return slice(self.tp_rank * self.local_num_heads, (self.tp_rank + 1) * self.local_num_heads)

    # the caller passes tensors already sliced to the local heads, as in a tensor-parallel attention layer
    def append(self, layer_id: int, key: torch.Tensor, value: torch.Tensor):
        self.cache.append(layer_id, key, value)

    def attention_scores(self, layer_id: int, query: torch.Tensor) -> torch.Tensor:
        return self.cache.attention_scores(layer_id, query)

    def attention_values(self, layer_id: int, attn_weights: torch.Tensor) -> torch.Tensor:
        return self.cache.attention_values(layer_id, attn_weights)

    def decode_attention(self, layer_id: int, query: torch.Tensor, scale: Optional[float] = None,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.cache.decode_attention(layer_id, query, scale=scale, out=out)

    def decode_step(self, layer_id: int, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                    scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Append the local heads' new token and attend, in one launch (QuantizedKVCache.decode_step)."""
        return self.cache.decode_step(layer_id, query, key, value, scale=scale, out=out)

    def decode_status(self) -> int:
        return self.cache.decode_status()

    @property
    def seq_lens(self) -> torch.Tensor:
        return self.cache.seq_lens

    def memory_bytes(self) -> int:
        return self.cache.memory_bytes()

    @property
    def compression_ratio(self) -> float:
        return self.cache.compression_ratio

    def __repr__(self) -> str:
        return (f"DistributedQuantizedKVCache(tp_rank={self.tp_rank}/{self.tp_size}, "
                f"local_heads={self.local_num_heads}, layers={self.num_layers}, "
                f"max_seq={self.max_seq_len}, device={self.device})")


def shard_rows(n_rows: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous row range [begin, end) of `rank`: the first n % world ranks get one extra row."""
    base, extra = divmod(n_rows, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def gather_and_merge(local_scores: torch.Tensor, local_ids: torch.Tensor, k: int, group=None):
    """All-gather every rank's (Q, k) candidates and merge to the global top-k (same result on all ranks).

    Works on whatever device the tensors live on (NCCL for CUDA tensors, gloo for host tensors).
    """
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local_scores, local_ids
    world = dist.get_world_size(group)
    q = local_scores.shape[0]
    s_all = torch.empty(world * q, k, dtype=torch.float32, device=local_scores.device)
    i_all = torch.empty(world * q, k, dtype=torch.int64, device=local_ids.device)
    dist.all_gather_into_tensor(s_all, local_scores.contiguous().float(), group=group)   # rank-major rows
    dist.all_gather_into_tensor(i_all, local_ids.contiguous().to(torch.int64), group=group)
    s_all, i_all = s_all.view(world, q, k), i_all.view(world, q, k)
    return merge_topk(s_all.permute(1, 0, 2).contiguous(), i_all.permute(1, 0, 2).contiguous(), k)


class ShardedTurboQuantIndex:
    """Row-sharded ``TurboQuantIndex``: every rank adds ITS rows, every rank gets the global answer."""

    def __init__(self, dim: int, bit_width: int = 3, mode: str = "mse", rotation: str = "dense_qr",
                 seed: int = 42, id_offset: int = 0, group=None, device=None):
        self.local = TurboQuantIndex(dim, bit_width=bit_width, mode=mode, rotation=rotation, seed=seed, device=device)
        self.local.id_offset = id_offset
        self.group = group

    def add(self, local_vectors: torch.Tensor):
        self.local.add(local_vectors)

    @property
    def n_vectors(self) -> int:
        return self.local.n_vectors

    def search(self, queries: torch.Tensor, k: int = 10):
        """`queries` must be the same on every rank.  Shards shorter than k pad with (-inf, -1)."""
        if queries.dim() == 1:
            queries = queries.unsqueeze(0)
        q = queries.to(self.local.device, torch.float32)
        kk = min(k, max(self.local.n_vectors, 1))
        if self.local.n_vectors > 0:
            s, i = self.local.search(q, kk)
        else:
            s = q.new_full((q.shape[0], 0), float("-inf"))
            i = torch.empty(q.shape[0], 0, dtype=torch.int64, device=q.device)
        if s.shape[1] < k:
            pad = k - s.shape[1]
            s = torch.cat([s, s.new_full((s.shape[0], pad), float("-inf"))], 1)
            i = torch.cat([i, i.new_full((i.shape[0], pad), -1)], 1)
        s, i = gather_and_merge(s, i, k, self.group)
        return s.to(queries.device), i.to(queries.device)
