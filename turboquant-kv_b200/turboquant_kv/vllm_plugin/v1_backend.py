"""Attention backend for vLLM's v1 engine interface (``vllm.v1.attention.backend``).

Upstream's plugin targets ``vllm.attention.backends.abstract``, an import path that newer vLLM
releases no longer have, so its classes fall back to stand-in bases
(upstream ``turboquant_kv/vllm_plugin/__init__.py:33-64, 420-458``).  This module implements the
interface the installed engine really has:

  ``TurboQuantV1Backend``           ``AttentionBackend``: name, KV-cache shape, impl / builder classes
  ``TurboQuantV1Metadata``          per-step metadata (block table, lengths, slot mapping)
  ``TurboQuantV1MetadataBuilder``   ``AttentionMetadataBuilder.build`` from ``CommonAttentionMetadata``
  ``TurboQuantV1Impl``              ``AttentionImpl.forward``: scatter the step's new K/V into the paged
                                    record pool (one launch), then attend

The KV cache of a layer is one uint8 tensor ``(num_blocks, kv_heads, block_size / 16 * record_bytes)``:
the 16-token records of ``kvstore.PackedKVStore`` (keys ``KEY_BITS``, values ``VALUE_BITS``), page-major,
so vLLM's block ids and slot mapping address it directly.  Requests with one new token (decode) run the
fused paged decode kernel.  Batches with several new tokens per request (prefill, chunked prefill,
speculative verification) run the same kernel with every query token as a sequence of its own (its
request's block-table row, its causal prefix as the length): nothing is dequantised, but every token
streams its prefix again -- right for short chunks, quadratic for long prompts.  Very large calls are split
into several launches of that kernel; there is no library attention path.

vLLM is imported when this module is imported; nothing else in the package depends on it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import ClassVar, List, Optional

import torch
from vllm.v1.attention.backend import (AttentionBackend, AttentionCGSupport, AttentionImpl, AttentionMetadataBuilder,
                                       AttentionType, CommonAttentionMetadata, MultipleOf)

from .. import _native as N
from ..kvstore import PackedKVStore


class TurboQuantV1Backend(AttentionBackend):
    """TurboQuant packed-KV attention for the v1 engine (MSE mode)."""

    KEY_BITS: ClassVar[int] = 4
    VALUE_BITS: ClassVar[int] = 2
    SEED: ClassVar[int] = 42
    ROTATION: ClassVar[str] = "dense_qr"
    supported_dtypes: ClassVar[List[torch.dtype]] = [torch.float16, torch.bfloat16, torch.float32]
    supported_kv_cache_dtypes: ClassVar[list] = ["auto", "uint8"]
    forward_includes_kv_cache_update: bool = True

    @classmethod
    def configure(cls, key_bits: int = 4, value_bits: int = 2, seed: int = 42, rotation: str = "dense_qr") -> None:
        """Bit widths / seed of every cache created afterwards (class-wide, like vLLM's backend selection)."""
        cls.KEY_BITS, cls.VALUE_BITS, cls.SEED, cls.ROTATION = key_bits, value_bits, seed, rotation

    @staticmethod
    def get_supported_kernel_block_sizes():
        return [MultipleOf(16)]

    @classmethod
    def get_supported_head_sizes(cls) -> List[int]:
        return [64, 128]

    @staticmethod
    def get_name() -> str:
        return "TURBOQUANT"

    @staticmethod
    def get_impl_cls():
        return TurboQuantV1Impl

    @staticmethod
    def get_builder_cls():
        return TurboQuantV1MetadataBuilder

    @staticmethod
    def record_bytes(head_size: int) -> int:
        rb = int(N.lib().tqb_kv_record_bytes(head_size, TurboQuantV1Backend.KEY_BITS, TurboQuantV1Backend.VALUE_BITS))
        if rb == 0:
            raise ValueError(f"unsupported head_size {head_size} / bits "
                             f"{TurboQuantV1Backend.KEY_BITS}/{TurboQuantV1Backend.VALUE_BITS}")
        return rb

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto"):
        if block_size % 16:
            raise ValueError("TurboQuant pages hold whole 16-token records: block_size must be a multiple of 16")
        return (num_blocks, num_kv_heads, block_size // 16 * TurboQuantV1Backend.record_bytes(head_size))

    @staticmethod
    def kv_cache_dtype() -> torch.dtype:
        return torch.uint8


@dataclass
class TurboQuantV1Metadata:
    num_reqs: int
    num_actual_tokens: int
    max_query_len: int
    max_seq_len: int
    query_start_loc: torch.Tensor          # (num_reqs + 1,) int32, device
    query_start_loc_cpu: torch.Tensor      # the same on the host (prefill path only)
    seq_lens: torch.Tensor                 # (num_reqs,) int32, device: tokens of each request incl. the new ones
    block_table: torch.Tensor              # (num_reqs, max_blocks) int32, device
    slot_mapping: torch.Tensor             # (num_tokens,) int64, device; negative = padding
    causal: bool = True


class TurboQuantV1MetadataBuilder(AttentionMetadataBuilder[TurboQuantV1Metadata]):
    # single-token decode batches contain no host-dependent work: safe to capture in a CUDA graph
    _cudagraph_support: ClassVar[AttentionCGSupport] = AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)

    def build(self, common_prefix_len: int, common_attn_metadata: CommonAttentionMetadata,
              fast_build: bool = False) -> TurboQuantV1Metadata:
        m = common_attn_metadata
        return TurboQuantV1Metadata(
            num_reqs=m.num_reqs, num_actual_tokens=m.num_actual_tokens, max_query_len=m.max_query_len,
            max_seq_len=m.max_seq_len, query_start_loc=m.query_start_loc, query_start_loc_cpu=m.query_start_loc_cpu,
            seq_lens=m.seq_lens, block_table=m.block_table_tensor, slot_mapping=m.slot_mapping, causal=m.causal)


class TurboQuantV1Impl(AttentionImpl[TurboQuantV1Metadata]):
    """``forward`` = quantise-and-scatter the new K/V of the step, then attention over the packed pool."""

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: Optional[int] = None,
                 alibi_slopes=None, sliding_window=None, kv_cache_dtype: str = "auto", logits_soft_cap=None,
                 attn_type: str = AttentionType.DECODER, kv_sharing_target_layer_name: Optional[str] = None) -> None:
        if alibi_slopes is not None or sliding_window is not None or logits_soft_cap:
            raise NotImplementedError("TurboQuant attention: ALiBi, sliding windows and logit soft caps are not supported")
        if attn_type != AttentionType.DECODER:
            raise NotImplementedError("TurboQuant attention covers decoder self-attention only")
        if kv_sharing_target_layer_name is not None:
            raise NotImplementedError("TurboQuant attention: KV sharing between layers is not supported")
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_kv_heads if num_kv_heads is not None else num_heads
        if self.num_heads % self.num_kv_heads or self.num_heads // self.num_kv_heads > 8:
            raise NotImplementedError("TurboQuant attention: 1 to 8 query heads per KV head")
        self.kv_cache_dtype = kv_cache_dtype
        self._kv: Optional[PackedKVStore] = None

    # largest (tokens x blocks per request) table the multi-token path materialises per launch (int32 entries)
    MAX_EXPANDED_TABLE = 1 << 26

    def _store(self, device) -> PackedKVStore:
        if self._kv is None:
            B = TurboQuantV1Backend
            self._kv = PackedKVStore(self.head_size, B.KEY_BITS, B.VALUE_BITS, B.SEED, B.ROTATION, device)
        return self._kv

    def forward(self, layer, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                attn_metadata: Optional[TurboQuantV1Metadata], output: Optional[torch.Tensor] = None,
                output_scale=None, output_block_scale=None) -> torch.Tensor:
        """query (tokens, heads * head_size) or (tokens, heads, head_size); key / value likewise with KV heads;
        kv_cache: the layer's uint8 pool (``TurboQuantV1Backend.get_kv_cache_shape``).  Returns ``output``."""
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("TurboQuant attention: fused output quantisation is not supported")
        if output is None:
            output = torch.empty_like(query)
        if attn_metadata is None:                      # memory-profiling run of the engine: nothing to attend to
            return output.zero_()
        md = attn_metadata
        n, H, HK, D = md.num_actual_tokens, self.num_heads, self.num_kv_heads, self.head_size
        kv = self._store(query.device)
        rec = kv.record_bytes
        nblocks, heads, page_bytes = kv_cache.shape
        if kv_cache.dtype != torch.uint8 or heads != HK or page_bytes % rec:
            raise RuntimeError(f"kv_cache {tuple(kv_cache.shape)} {kv_cache.dtype} is not a TurboQuant pool for "
                               f"{HK} KV heads (record {rec} bytes)")
        block_size = page_bytes // rec * 16
        pool = kv_cache.view(nblocks * HK, page_bytes // rec, rec)
        q = query[:n].reshape(n, H, D)
        out = output[:n].view(n, H, D)

        # 1. the step's new tokens -> their slots (one launch; negative slots are padding)
        slots = md.slot_mapping[:n].to(torch.int64).contiguous()
        rm = N.RowMap(HK, 0, 0, 0, None, 1, N.ptr(slots), block_size)
        kv.append(pool, key[:n].reshape(n, HK, D), value[:n].reshape(n, HK, D), rm)

        # 2a. pure decode batch: one fused launch sequence over block tables
        bt = md.block_table.to(torch.int32).contiguous()
        lens = md.seq_lens.to(torch.int32).contiguous()
        if md.max_query_len == 1 and n == md.num_reqs:
            if q.dtype == out.dtype and out.is_contiguous():
                # (the workspace is sized for the block table's capacity once: a captured graph keeps its address)
                kv.decode_attention(pool, q, HK, lens, md.max_seq_len, block_tables=bt, block_size=block_size,
                                    scale=self.scale, out=out, reserve_len=bt.shape[1] * block_size)
            else:
                out.copy_(kv.decode_attention(pool, q, HK, lens, md.max_seq_len, block_tables=bt,
                                              block_size=block_size, scale=self.scale,
                                              reserve_len=bt.shape[1] * block_size))
            return output

        # 2b. requests with several new tokens (prefill chunks, speculative verification): every query token is
        # handed to the fused kernel as a sequence of its own -- the request's block-table row and its causal
        # prefix as the length -- so nothing is dequantised and no library attention runs.  The per-token copy of
        # the block table is built for at most MAX_EXPANDED_TABLE entries at a time: larger calls take several
        # launches.  (Each token streams its prefix again; a kernel that shares the stream between the tokens
        # of a request is not part of this build.)
        qsl = md.query_start_loc.to(torch.int64)
        qlens = qsl[1:md.num_reqs + 1] - qsl[:md.num_reqs]
        req = torch.repeat_interleave(torch.arange(md.num_reqs, device=q.device), qlens, output_size=n)
        if md.causal:
            pos = torch.arange(n, device=q.device) - qsl[req]
            tok_lens = (lens.to(torch.int64)[req] - qlens[req] + pos + 1).to(torch.int32)
        else:
            tok_lens = lens[req].to(torch.int32)
        step = max(1, self.MAX_EXPANDED_TABLE // max(1, bt.shape[1]))
        for c0 in range(0, n, step):
            c1 = min(n, c0 + step)
            res = kv.decode_attention(pool, q[c0:c1].contiguous(), HK, tok_lens[c0:c1].contiguous(), md.max_seq_len,
                                      block_tables=bt[req[c0:c1]].contiguous(), block_size=block_size,
                                      scale=self.scale)
            out[c0:c1].copy_(res)
        return output


__all__ = ["TurboQuantV1Backend", "TurboQuantV1Metadata", "TurboQuantV1MetadataBuilder", "TurboQuantV1Impl"]
