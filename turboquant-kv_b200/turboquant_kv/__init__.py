"""turboquant_kv -- TurboQuant KV-cache compression and vector search (arXiv:2504.19874), B200 build.

Drop-in for the upstream ``turboquant_kv`` package on its hot path: the same names are exported,
the tensor work runs in hand-written sm_100a CUDA kernels behind ``libtqb200.so`` (C ABI in
``include/tqb200.h``).  There is no Triton, no backend dispatch and no CPU fallback.
"""
from .config import TurboQuantConfig
from .cache import QuantizedKVCache
from .search import TurboQuantIndex
from .distributed import DistributedQuantizedKVCache, ShardedTurboQuantIndex
from .reference import quantize_mse, dequantize_mse, quantize_prod, dequantize_prod

try:  # needs transformers
    from .hf_integration import TurboQuantCache
except ImportError:  # pragma: no cover
    TurboQuantCache = None  # type: ignore[assignment,misc]

from .vllm_plugin import TurboQuantKVCacheConfig, TurboQuantPagedKVCache, TurboQuantAttentionBackend

__version__ = "0.1.0"

__all__ = [
    "TurboQuantConfig", "QuantizedKVCache", "TurboQuantIndex", "DistributedQuantizedKVCache",
    "ShardedTurboQuantIndex", "quantize_mse", "dequantize_mse", "quantize_prod", "dequantize_prod",
    "TurboQuantCache", "TurboQuantKVCacheConfig", "TurboQuantPagedKVCache", "TurboQuantAttentionBackend",
]
