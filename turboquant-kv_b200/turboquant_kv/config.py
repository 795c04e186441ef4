"""Configuration dataclass (same fields, order and defaults as upstream turboquant_kv/config.py:6-30)."""
from dataclasses import dataclass


@dataclass
class TurboQuantConfig:
    """Settings of a TurboQuant KV cache.

    key_bits / value_bits   bits per coordinate for keys / values
    mode                    "mse" (Algorithm 1) or "prod" (Algorithm 2, one bit spent on QJL signs)
    rotation                "dense_qr" or "rht"
    outlier_channels, quantize_on_append, block_size
                            accepted for compatibility; like upstream, no compute path reads them
    protected_layers        the first N layers stay in fp16
    seed                    rotation seed (values use seed + 1)
    """

    key_bits: int = 4
    value_bits: int = 2
    mode: str = "mse"
    rotation: str = "dense_qr"
    outlier_channels: int = 0
    protected_layers: int = 0
    quantize_on_append: bool = True
    block_size: int = 0
    seed: int = 42
