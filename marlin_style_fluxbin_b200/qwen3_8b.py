"""Architecture constants of Qwen3-8B that the packed model loaders check against.

Mirrors the constants of the reference's ``qwen3_8b`` module (``src/fluxbin_style/qwen3_8b.py:20-37``);
its checkpoint-snapshot preflight is not part of the decode path and is not mirrored.
"""
from __future__ import annotations

from typing import Any

ARCHITECTURE = {
    "model_type": "qwen3", "num_hidden_layers": 36, "hidden_size": 4096, "intermediate_size": 12288,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
}


def validate_architecture(config: dict[str, Any]) -> None:
    for key, expected in ARCHITECTURE.items():
        if config.get(key) != expected:
            raise ValueError(f"8B architecture drift: {key}")
