"""Qwen3 decoder-block Linear inventory (names and expected shapes).

Mirrors the constants and helpers of the reference's ``qwen3`` module that the packed
Linear adapters use (reference file ``src/fluxbin_style/qwen3.py:16-69``).
"""
from __future__ import annotations

import re
from typing import Any

QWEN3_LINEAR_MODULES = (
    "self_attn.q_proj",
    "self_attn.k_proj",
    "self_attn.v_proj",
    "self_attn.o_proj",
    "mlp.gate_proj",
    "mlp.up_proj",
    "mlp.down_proj",
)

_NAME = re.compile(r"^model\.layers\.(\d+)\.(" + "|".join(re.escape(m) for m in QWEN3_LINEAR_MODULES) + r")\.weight$")


def qwen3_linear_weight_names(num_layers: int) -> tuple[str, ...]:
    if not isinstance(num_layers, int) or num_layers <= 0:
        raise ValueError("num_layers must be a positive integer")
    return tuple(f"model.layers.{i}.{m}.weight" for i in range(num_layers) for m in QWEN3_LINEAR_MODULES)


def parse_qwen3_linear_name(name: str) -> tuple[int, str]:
    found = _NAME.fullmatch(name)
    if found is None:
        raise ValueError(f"not a Qwen3 transformer-block Linear: {name}")
    return int(found.group(1)), found.group(2)


def expected_qwen3_linear_shape(config: dict[str, Any], module: str) -> list[int]:
    """``[out_features, in_features]`` of one of the seven Linears for a model config."""
    dims = {}
    for key in ("hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads", "head_dim"):
        value = config.get(key)
        if not isinstance(value, int) or value <= 0:
            raise ValueError(f"Qwen3 config requires positive integer {key}")
        dims[key] = value
    hidden, inter = dims["hidden_size"], dims["intermediate_size"]
    q_width = dims["num_attention_heads"] * dims["head_dim"]
    kv_width = dims["num_key_value_heads"] * dims["head_dim"]
    table = {
        "self_attn.q_proj": [q_width, hidden],
        "self_attn.k_proj": [kv_width, hidden],
        "self_attn.v_proj": [kv_width, hidden],
        "self_attn.o_proj": [hidden, q_width],
        "mlp.gate_proj": [inter, hidden],
        "mlp.up_proj": [inter, hidden],
        "mlp.down_proj": [hidden, inter],
    }
    if module not in table:
        raise ValueError(f"unsupported Qwen3 module: {module}")
    return table[module]
