"""Hash-bound loading of offline W3 deployment artifacts and whole-model replacement.

Mirror of the reference's ``w3_lut_artifacts`` (``src/fluxbin_style/w3_lut_artifacts.py:14-118``):
a ``manifest.json`` pins every per-layer safetensors file by size and sha256; nothing is mutated
until every layer has been validated.
"""
from __future__ import annotations

import json
from pathlib import Path

from .evaluation import sha256_file
from .gptq_deployment import FIELDS, FORMAT, validate_planar_w3
from .qwen3 import QWEN3_LINEAR_MODULES


def load_w3_lut_layer(root: Path, layer: int, *, expected_manifest_sha256: str) -> tuple[dict, dict]:
    """Tensors of one decoder layer (seven Linears x three fields) and its manifest entry."""
    from safetensors.torch import load_file

    root = Path(root)
    manifest_path = root / "manifest.json"
    if sha256_file(manifest_path) != expected_manifest_sha256:
        raise ValueError("W3 LUT manifest drift")
    manifest = json.loads(manifest_path.read_text(encoding="utf-8"))
    if manifest.get("status") != "completed_pending_gpu_validation" or manifest.get("format") != FORMAT:
        raise ValueError("W3 LUT manifest status/format drift")
    gate = manifest.get("canonical_semantics_gate", {})
    if (gate.get("status") != "confirmed_before_payload_writes" or gate.get("inspected_linears") != 252
            or gate.get("all_groups_have_128_columns") is not True or gate.get("decoded_zero_unique") != [4]):
        raise ValueError("W3 LUT canonical-semantics gate missing or drifted")
    if not 0 <= layer < 36:
        raise ValueError("layer outside 0..35")
    relative = f"payloads/layer-{layer:03d}.safetensors"
    entry = next((item for item in manifest["files"] if item["path"] == relative), None)
    if entry is None:
        raise ValueError("W3 LUT layer missing from the manifest")
    path = root / relative
    if path.stat().st_size != entry["bytes"] or sha256_file(path) != entry["sha256"]:
        raise ValueError("W3 LUT layer hash/size drift")
    tensors = load_file(path)
    if set(tensors) != {f"{module}.{field}" for module in QWEN3_LINEAR_MODULES for field in FIELDS}:
        raise ValueError("W3 LUT layer inventory drift")
    for module in QWEN3_LINEAR_MODULES:
        validate_planar_w3({field: tensors[f"{module}.{field}"] for field in FIELDS})
    return tensors, entry


def replace_w3_model_linears(model, artifact_root: Path, *, expected_manifest_sha256: str,
                             allow_prefill_fallback: bool = False, route: str = "structural") -> dict:
    """Install all 252 hash-bound W3 Linears of a Qwen3-8B model; attention and cache code stay untouched."""
    from torch import nn

    from .qwen3 import expected_qwen3_linear_shape
    from .qwen3_8b import ARCHITECTURE, validate_architecture
    from .w3_lut_deployment import QWEN3_ROW_TILE_BY_SHAPE, QWEN3_W3_ROUTE_POLICIES, replace_w3_block_linears

    validate_architecture(model.config.to_dict())
    if len(model.model.layers) != 36:
        raise ValueError("expected 36 decoder layers")
    if route not in QWEN3_W3_ROUTE_POLICIES:
        raise ValueError(f"unknown Qwen3-8B W3 route: {route}")
    records = []
    for index in range(36):  # first pass: validate everything, change nothing
        payload, entry = load_w3_lut_layer(artifact_root, index, expected_manifest_sha256=expected_manifest_sha256)
        for name in QWEN3_LINEAR_MODULES:
            shape = validate_planar_w3({field: payload[f"{name}.{field}"] for field in FIELDS})
            if list(shape) != expected_qwen3_linear_shape(ARCHITECTURE, name):
                raise ValueError(f"8B W3 shape drift: layer {index} {name}")
            target = model.model.layers[index].get_submodule(name)
            if not isinstance(target, nn.Linear) or (target.out_features, target.in_features) != shape:
                raise ValueError(f"Linear shape/type mismatch: layer {index} {name}")
        records.append(entry)
    coverage = []
    for index, block in enumerate(model.model.layers):
        payload, _ = load_w3_lut_layer(artifact_root, index, expected_manifest_sha256=expected_manifest_sha256)
        names = replace_w3_block_linears(block, payload, fallback="dense" if allow_prefill_fallback else "error", route=route)
        coverage.extend(f"model.layers.{index}.{name}" for name in names)
    return {
        "format": FORMAT, "manifest_sha256": expected_manifest_sha256, "layers": records, "coverage": coverage,
        "linear_count": len(coverage),
        "row_tile_by_shape": {f"{o}x{k}": tile for (o, k), tile in QWEN3_ROW_TILE_BY_SHAPE.items()},
        "prefill_fallback_enabled": allow_prefill_fallback, "route": route,
        "route_policy": {f"{o}x{k}": dict(policy) for (o, k), policy in QWEN3_W3_ROUTE_POLICIES[route].items()},
        "status": "installed_not_validated",
    }
