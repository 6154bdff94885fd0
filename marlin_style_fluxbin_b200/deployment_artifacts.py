"""Hash-pinned loading of the two-base (hybrid g128-s8) model artifact and whole-model replacement.

Mirror of the reference's ``deployment_artifacts`` (``src/fluxbin_style/deployment_artifacts.py:13-69``).
The manifest hash below is the one the reference pins for its retained artifact; pass
``manifest_sha256`` to use another artifact of the same format.
"""
from __future__ import annotations

import json
from pathlib import Path

from .deployment import FIELDS
from .evaluation import sha256_file
from .qwen3 import QWEN3_LINEAR_MODULES, expected_qwen3_linear_shape
from .qwen3_8b import ARCHITECTURE

MANIFEST_SHA = "253ab448797ef4d798522875014b7e47a4edb84c5c3c1ca5cf6179edfd339fec"


def load_accepted_layer(root, layer, *, manifest_sha256: str = MANIFEST_SHA):
    from safetensors.torch import load_file

    root = Path(root)
    manifest_path = root / "manifest.json"
    if sha256_file(manifest_path) != manifest_sha256:
        raise ValueError("step400 manifest drift")
    manifest = json.loads(manifest_path.read_text())
    if not 0 <= layer < 36:
        raise ValueError("layer outside 0..35")
    relative = f"payloads/layer-{layer:03d}.safetensors"
    entry = next((e for e in manifest["files"] if e["path"] == relative), None)
    if entry is None:
        raise ValueError("layer missing from the manifest")
    path = root / relative
    if path.stat().st_size != entry["bytes"] or sha256_file(path) != entry["sha256"]:
        raise ValueError("layer payload hash/size drift")
    tensors = load_file(path)
    if set(tensors) != {f"{name}.{field}" for name in QWEN3_LINEAR_MODULES for field in FIELDS}:
        raise ValueError("layer inventory drift")
    for name in QWEN3_LINEAR_MODULES:
        shape = tensors[f"{name}.global_sign_codes"].shape
        if [shape[0], shape[1] * 4] != expected_qwen3_linear_shape(ARCHITECTURE, name):
            raise ValueError(f"8B shape drift: {name}")
    return tensors, entry


def replace_model_linears(model, artifact_root: Path, *, allow_prefill_fallback=False, groups_per_split=8, kernel="v1",
                          manifest_sha256: str = MANIFEST_SHA):
    """Install the two-base Linears in all 36 blocks of a Qwen3-8B model after validating every layer first."""
    from torch import nn

    from .deployment import FORMAT, KERNELS, PLANAR_FORMAT, PLANAR_KERNELS, replace_block_linears, validate_artifact, workspace_shape
    from .qwen3_8b import validate_architecture

    validate_architecture(model.config.to_dict())
    if len(model.model.layers) != 36:
        raise ValueError("expected 36 decoder layers")
    if kernel not in KERNELS:
        raise ValueError("unknown kernel")
    workspace_shape(1, 128, groups_per_split)
    records = []
    for index in range(36):
        payload, entry = load_accepted_layer(artifact_root, index, manifest_sha256=manifest_sha256)
        for name in QWEN3_LINEAR_MODULES:
            o, g = validate_artifact({field: payload[f"{name}.{field}"] for field in FIELDS})
            target = model.model.layers[index].get_submodule(name)
            if not isinstance(target, nn.Linear) or (target.out_features, target.in_features) != (o, g * 128):
                raise ValueError(f"Linear shape/type mismatch: layer {index} {name}")
        records.append(entry)
    coverage = []
    for index, block in enumerate(model.model.layers):
        payload, _ = load_accepted_layer(artifact_root, index, manifest_sha256=manifest_sha256)
        names = replace_block_linears(block, payload, fallback="dense" if allow_prefill_fallback else "error",
                                      groups_per_split=groups_per_split, kernel=kernel)
        coverage.extend(f"model.layers.{index}.{name}" for name in names)
    return {"format": PLANAR_FORMAT if kernel in PLANAR_KERNELS else FORMAT, "manifest_sha256": manifest_sha256,
            "layers": records, "coverage": coverage, "linear_count": len(coverage), "kernel": kernel,
            "groups_per_split": groups_per_split, "prefill_fallback_enabled": allow_prefill_fallback,
            "status": "installed_not_validated"}
