"""Hash-pinned loading of the two-base (hybrid g128-s8) model artifact and whole-model replacement.

Same two entry points, argument meaning and error behaviour as the reference's
``deployment_artifacts`` (``src/fluxbin_style/deployment_artifacts.py:13-69``).  The artifact is a
directory with a ``manifest.json`` (pinned by its own sha256; the default pin is the one the
reference holds for its retained artifact, ``manifest_sha256`` selects another artifact of the
same format) and one safetensors payload per decoder layer, pinned by the manifest through size
and sha256.  Loading is organised as a chain of small verifiers, each of which either returns what
the next one needs or raises ``ValueError``; the model is only touched after every layer has gone
through the whole chain.
"""
from __future__ import annotations

import json
from pathlib import Path

from .deployment import FIELDS
from .evaluation import sha256_file
from .qwen3 import QWEN3_LINEAR_MODULES, expected_qwen3_linear_shape
from .qwen3_8b import ARCHITECTURE

MANIFEST_SHA = "253ab448797ef4d798522875014b7e47a4edb84c5c3c1ca5cf6179edfd339fec"
_LAYERS = 36


def _manifest(root: Path, pin: str) -> dict:
    source = root / "manifest.json"
    if sha256_file(source) != pin:
        raise ValueError("step400 manifest drift")
    return json.loads(source.read_text())


def _listed_payload(root: Path, manifest: dict, layer: int) -> tuple[Path, dict]:
    """The payload file of ``layer`` and its manifest entry, after the size and hash pins held."""
    if layer not in range(_LAYERS):
        raise ValueError(f"layer outside 0..{_LAYERS - 1}")
    wanted = f"payloads/layer-{layer:03d}.safetensors"
    for entry in manifest["files"]:
        if entry["path"] == wanted:
            break
    else:
        raise ValueError("layer missing from the manifest")
    payload = root / wanted
    if (payload.stat().st_size, sha256_file(payload)) != (entry["bytes"], entry["sha256"]):
        raise ValueError("layer payload hash/size drift")
    return payload, entry


def _module_fields(tensors: dict, module: str) -> dict:
    return {field: tensors[f"{module}.{field}"] for field in FIELDS}


def load_accepted_layer(root, layer, *, manifest_sha256: str = MANIFEST_SHA):
    """All tensors of one decoder layer (seven Linears x the seven payload fields) and the layer's manifest entry."""
    from safetensors.torch import load_file

    root = Path(root)
    payload, entry = _listed_payload(root, _manifest(root, manifest_sha256), layer)
    tensors = load_file(payload)
    inventory = {f"{module}.{field}" for module in QWEN3_LINEAR_MODULES for field in FIELDS}
    if inventory.symmetric_difference(tensors):
        raise ValueError("layer inventory drift")
    for module in QWEN3_LINEAR_MODULES:
        rows, packed_columns = tensors[f"{module}.global_sign_codes"].shape  # four input positions per code byte
        if [rows, 4 * packed_columns] != expected_qwen3_linear_shape(ARCHITECTURE, module):
            raise ValueError(f"8B shape drift: {module}")
    return tensors, entry


def replace_model_linears(model, artifact_root: Path, *, allow_prefill_fallback=False, groups_per_split=8, kernel="v1",
                          manifest_sha256: str = MANIFEST_SHA):
    """Install the two-base Linears in all 36 blocks of a Qwen3-8B model.  Pass 1 reads and checks
    every layer against the model and changes nothing; pass 2 swaps the modules in, one layer's
    tensors in memory at a time.  Returns the installation report."""
    from torch import nn

    from . import deployment as two_base
    from .qwen3_8b import validate_architecture

    validate_architecture(model.config.to_dict())
    blocks = model.model.layers
    if len(blocks) != _LAYERS:
        raise ValueError(f"expected {_LAYERS} decoder layers")
    if kernel not in two_base.KERNELS:
        raise ValueError("unknown kernel")
    two_base.workspace_shape(1, 128, groups_per_split)  # rejects a groups_per_split outside the bounds

    def fetch(index):
        return load_accepted_layer(artifact_root, index, manifest_sha256=manifest_sha256)

    entries = []
    for index in range(_LAYERS):
        tensors, entry = fetch(index)
        for module in QWEN3_LINEAR_MODULES:
            out_features, groups = two_base.validate_artifact(_module_fields(tensors, module))
            dense = blocks[index].get_submodule(module)
            if not (isinstance(dense, nn.Linear) and (dense.out_features, dense.in_features) == (out_features, 128 * groups)):
                raise ValueError(f"Linear shape/type mismatch: layer {index} {module}")
        entries.append(entry)
        del tensors
    on_prefill = "dense" if allow_prefill_fallback else "error"
    installed = []
    for index, block in enumerate(blocks):
        swapped = two_base.replace_block_linears(block, fetch(index)[0], fallback=on_prefill, groups_per_split=groups_per_split, kernel=kernel)
        installed += [f"model.layers.{index}.{module}" for module in swapped]
    return {
        "format": two_base.PLANAR_FORMAT if kernel in two_base.PLANAR_KERNELS else two_base.FORMAT,
        "manifest_sha256": manifest_sha256,
        "layers": entries,
        "coverage": installed,
        "linear_count": len(installed),
        "kernel": kernel,
        "groups_per_split": groups_per_split,
        "prefill_fallback_enabled": allow_prefill_fallback,
        "status": "installed_not_validated",
    }
