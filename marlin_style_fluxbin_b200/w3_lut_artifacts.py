"""Hash-bound loading of offline W3 deployment artifacts and whole-model replacement.

Same two entry points and error behaviour as the reference's ``w3_lut_artifacts``
(``src/fluxbin_style/w3_lut_artifacts.py:14-118``).  An artifact directory holds a
``manifest.json`` whose sha256 the caller pins, and one safetensors file per decoder layer which
the manifest pins by size and sha256.  The checks are organised as a small pipeline here
(manifest -> entry -> file -> inventory -> per-Linear layout), and ``replace_w3_model_linears``
changes no module until every layer of the model has passed all of them.
"""
from __future__ import annotations

import json
from pathlib import Path

from .evaluation import sha256_file
from .gptq_deployment import FIELDS, FORMAT, validate_planar_w3
from .qwen3 import QWEN3_LINEAR_MODULES

_LAYERS = 36
_LINEARS = _LAYERS * len(QWEN3_LINEAR_MODULES)
_MANIFEST_STATUS = "completed_pending_gpu_validation"
# the quantiser's self-check that the manifest must carry (w3_lut_artifacts.py:23-30): all
# Linears inspected, every group 128 columns wide, zero point 4 everywhere
_GATE = {
    "status": "confirmed_before_payload_writes",
    "inspected_linears": _LINEARS,
    "all_groups_have_128_columns": True,
    "decoded_zero_unique": [4],
}


def _fail(what: str):
    raise ValueError(f"W3 LUT {what}")


def _pinned_manifest(root: Path, pin: str) -> dict:
    """The manifest, after its own hash, status, format and semantics gate have been checked."""
    source = root / "manifest.json"
    if sha256_file(source) != pin:
        _fail("manifest drift")
    manifest = json.loads(source.read_text(encoding="utf-8"))
    if (manifest.get("status"), manifest.get("format")) != (_MANIFEST_STATUS, FORMAT):
        _fail("manifest status/format drift")
    gate = manifest.get("canonical_semantics_gate", {})
    for key, wanted in _GATE.items():
        found = gate.get(key)
        if found != wanted or (wanted is True and found is not True):
            _fail("canonical-semantics gate missing or drifted")
    return manifest


def _linear_fields(tensors: dict, module: str) -> dict:
    return {field: tensors[f"{module}.{field}"] for field in FIELDS}


def load_w3_lut_layer(root: Path, layer: int, *, expected_manifest_sha256: str) -> tuple[dict, dict]:
    """Tensors of one decoder layer (seven Linears x three fields) and its manifest entry."""
    from safetensors.torch import load_file

    root = Path(root)
    manifest = _pinned_manifest(root, expected_manifest_sha256)
    if layer not in range(_LAYERS):
        raise ValueError(f"layer outside 0..{_LAYERS - 1}")
    name = f"payloads/layer-{layer:03d}.safetensors"
    listed = [item for item in manifest["files"] if item["path"] == name]
    if not listed:
        _fail("layer missing from the manifest")
    entry, payload = listed[0], root / name
    if (payload.stat().st_size, sha256_file(payload)) != (entry["bytes"], entry["sha256"]):
        _fail("layer hash/size drift")
    tensors = load_file(payload)
    wanted = {f"{module}.{field}" for module in QWEN3_LINEAR_MODULES for field in FIELDS}
    if wanted.symmetric_difference(tensors):
        _fail("layer inventory drift")
    for module in QWEN3_LINEAR_MODULES:
        validate_planar_w3(_linear_fields(tensors, module))
    return tensors, entry


def _shape_table(table: dict, convert=lambda value: value) -> dict:
    """{(out, in): v} -> {"OUTxIN": v}, the JSON-friendly form the report uses."""
    return {f"{shape[0]}x{shape[1]}": convert(value) for shape, value in table.items()}


def replace_w3_model_linears(model, artifact_root: Path, *, expected_manifest_sha256: str,
                             allow_prefill_fallback: bool = False, route: str = "structural") -> dict:
    """Install all 252 hash-bound W3 Linears of a Qwen3-8B model; attention and cache code stay
    untouched.  Returns the installation report (``w3_lut_artifacts.py:97-118``)."""
    from torch import nn

    from . import w3_lut_deployment as lut
    from .qwen3 import expected_qwen3_linear_shape
    from .qwen3_8b import ARCHITECTURE, validate_architecture

    validate_architecture(model.config.to_dict())
    blocks = model.model.layers
    if len(blocks) != _LAYERS:
        raise ValueError(f"expected {_LAYERS} decoder layers")
    if route not in lut.QWEN3_W3_ROUTE_POLICIES:
        raise ValueError(f"unknown Qwen3-8B W3 route: {route}")

    def fetch(index):
        return load_w3_lut_layer(artifact_root, index, expected_manifest_sha256=expected_manifest_sha256)

    def check(index, module, tensors):
        shape = validate_planar_w3(_linear_fields(tensors, module))
        if list(shape) != expected_qwen3_linear_shape(ARCHITECTURE, module):
            raise ValueError(f"8B W3 shape drift: layer {index} {module}")
        dense = blocks[index].get_submodule(module)
        if not (isinstance(dense, nn.Linear) and (dense.out_features, dense.in_features) == shape):
            raise ValueError(f"Linear shape/type mismatch: layer {index} {module}")

    # pass 1 reads and validates every layer and mutates nothing
    entries = []
    for index in range(_LAYERS):
        tensors, entry = fetch(index)
        for module in QWEN3_LINEAR_MODULES:
            check(index, module, tensors)
        entries.append(entry)
        del tensors
    # pass 2 swaps the modules in, one layer's tensors in memory at a time
    on_prefill = "dense" if allow_prefill_fallback else "error"
    installed = []
    for index, block in enumerate(blocks):
        swapped = lut.replace_w3_block_linears(block, fetch(index)[0], fallback=on_prefill, route=route)
        installed += [f"model.layers.{index}.{module}" for module in swapped]
    return {
        "format": FORMAT,
        "manifest_sha256": expected_manifest_sha256,
        "layers": entries,
        "coverage": installed,
        "linear_count": len(installed),
        "row_tile_by_shape": _shape_table(lut.QWEN3_ROW_TILE_BY_SHAPE),
        "prefill_fallback_enabled": allow_prefill_fallback,
        "route": route,
        "route_policy": _shape_table(lut.QWEN3_W3_ROUTE_POLICIES[route], dict),
        "status": "installed_not_validated",
    }
