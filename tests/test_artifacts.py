"""Artifact loaders: manifest and hash checks run before anything is mutated
(behaviour of the reference's w3_lut_artifacts / deployment_artifacts, exercised on toy artifacts)."""
import hashlib
import json

import pytest
import torch
from safetensors.torch import save_file

from marlin_style_fluxbin_b200.gptq_deployment import FORMAT, convert_gptq_w3_to_planar
from marlin_style_fluxbin_b200.qwen3 import QWEN3_LINEAR_MODULES
from marlin_style_fluxbin_b200.w3_lut_artifacts import load_w3_lut_layer
from test_gptq_w3_planar import synthetic_raw


def _sha(path):
    return hashlib.sha256(path.read_bytes()).hexdigest()


def _write_artifact(root, *, status="completed_pending_gpu_validation"):
    (root / "payloads").mkdir(parents=True)
    raw, _, _ = synthetic_raw(k=128, o=32)
    layout = convert_gptq_w3_to_planar(raw, qzero_format=1)
    tensors = {f"{m}.{f}": v.clone() for m in QWEN3_LINEAR_MODULES for f, v in layout.items()}
    path = root / "payloads" / "layer-000.safetensors"
    save_file(tensors, str(path))
    manifest = {"status": status, "format": FORMAT,
                "canonical_semantics_gate": {"status": "confirmed_before_payload_writes", "inspected_linears": 252,
                                             "all_groups_have_128_columns": True, "decoded_zero_unique": [4]},
                "files": [{"path": "payloads/layer-000.safetensors", "bytes": path.stat().st_size, "sha256": _sha(path)}]}
    (root / "manifest.json").write_text(json.dumps(manifest))
    return _sha(root / "manifest.json")


def test_layer_loads_only_when_every_hash_matches(tmp_path):
    sha = _write_artifact(tmp_path)
    tensors, entry = load_w3_lut_layer(tmp_path, 0, expected_manifest_sha256=sha)
    assert len(tensors) == 21 and entry["path"].endswith("layer-000.safetensors")
    with pytest.raises(ValueError, match="manifest drift"):
        load_w3_lut_layer(tmp_path, 0, expected_manifest_sha256="0" * 64)
    with pytest.raises(ValueError, match="outside"):
        load_w3_lut_layer(tmp_path, 36, expected_manifest_sha256=sha)
    payload = tmp_path / "payloads" / "layer-000.safetensors"
    payload.write_bytes(payload.read_bytes()[:-1] + b"\x00")
    with pytest.raises(ValueError, match="hash/size drift"):
        load_w3_lut_layer(tmp_path, 0, expected_manifest_sha256=sha)


def test_manifest_status_is_checked(tmp_path):
    sha = _write_artifact(tmp_path, status="failed")
    with pytest.raises(ValueError, match="status/format drift"):
        load_w3_lut_layer(tmp_path, 0, expected_manifest_sha256=sha)


def test_public_surface_imports():
    import marlin_style_fluxbin_b200 as pkg
    from marlin_style_fluxbin_b200 import deployment_artifacts, engine_interface, w3_lut_artifacts  # noqa: F401

    assert int(pkg.pack_two_bases(torch.tensor([[[-1, 1, -1, 1]], [[-1, -1, 1, 1]]], dtype=torch.int8)).item()) == 0b11100100
    assert deployment_artifacts.MANIFEST_SHA.startswith("253ab448")
