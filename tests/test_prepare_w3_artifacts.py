"""The raw-GPTQ -> planar converter (counterpart of the reference's
scripts/prepare_qwen3_8b_w3_lut_artifacts.py): a toy 36-layer source tree goes through the
command line, and what it publishes loads back through ``load_w3_lut_layer`` with every hash
pinned; a source whose decoded weights disagree is never published."""
import hashlib
import json

import pytest
import torch
from safetensors.torch import save_file

from marlin_style_fluxbin_b200 import prepare_w3_artifacts as tool
from marlin_style_fluxbin_b200.gptq_deployment import convert_gptq_w3_to_planar, restore_planar_w3
from marlin_style_fluxbin_b200.qwen3 import QWEN3_LINEAR_MODULES
from marlin_style_fluxbin_b200.w3_lut_artifacts import load_w3_lut_layer
from test_gptq_w3_planar import synthetic_raw


def _sha(path):
    return hashlib.sha256(path.read_bytes()).hexdigest()


def write_source(root, *, corrupt_layer=None):
    """36 layers x 7 tiny Linears (128 or 256 inputs, 32 outputs), two raw shards, decoded weights per layer."""
    (root / "raw_quantized").mkdir(parents=True)
    (root / "decoded_bf16").mkdir()
    shards = ({}, {})
    for layer in range(tool.LAYERS):
        decoded = {}
        for index, module in enumerate(QWEN3_LINEAR_MODULES):
            raw, _, _ = synthetic_raw(k=128 if index % 2 else 256, o=32, seed=1000 * layer + index)
            for field, value in raw.items():
                shards[layer % 2][f"model.layers.{layer}.{module}.{field}"] = value
            weight = restore_planar_w3(convert_gptq_w3_to_planar(raw, qzero_format=1), dtype=torch.bfloat16)
            if layer == corrupt_layer and index == 3:
                weight = weight.clone()
                weight[0, 0] += 1
            decoded[f"{module}.weight"] = weight
        save_file(decoded, str(root / "decoded_bf16" / f"layer-{layer:03d}.safetensors"))
    for number, shard in enumerate(shards):
        save_file(shard, str(root / "raw_quantized" / f"model-{number:05d}.safetensors"))
    manifest = {"status": "completed_pending_review", "gptq": {"bits": 3, "group_size": 128, "sym": True, "desc_act": True},
                "coverage": {"linear_count": tool.LAYERS * len(QWEN3_LINEAR_MODULES)}, "runtime": {"torch": torch.__version__}}
    (root / "manifest.json").write_text(json.dumps(manifest))
    return _sha(root / "manifest.json")


def test_convert_publish_and_load_back(tmp_path, capsys):
    source, target = tmp_path / "gptq", tmp_path / "artifact"
    pin = write_source(source)
    tool.main(["--gptq-root", str(source), "--expected-source-manifest-sha256", pin, "--validate-only",
               "--inspection-output", str(tmp_path / "inspection.json")])
    inspection = json.loads((tmp_path / "inspection.json").read_text())
    assert inspection["coverage"]["linears"] == 252 and inspection["coverage"]["nonidentity_permutations"] == 36 * 4  # the one-group Linears sort to the identity
    assert not target.exists()
    tool.main(["--gptq-root", str(source), "--expected-source-manifest-sha256", pin, "--output-dir", str(target)])
    assert "FLUXBIN_W3_LUT_ARTIFACT=" in capsys.readouterr().out
    assert not (tmp_path / "artifact.incomplete").exists()
    manifest = json.loads((target / "manifest.json").read_text())
    assert manifest["coverage"]["decoded_bf16_bitwise_exact"] and len(manifest["files"]) == 36 and len(manifest["modules"]) == 252
    artifact_pin = _sha(target / "manifest.json")
    for layer in (0, 17, 35):
        tensors, entry = load_w3_lut_layer(target, layer, expected_manifest_sha256=artifact_pin)
        assert entry["layer"] == layer and len(tensors) == 21
        raw, _, _ = synthetic_raw(k=256, o=32, seed=1000 * layer)  # module 0 of that layer
        expected = convert_gptq_w3_to_planar(raw, qzero_format=1)
        for field, value in expected.items():
            assert torch.equal(tensors[f"{QWEN3_LINEAR_MODULES[0]}.{field}"], value)
    with pytest.raises(FileExistsError):
        tool.main(["--gptq-root", str(source), "--expected-source-manifest-sha256", pin, "--output-dir", str(target)])
    with pytest.raises(ValueError, match="manifest hash drifted"):
        tool.main(["--gptq-root", str(source), "--expected-source-manifest-sha256", "0" * 64, "--validate-only"])


def test_a_weight_that_does_not_round_trip_is_never_published(tmp_path):
    source, target = tmp_path / "gptq", tmp_path / "artifact"
    pin = write_source(source, corrupt_layer=2)
    with pytest.raises(RuntimeError, match="BF16 bitwise round-trip failed"):
        tool.main(["--gptq-root", str(source), "--expected-source-manifest-sha256", pin, "--output-dir", str(target)])
    assert not target.exists()
    assert json.loads((tmp_path / "artifact.incomplete" / "failure.json").read_text()) == {"status": "failed"}
