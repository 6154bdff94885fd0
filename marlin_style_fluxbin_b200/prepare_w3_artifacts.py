"""Offline conversion of a raw GPTQ W3 checkpoint into the hash-pinned planar artifact that
``w3_lut_artifacts.load_w3_lut_layer`` / ``replace_w3_model_linears`` load.  CPU only.

    python -m marlin_style_fluxbin_b200.prepare_w3_artifacts --gptq-root SRC --expected-source-manifest-sha256 HEX --validate-only
    python -m marlin_style_fluxbin_b200.prepare_w3_artifacts --gptq-root SRC --expected-source-manifest-sha256 HEX --output-dir DST

Same protocol, inputs and outputs as the reference's converter script
(``scripts/prepare_qwen3_8b_w3_lut_artifacts.py:145-295``):

* the source is a directory with a pinned ``manifest.json`` (GPTQ bits 3, group 128, symmetric,
  desc_act; 252 Linears), ``raw_quantized/*.safetensors`` (``qweight / qzeros / scales / g_idx`` per
  Linear) and ``decoded_bf16/layer-NNN.safetensors`` (the quantiser's own dequantised weights);
* pass 1 inspects every Linear (groups of exactly 128 columns, decoded zero point 4 everywhere)
  before anything is written;
* pass 2 converts layer by layer and proves three things per Linear before its payload is kept:
  the stored scales equal the fp16 scales cast to bf16, the planes decode back to the checkpoint's
  integer codes, and the restored bf16 weight equals the quantiser's decoded weight bit for bit;
* payloads go to ``DST.incomplete/`` and the directory is renamed to ``DST`` only after the
  manifest (per-file size and sha256, the semantics gate, per-module records) has been written; a
  failure leaves ``DST.incomplete/failure.json`` and never a ``DST``.
"""
from __future__ import annotations

import argparse
import datetime as dt
import json
import os
from pathlib import Path

import torch

from .evaluation import sha256_file, tensor_sha256
from .gptq_deployment import (FIELDS, FORMAT, convert_gptq_w3_to_planar, decode_planar_w3_codes, inspect_gptq_checkpoint,
                              layout_storage, restore_planar_w3, unpack_gptq_w3_qweight)
from .qwen3 import QWEN3_LINEAR_MODULES

LAYERS = 36
RAW_FIELDS = ("qweight", "qzeros", "scales", "g_idx")
_SOURCE_GPTQ = {"bits": 3, "group_size": 128, "sym": True, "desc_act": True}
_CANONICALISATION = "per-Linear stable argsort(g_idx); identical permutation applied to K weights and runtime x"


def write_json_atomically(path: Path, value) -> None:
    """Write beside the target, flush to disk, then rename over it."""
    temporary = path.with_name(path.name + ".tmp")
    with open(temporary, "w", encoding="utf-8") as handle:
        json.dump(value, handle, indent=2, sort_keys=True)
        handle.flush()
        os.fsync(handle.fileno())
    temporary.replace(path)


class GptqSource:
    """A validated raw GPTQ W3 checkpoint directory: where every tensor lives, nothing loaded yet."""

    def __init__(self, root: Path, manifest_sha256: str, layers: int = LAYERS):
        from safetensors import safe_open

        self.root, self.layers, self._open = Path(root), layers, safe_open
        manifest_path = self.root / "manifest.json"
        if sha256_file(manifest_path) != manifest_sha256:
            raise ValueError("accepted GPTQ source manifest hash drifted")
        self.manifest = json.loads(manifest_path.read_text(encoding="utf-8"))
        if self.manifest.get("status") != "completed_pending_review":
            raise ValueError("GPTQ source status drifted")
        for name, wanted in _SOURCE_GPTQ.items():
            if self.manifest.get("gptq", {}).get(name) != wanted:
                raise ValueError(f"GPTQ source config drifted: {name}")
        self.linears = layers * len(QWEN3_LINEAR_MODULES)
        if self.manifest.get("coverage", {}).get("linear_count") != self.linears:
            raise ValueError("GPTQ source coverage drifted")
        raw_root, self.decoded_root = self.root / "raw_quantized", self.root / "decoded_bf16"
        if not raw_root.is_dir() or not self.decoded_root.is_dir():
            raise FileNotFoundError("raw_quantized/decoded_bf16 source directories are required")
        self.where: dict[str, Path] = {}
        for shard in sorted(raw_root.glob("*.safetensors")):
            with safe_open(shard, framework="pt", device="cpu") as handle:
                for key in handle.keys():
                    if key in self.where:
                        raise ValueError(f"duplicate safetensor key: {key}")
                    self.where[key] = shard
        if not self.where:
            raise FileNotFoundError(f"no safetensors under {raw_root}")
        wanted_modules = {self.module_name(layer, module) for layer in range(layers) for module in QWEN3_LINEAR_MODULES}
        found_modules = {key.rsplit(".", 1)[0] for key in self.where if key.rsplit(".", 1)[-1] in RAW_FIELDS}
        if found_modules != wanted_modules:
            raise ValueError(f"raw GPTQ target coverage drifted: missing={len(wanted_modules - found_modules)} "
                             f"extra={len(found_modules - wanted_modules)}")
        for module in wanted_modules:
            if any(f"{module}.{field}" not in self.where for field in RAW_FIELDS):
                raise ValueError(f"incomplete raw GPTQ module: {module}")
        for layer in range(layers):
            if not self.decoded_path(layer).is_file():
                raise FileNotFoundError(f"missing decoded layer {layer}")

    @staticmethod
    def module_name(layer: int, module: str) -> str:
        return f"model.layers.{layer}.{module}"

    def decoded_path(self, layer: int) -> Path:
        return self.decoded_root / f"layer-{layer:03d}.safetensors"

    def raw(self, layer: int, module: str) -> dict[str, torch.Tensor]:
        name = self.module_name(layer, module)
        tensors = {}
        for field in RAW_FIELDS:
            with self._open(self.where[f"{name}.{field}"], framework="pt", device="cpu") as handle:
                tensors[field] = handle.get_tensor(f"{name}.{field}").contiguous()
        return tensors

    def decoded(self, layer: int) -> dict[str, torch.Tensor]:
        with self._open(self.decoded_path(layer), framework="pt", device="cpu") as handle:
            if set(handle.keys()) != {f"{module}.weight" for module in QWEN3_LINEAR_MODULES}:
                raise ValueError(f"decoded layer inventory drifted: {layer}")
            return {module: handle.get_tensor(f"{module}.weight").contiguous() for module in QWEN3_LINEAR_MODULES}


def inspect_linear(source: GptqSource, layer: int, module: str) -> tuple[dict, dict]:
    """Raw tensors and structural facts of one Linear; the constant zero point 4 is required."""
    raw = source.raw(layer, module)
    facts = inspect_gptq_checkpoint(raw, qzero_format=1)
    if facts["decoded_zero_unique"] != [4]:
        raise ValueError(f"non-constant decoded zero: {source.module_name(layer, module)}")
    return raw, facts


def survey(source: GptqSource) -> tuple[list[dict], int]:
    """Pass 1: every Linear inspected, nothing written.  Returns the records and the number of
    Linears whose column order is not the identity."""
    records = []
    for layer in range(source.layers):
        for module in QWEN3_LINEAR_MODULES:
            _, facts = inspect_linear(source, layer, module)
            records.append({"name": source.module_name(layer, module), "facts": facts})
    if len(records) != source.linears:
        raise RuntimeError("canonical-semantics inspection coverage drifted")
    return records, sum(1 for record in records if not record["facts"]["permutation_identity"])


def convert_layer(source: GptqSource, layer: int) -> tuple[dict[str, torch.Tensor], list[dict]]:
    """Pass 2 for one decoder layer: the payload tensors and one proof record per Linear."""
    reference_weights = source.decoded(layer)
    payload, records = {}, []
    for module in QWEN3_LINEAR_MODULES:
        name = source.module_name(layer, module)
        raw, facts = inspect_linear(source, layer, module)
        layout = convert_gptq_w3_to_planar(raw, qzero_format=1)
        if not torch.equal(layout["scales"], raw["scales"].to(torch.bfloat16)):
            raise RuntimeError(f"loaded-BF16 scale cast failed: {name}")
        if not torch.equal(decode_planar_w3_codes(layout), unpack_gptq_w3_qweight(raw["qweight"])):
            raise RuntimeError(f"integer code round-trip failed: {name}")
        restored, decoded = restore_planar_w3(layout, dtype=torch.bfloat16), reference_weights[module]
        if not torch.equal(restored, decoded):
            raise RuntimeError(f"BF16 bitwise round-trip failed: {name}; mismatch={int(torch.count_nonzero(restored != decoded))}")
        records.append({
            "name": name, "facts": facts, "storage": layout_storage(layout),
            "decoded_bf16_sha256": tensor_sha256(decoded),
            "source_fp16_scales_sha256": tensor_sha256(raw["scales"]),
            "deployment_bf16_scales_sha256": tensor_sha256(layout["scales"]),
            "integer_codes_exact": True, "decoded_zero_exact": True,
            "deployment_scales_match_loaded_bf16_cast": True, "decoded_bf16_bitwise_exact": True,
        })
        payload.update({f"{module}.{field}": layout[field] for field in FIELDS})
    return payload, records


def publish(source: GptqSource, source_manifest_sha256: str, output_dir: Path, inspected: list[dict], inspected_nonidentity: int) -> Path:
    """Write all payloads and the manifest into ``output_dir.incomplete`` and rename it on success."""
    from safetensors.torch import save_file

    output_dir = Path(output_dir)
    staging = output_dir.with_name(output_dir.name + ".incomplete")
    for path in (output_dir, staging):
        if path.exists():
            raise FileExistsError(path)
    (staging / "payloads").mkdir(parents=True)
    try:
        files, modules = [], []
        for layer in range(source.layers):
            payload, records = convert_layer(source, layer)
            relative = Path("payloads") / f"layer-{layer:03d}.safetensors"
            save_file(payload, str(staging / relative))
            files.append({"layer": layer, "path": str(relative), "bytes": (staging / relative).stat().st_size,
                          "sha256": sha256_file(staging / relative)})
            modules += records
            print(f"FLUXBIN_W3_LUT_LAYER={layer + 1}/{source.layers}", flush=True)
        if len(modules) != source.linears:
            raise RuntimeError("converted Linear coverage drifted")
        package = Path(__file__).resolve().parent
        manifest = {
            "schema_version": 1,
            "status": "completed_pending_gpu_validation",
            "created_at_utc": dt.datetime.now(dt.timezone.utc).isoformat(),
            "format": FORMAT,
            "source_manifest_sha256": source_manifest_sha256,
            "source_runtime": source.manifest.get("runtime"),
            "qzero_format": 1,
            "canonicalization": _CANONICALISATION,
            "constant_zero_fast_path": 4,
            "canonical_semantics_gate": {
                "status": "confirmed_before_payload_writes", "inspected_linears": len(inspected),
                "nonidentity_permutations": inspected_nonidentity, "all_groups_have_128_columns": True, "decoded_zero_unique": [4],
            },
            "coverage": {
                "layers": source.layers, "linears": len(modules),
                "nonidentity_permutations": sum(1 for record in modules if not record["facts"]["permutation_identity"]),
                "integer_code_round_trip_exact": True, "decoded_zero_exact": True,
                "deployment_scales_match_loaded_bf16_cast": True, "decoded_bf16_bitwise_exact": True,
            },
            "deployment_tensor_bytes": sum(int(record["storage"]["total_bytes"]) for record in modules),
            "source_sha256": {str(path.relative_to(package.parent)): sha256_file(path)
                              for path in sorted(package.rglob("*")) if path.suffix in {".py", ".cu", ".cuh"}},
            "files": files,
            "modules": modules,
        }
        write_json_atomically(staging / "manifest.json", manifest)
        staging.rename(output_dir)
    except Exception:
        # a failed staging tree is kept for diagnosis and never published under the final name
        if staging.exists():
            write_json_atomically(staging / "failure.json", {"status": "failed"})
        raise
    return output_dir / "manifest.json"


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description="Inspect all raw GPTQ W3 Linears of a Qwen3-8B checkpoint and create exact planar payloads.")
    parser.add_argument("--gptq-root", type=Path, required=True)
    parser.add_argument("--output-dir", type=Path)
    parser.add_argument("--validate-only", action="store_true")
    parser.add_argument("--inspection-output", type=Path, help="optional JSON record of the validate-only pass")
    parser.add_argument("--expected-source-manifest-sha256", required=True)
    args = parser.parse_args(argv)
    if args.validate_only == (args.output_dir is not None):
        parser.error("use exactly one of --validate-only or --output-dir")
    if args.inspection_output is not None and not args.validate_only:
        parser.error("--inspection-output is valid only with --validate-only")
    source = GptqSource(args.gptq_root, args.expected_source_manifest_sha256)
    inspected, nonidentity = survey(source)
    if args.validate_only:
        if args.inspection_output is not None:
            if args.inspection_output.exists():
                raise FileExistsError(args.inspection_output)
            write_json_atomically(args.inspection_output, {
                "schema_version": 1, "status": "canonical_semantics_confirmed",
                "source_manifest_sha256": args.expected_source_manifest_sha256, "raw_qzero_format": 1, "desc_act": True,
                "canonicalization": _CANONICALISATION,
                "coverage": {"layers": source.layers, "linears": len(inspected), "nonidentity_permutations": nonidentity,
                             "all_groups_have_128_columns": True, "decoded_zero_unique": [4]},
                "modules": inspected,
            })
        print("FLUXBIN_W3_LUT_SOURCE_PREFLIGHT=passed; no conversion launched")
        return
    manifest = publish(source, args.expected_source_manifest_sha256, args.output_dir, inspected, nonidentity)
    print(f"FLUXBIN_W3_LUT_ARTIFACT={manifest}")


if __name__ == "__main__":
    main()
