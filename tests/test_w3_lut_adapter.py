"""CPU-side contract of the W3 operator wrappers and the Linear adapter (no GPU needed);
cases follow the reference's tests/test_w3_lut_adapter.py and test_w3_lut_correctness.py."""
import ctypes
import re
from pathlib import Path

import pytest
import torch
from torch import nn

from marlin_style_fluxbin_b200.gptq_deployment import convert_gptq_w3_to_planar, restore_planar_w3
from marlin_style_fluxbin_b200.qwen3 import QWEN3_LINEAR_MODULES
from marlin_style_fluxbin_b200.w3_lut_deployment import (
    EXPERIMENTAL_ROW_TILES, PackedW3Linear, load_w3_lut_extension, qwen3_row_tile, qwen3_w3_route,
    replace_w3_block_linears, w3_lut_extension_build, workspace_shape,
)
from test_gptq_w3_planar import synthetic_raw

ROOT = Path(__file__).resolve().parents[1]


def tiny_layout(out_features=32, in_features=128):
    raw, _, _ = synthetic_raw(k=in_features, o=out_features)
    return convert_gptq_w3_to_planar(raw, qzero_format=1)


def tiny_block():
    block = nn.Module()
    block.self_attn, block.mlp = nn.Module(), nn.Module()
    for name in QWEN3_LINEAR_MODULES:
        parent, attribute = name.rsplit(".", 1)
        setattr(block.get_submodule(parent), attribute, nn.Linear(128, 32, bias=False))
    return block


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "fluxbin_b200.h").read_text()
    declared = set(re.findall(r"\b(fb_[a-z0-9_]+)\s*\(", header))
    assert {"fb_w3_gemv", "fb_w3_finish", "fb_last_error", "fb_query", "fb_w3_gemv_scratch_bytes"} <= declared
    from marlin_style_fluxbin_b200 import build

    lib = ctypes.CDLL(str(build.build()))
    for symbol in declared:
        assert hasattr(lib, symbol), symbol
    lib.fb_w3_gemv_scratch_bytes.restype = ctypes.c_size_t
    assert lib.fb_w3_gemv_scratch_bytes(1, 4096, 4096) == 16384 + (2 << 20)  # status block + combine words
    assert lib.fb_w3_gemv_scratch_bytes(1, 4096, 12288) == 16384 + (2 << 20) + 16 * 4096 * 4  # + partials of 16 super-blocks
    assert lib.fb_w3_gemv_scratch_bytes(1, 64, 256) == 16384 + (2 << 20)  # the layout does not depend on the problem


def test_workspace_and_extension_variants():
    assert workspace_shape(1024, 4096) == (32, 1024)
    assert workspace_shape(1024, 4096, 4) == (8, 1024)
    assert workspace_shape(1024, 4096, 32) == (1, 1024)
    for bad in ((1024, 4097, 1), (1024, 4096, 0)):
        with pytest.raises(ValueError):
            workspace_shape(*bad)
    for row_tile in EXPERIMENTAL_ROW_TILES:
        kwargs, contract = w3_lut_extension_build(row_tile)
        assert kwargs["sources"][0].endswith("fb_w3_gemv.cu") and contract["row_tile"] == row_tile
        assert "arch=compute_100a,code=sm_100a" in kwargs["extra_cuda_cflags"]
    with pytest.raises(ValueError):
        load_w3_lut_extension(128)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU"):
            load_w3_lut_extension(256)


def test_dense_fallback_and_fail_closed():
    layout = tiny_layout()
    module = PackedW3Linear(layout, fallback="dense", row_tile=256)
    x = torch.randn(2, 128, dtype=torch.bfloat16)
    with torch.inference_mode():
        assert torch.equal(module(x), torch.nn.functional.linear(x, restore_planar_w3(layout)))
    assert module.route_counts == {"packed_m1": 0, "dense_fallback": 1}
    strict = PackedW3Linear(layout, row_tile=256)
    with torch.inference_mode(), pytest.raises(ValueError, match="unsupported input"):
        strict(torch.randn(1, 128, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        strict(torch.randn(1, 128, dtype=torch.bfloat16))  # grad enabled
    with pytest.raises(ValueError, match="prepared decode requires CUDA"):
        strict.bind_prepared_decode(torch.bfloat16)
    strict._decode_binding = lambda x: x
    strict.to("cpu")
    assert strict._decode_binding is None


def test_policies_are_frozen():
    assert [qwen3_row_tile(*s) for s in ((4096, 4096), (1024, 4096), (12288, 4096), (4096, 12288))] == [256, 512, 1024, 1024]
    with pytest.raises(ValueError):
        qwen3_row_tile(32, 128)
    for shape, (tile, split) in {(4096, 4096): (256, 1), (1024, 4096): (512, 1), (12288, 4096): (1024, 4), (4096, 12288): (1024, 2)}.items():
        assert qwen3_w3_route("fast_corrected", *shape) == {"row_tile": tile, "groups_per_split": 1, "arithmetic": "decoded_bf16"}
        assert qwen3_w3_route("observed_exact", *shape) == {"row_tile": tile, "groups_per_split": split, "arithmetic": "decoded_bf16"}
        assert qwen3_w3_route("structural", *shape)["arithmetic"] == "structural"
    with pytest.raises(ValueError):
        qwen3_w3_route("missing", 4096, 4096)
    module = PackedW3Linear(tiny_layout(), row_tile=256, arithmetic="decoded_bf16", route="fast_corrected")
    assert (module.arithmetic, module.groups_per_split, module.route) == ("decoded_bf16", 1, "fast_corrected")
    with pytest.raises(ValueError):
        PackedW3Linear(tiny_layout(), row_tile=256, arithmetic="missing")


def test_block_replacement_validates_before_mutating():
    layout = tiny_layout()
    payload = {f"{name}.{field}": value.clone() for name in QWEN3_LINEAR_MODULES for field, value in layout.items()}
    block = tiny_block()
    broken = dict(payload)
    broken.pop("mlp.down_proj.perm")
    with pytest.raises(ValueError):
        replace_w3_block_linears(block, broken, row_tile_by_shape={(32, 128): 256})
    assert all(isinstance(block.get_submodule(n), nn.Linear) for n in QWEN3_LINEAR_MODULES)
    names = replace_w3_block_linears(block, payload, fallback="dense", row_tile_by_shape={(32, 128): 256})
    assert names == list(QWEN3_LINEAR_MODULES)
    assert all(isinstance(block.get_submodule(n), PackedW3Linear) for n in QWEN3_LINEAR_MODULES)
    with torch.inference_mode():
        assert tuple(block.self_attn.q_proj(torch.zeros(3, 128)).shape) == (3, 32)
