"""Two-base binary-basis (hybrid g128-s8) layout, M=1 operator and ``nn.Linear`` replacement.

Mirror of the reference's ``deployment`` module (``src/fluxbin_style/deployment.py:19-320``):
the seven-field payload, its lossless permutation into the kernel layout (interleaved or
planar codes), the ``m1_out`` operator and ``PackedHybridLinear``.  All of the reference's
kernel names are accepted; they select the LAYOUT (planar for ``v5_p*``, interleaved
otherwise) and the workspace shape contract, and all run the one sm_100a kernel
(``fb_bb_gemv``), whose arithmetic is the reference's factored fp32 form (``v4``/``v5``).
``groups_per_split`` and the caller's ``workspace`` are validated but advisory.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Mapping

import torch
from torch import nn
from torch.nn import functional as F

from . import _native
from .evaluation import materialize_hybrid_s8_weight, tensor_sha256

FORMAT = "fluxbin-hybrid-g128-s8-m1-v1"
PLANAR_FORMAT = "fluxbin-hybrid-g128-s8-m1-planar-v1"
PLANAR_KERNELS = ("v5_p256", "v5_p512", "v5_p1024")
FACTORED_KERNELS = ("v4", "v4_late", "v5") + PLANAR_KERNELS
KERNELS = ("v1", "v2_r1", "v2_r2", "v2", "v3") + FACTORED_KERNELS
FIELDS = ("global_sign_codes", "global_row_scales", "global_column_scales", "refinement_indices",
          "refinement_sign_codes", "refinement_row_scales", "refinement_column_scales")
LAYOUT_FIELDS = ("codes", "rows", "columns", "indices", "sparse_codes", "sparse_rows", "sparse_columns", "lookup")


def validate_artifact(p: Mapping[str, torch.Tensor]) -> tuple[int, int]:
    """Check the seven payload fields; returns ``(out_features, groups)``."""
    if set(p) != set(FIELDS):
        raise ValueError("expected exactly seven hybrid payload fields")
    codes = p["global_sign_codes"]
    if codes.ndim != 2 or codes.dtype != torch.uint8:
        raise ValueError("global codes must be uint8 [O,K/4]")
    o, width = codes.shape
    if not 1 <= o <= 65536 or not 32 <= width <= 32768 or width % 32:
        raise ValueError("v1 requires O=1..65536 and K=128..131072 divisible by 128")
    g = width // 32
    expected = {"global_sign_codes": (o, width), "global_row_scales": (2, o, g), "global_column_scales": (2, g, 128),
                "refinement_indices": (g, 8), "refinement_sign_codes": (o, g * 2),
                "refinement_row_scales": (2, o, g), "refinement_column_scales": (2, g, 8)}
    for name, shape in expected.items():
        value = p[name]
        if tuple(value.shape) != shape or value.device != codes.device:
            raise ValueError(f"shape/device mismatch: {name}")
        if "scales" in name and (value.dtype != torch.float32 or not bool(torch.isfinite(value).all())):
            raise ValueError(f"finite FP32 scales required: {name}")
    if p["refinement_sign_codes"].dtype != torch.uint8:
        raise ValueError("refinement codes must be uint8")
    index = p["refinement_indices"]
    if index.dtype not in (torch.int16, torch.int32, torch.int64):
        raise ValueError("integer refinement indices required")
    if bool((index < 0).any()) or bool((index >= 128).any()) or bool((index[:, 1:] <= index[:, :-1]).any()):
        raise ValueError("indices must be sorted, unique and inside each group")
    return o, g


def _gather_bits(word: torch.Tensor, offset: int) -> torch.Tensor:
    """Bits ``offset, offset+2, ...`` (eight of them) of a 16-bit value -> one byte."""
    out = torch.zeros_like(word)
    for j in range(8):
        out |= ((word >> (2 * j + offset)) & 1) << j
    return out.to(torch.uint8)


def _to_planes(codes: torch.Tensor) -> torch.Tensor:
    """Interleaved bytes ``[..., 2n]`` -> planes ``[..., 2, n]`` (base 0 bits, base 1 bits)."""
    word = codes[..., 0::2].to(torch.int32) | (codes[..., 1::2].to(torch.int32) << 8)
    return torch.stack((_gather_bits(word, 0), _gather_bits(word, 1)), dim=-2)


def _from_planes(planes: torch.Tensor) -> torch.Tensor:
    low, high = planes[..., 0, :].to(torch.int32), planes[..., 1, :].to(torch.int32)
    word = torch.zeros_like(low)
    for j in range(8):
        word |= (((low >> j) & 1) << (2 * j)) | (((high >> j) & 1) << (2 * j + 1))
    return torch.stack((word & 0xFF, word >> 8), dim=-1).flatten(-2).to(torch.uint8)


def layout_format(layout) -> str:
    return PLANAR_FORMAT if layout["codes"].ndim == 4 else FORMAT


def convert_artifact(p: Mapping[str, torch.Tensor], *, kernel="v1") -> dict[str, torch.Tensor]:
    """Payload -> kernel layout.  A pure permutation: sign bits, fp32 scales and indices survive unchanged."""
    if kernel not in KERNELS:
        raise ValueError("unknown kernel")
    o, g = validate_artifact(p)
    index = p["refinement_indices"].to(torch.int16)
    lookup = torch.full((g, 128), -1, dtype=torch.int16, device=index.device)
    lookup.scatter_(1, index.long(), torch.arange(8, dtype=torch.int16, device=index.device).expand(g, 8))
    layout = {
        "codes": p["global_sign_codes"].reshape(o, g, 32).transpose(0, 1),
        "rows": p["global_row_scales"].permute(2, 1, 0),
        "columns": p["global_column_scales"].permute(1, 2, 0),
        "indices": index,
        "sparse_codes": p["refinement_sign_codes"].reshape(o, g, 2).transpose(0, 1),
        "sparse_rows": p["refinement_row_scales"].permute(2, 1, 0),
        "sparse_columns": p["refinement_column_scales"].permute(1, 2, 0),
        "lookup": lookup,
    }
    layout = {name: value.contiguous().clone() for name, value in layout.items()}
    if kernel in PLANAR_KERNELS:
        layout["codes"] = _to_planes(layout["codes"]).contiguous()
        layout["sparse_codes"] = _to_planes(layout["sparse_codes"]).contiguous()
    return layout


def restore_artifact(layout: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    g, o = layout["codes"].shape[:2]
    codes, sparse = layout["codes"], layout["sparse_codes"]
    if codes.ndim == 4:
        codes, sparse = _from_planes(codes), _from_planes(sparse)
    payload = {
        "global_sign_codes": codes.transpose(0, 1).reshape(o, g * 32),
        "global_row_scales": layout["rows"].permute(2, 1, 0),
        "global_column_scales": layout["columns"].permute(2, 0, 1),
        "refinement_indices": layout["indices"],
        "refinement_sign_codes": sparse.transpose(0, 1).reshape(o, g * 2),
        "refinement_row_scales": layout["sparse_rows"].permute(2, 1, 0),
        "refinement_column_scales": layout["sparse_columns"].permute(2, 0, 1),
    }
    return {name: value.contiguous() for name, value in payload.items()}


def decode_layout(layout: Mapping[str, torch.Tensor], dtype=torch.bfloat16) -> torch.Tensor:
    """Dense ``[O,K]`` weight of a kernel layout (prefill fallback and oracle)."""
    return materialize_hybrid_s8_weight(**restore_artifact(layout), group_size=128, columns_per_group=8,
                                        device=layout["codes"].device, output_dtype=dtype)


def conversion_record(source, layout) -> dict:
    return {"format": layout_format(layout),
            "source": {name: tensor_sha256(value) for name, value in source.items()},
            "layout": {name: tensor_sha256(value) for name, value in layout.items()},
            "layout_bytes": sum(value.numel() * value.element_size() for value in layout.values())}


def workspace_shape(out_features: int, in_features: int, groups_per_split=8, *, kernel="v1"):
    """Shape contract of the caller-owned FP32 workspace (kept for drop-in use; not written)."""
    if kernel not in KERNELS:
        raise ValueError("unknown kernel")
    if (not isinstance(groups_per_split, int) or not 1 <= groups_per_split <= 1024
            or not 1 <= out_features <= 65536 or not 128 <= in_features <= 131072 or in_features % 128):
        raise ValueError("invalid group/split dimensions")
    groups = in_features // 128
    splits = -(-groups // groups_per_split)
    if kernel in ("v4", "v4_late"):
        return (groups * 272 + splits * out_features,)
    return (splits, out_features)


def _check_call(x, layout, out, workspace, groups_per_split, kernel) -> None:
    """Argument contract of the reference extension (csrc/m1_v5.cu:136-180), as RuntimeError."""
    planar = kernel in PLANAR_KERNELS
    tensors = [x, out, workspace] + [layout[name] for name in LAYOUT_FIELDS]
    if not (x.is_cuda and x.ndim == 2 and x.shape[0] == 1):
        raise RuntimeError("CUDA [1,K] required")
    if any(not (t.is_cuda and t.device == x.device and t.is_contiguous()) for t in tensors):
        raise RuntimeError("all tensors must be contiguous on input CUDA device")
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError("BF16/FP16 only")
    codes = layout["codes"]
    if codes.dtype != torch.uint8 or (planar and (codes.ndim != 4 or tuple(codes.shape[2:]) != (2, 16))) or (
            not planar and (codes.ndim != 3 or codes.shape[2] != 32)):
        raise RuntimeError("codes do not match the kernel's layout; use convert_artifact")
    groups, o = codes.shape[0], codes.shape[1]
    if x.shape[1] != groups * 128:
        raise RuntimeError("K mismatch")
    if tuple(out.shape) != (1, o) or out.dtype != x.dtype:
        raise RuntimeError("output mismatch")
    if tuple(workspace.shape) != workspace_shape(o, groups * 128, groups_per_split, kernel=kernel) or workspace.dtype != torch.float32:
        raise RuntimeError("workspace shape mismatch")
    for name in ("rows", "columns", "sparse_rows", "sparse_columns"):
        if layout[name].dtype != torch.float32:
            raise RuntimeError("FP32 scales/workspace required")


def load_extension(kernel="v1"):
    """Object with the reference extension's ``m1_out`` entry point for ``kernel``."""
    if kernel not in KERNELS:
        raise ValueError(f"kernel must be one of {KERNELS}")
    if not torch.cuda.is_available():
        raise RuntimeError("M=1 kernel requires NVIDIA CUDA; no CPU/MPS substitution")
    _native.library()

    def native_m1_out(x, codes, rows, cols, sparse, sparse_rows, sparse_cols, indices_or_lookup, out, workspace, gps):
        layout = {"codes": codes, "rows": rows, "columns": cols, "sparse_codes": sparse, "sparse_rows": sparse_rows,
                  "sparse_columns": sparse_cols, "indices": indices_or_lookup, "lookup": indices_or_lookup}
        if kernel not in FACTORED_KERNELS:  # those extensions receive the [G,128] lookup instead of the indices
            lookup = indices_or_lookup
            layout["indices"] = _indices_from_lookup(lookup)
        _check_call(x, layout, out, workspace, int(gps), kernel)
        _native.bb_gemv(x, layout, out)

    return SimpleNamespace(m1_out=native_m1_out)


_LOOKUP_CACHE: dict[int, torch.Tensor] = {}


def _indices_from_lookup(lookup: torch.Tensor) -> torch.Tensor:
    """Recover the sorted ``[G,8]`` column indices from a ``[G,128]`` position lookup (cached per tensor)."""
    key = lookup.data_ptr()
    cached = _LOOKUP_CACHE.get(key)
    if cached is None or cached.shape[0] != lookup.shape[0] or cached.device != lookup.device:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("first use of a lookup tensor must happen before graph capture")
        cached = torch.nonzero(lookup >= 0)[:, 1].reshape(lookup.shape[0], 8).to(torch.int16).contiguous()
        _LOOKUP_CACHE[key] = cached
    return cached


def m1_out(x, layout, out, workspace, *, groups_per_split=8, kernel="v1"):
    """Engine-neutral M=1 operator on the current CUDA stream; the caller owns ``out`` and ``workspace``.

    fp16/bf16 activations, fp32 accumulation, no allocation after warm-up, only a contiguous
    ``[1,K]`` input, no hidden fallback.  Returns ``out``.
    """
    if kernel not in KERNELS:
        raise ValueError(f"kernel must be one of {KERNELS}")
    if not torch.cuda.is_available():
        raise RuntimeError("M=1 kernel requires NVIDIA CUDA; no CPU/MPS substitution")
    _check_call(x, layout, out, workspace, groups_per_split, kernel)
    _native.bb_gemv(x, layout, out)
    return out


class PackedHybridLinear(nn.Module):
    """Decode-only two-base ``Linear`` for HF blocks; serving engines may call ``m1_out`` directly.

    Strict by default (anything but one CUDA fp16/bf16 token is rejected); ``fallback='dense'``
    reconstructs the weight on demand for prefill.  The fp32 scale buffers must stay fp32:
    move the module with ``.to(device)``, never ``.half()``.
    """

    def __init__(self, payload, *, bias=None, fallback="error", groups_per_split=8, kernel="v1"):
        super().__init__()
        if fallback not in ("error", "dense"):
            raise ValueError("fallback must be error or dense")
        if kernel not in KERNELS:
            raise ValueError("unknown kernel")
        self.kernel = kernel
        self.route_counts = {"packed_m1": 0, "dense_fallback": 0}
        self.out_features, groups = validate_artifact(payload)
        self.in_features = groups * 128
        self.fallback, self.groups_per_split = fallback, groups_per_split
        workspace_shape(self.out_features, self.in_features, groups_per_split)
        for name, value in convert_artifact(payload, kernel=kernel).items():
            self.register_buffer(name, value)
        self.register_buffer("bias", None if bias is None else bias.detach().clone())
        self.register_buffer("_workspace", None, persistent=False)
        self.register_buffer("_decode_output", None, persistent=False)
        self.last_route = "not_called"
        self._decode_binding = None
        self._decode_audit = False

    def layout(self):
        return {name: getattr(self, name) for name in LAYOUT_FIELDS}

    def clear_prepared_decode(self):
        self._decode_binding = None
        self._decode_output = None
        self._decode_audit = False

    def _apply(self, fn, recurse=True):
        self.clear_prepared_decode()  # captured tensor references die with a device / dtype move
        return super()._apply(fn, recurse=recurse)

    def _require_fp32_scales(self):
        if any(getattr(self, n).dtype != torch.float32 for n in ("rows", "columns", "sparse_rows", "sparse_columns")):
            raise ValueError("FP32 scale buffers were cast; move devices without dtype conversion")

    def bind_prepared_decode(self, dtype):
        """Bind serial ``[1,1,K]`` decoding; every call returns a view of one reusable output buffer."""
        if self._decode_binding is not None:
            raise ValueError("decode already bound")
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("FP16/BF16 required")
        layout = self.layout()
        device = self.codes.device
        if device.type != "cuda":
            raise ValueError("prepared decode requires CUDA")
        if any(t.device != device or not t.is_contiguous() for t in layout.values()):
            raise ValueError("contiguous same-device layout required")
        self._require_fp32_scales()
        load_extension(self.kernel)
        self._workspace = torch.empty(workspace_shape(self.out_features, self.in_features, self.groups_per_split,
                                                      kernel=self.kernel), device=device, dtype=torch.float32)
        _native.scratch_for(device, _native.bb_scratch_bytes(self.out_features, self.in_features, False), "bb")
        self._decode_output = torch.empty((1, self.out_features), device=device, dtype=dtype)
        output = self._decode_output
        shaped = output.view(1, 1, self.out_features)
        expected = (1, 1, self.in_features)
        in_features = self.in_features

        def apply(x):
            if torch.is_grad_enabled():
                raise RuntimeError("prepared decode is inference only")
            if tuple(x.shape) != expected or x.dtype != dtype or x.device != device or not x.is_contiguous():
                raise ValueError("prepared decode input shape/dtype/device/stride mismatch")
            if self._decode_audit:
                self.route_counts["packed_m1"] += 1
                self.last_route = "packed_m1"
            _native.bb_gemv(x.view(1, in_features), layout, output)
            if self.bias is not None:
                output.add_(self.bias)
            return shaped

        self._decode_binding = apply

    def forward(self, x):
        if self._decode_binding is not None:
            return self._decode_binding(x)
        if torch.is_grad_enabled():
            raise RuntimeError("packed inference requires no_grad/inference_mode")
        if x.ndim < 2 or x.shape[-1] != self.in_features:
            raise ValueError("expected [...,K] input")
        self._require_fp32_scales()
        rows = x.numel() // self.in_features
        if rows != 1 or not x.is_cuda or x.dtype not in (torch.float16, torch.bfloat16):
            if self.fallback != "dense":
                raise ValueError("unsupported input; enable explicit dense fallback if needed")
            self.last_route = "dense_fallback"
            self.route_counts["dense_fallback"] += 1
            return F.linear(x, decode_layout(self.layout(), x.dtype), self.bias)
        self.last_route = "packed_m1"
        self.route_counts["packed_m1"] += 1
        shape = workspace_shape(self.out_features, self.in_features, self.groups_per_split, kernel=self.kernel)
        if self._workspace is None or self._workspace.device != x.device:
            self._workspace = torch.empty(shape, device=x.device, dtype=torch.float32)
        y = torch.empty((1, self.out_features), device=x.device, dtype=x.dtype)
        m1_out(x.reshape(1, self.in_features).contiguous(), self.layout(), y, self._workspace,
               groups_per_split=self.groups_per_split, kernel=self.kernel)
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*x.shape[:-1], self.out_features)


def replace_block_linears(block, layer_payload, *, fallback="error", groups_per_split=8, kernel="v1"):
    """Swap the seven Linears of one Qwen3 block; every replacement is built before any is installed."""
    from .qwen3 import QWEN3_LINEAR_MODULES

    if set(layer_payload) != {f"{module}.{field}" for module in QWEN3_LINEAR_MODULES for field in FIELDS}:
        raise ValueError("layer must contain exactly seven complete hybrid payloads")
    staged = []
    for name in QWEN3_LINEAR_MODULES:
        old = block.get_submodule(name)
        payload = {field: layer_payload[f"{name}.{field}"] for field in FIELDS}
        o, g = validate_artifact(payload)
        if not isinstance(old, nn.Linear) or (old.out_features, old.in_features) != (o, g * 128):
            raise ValueError(f"Linear shape/type mismatch: {name}")
        staged.append((name, PackedHybridLinear(payload, bias=old.bias, fallback=fallback,
                                                groups_per_split=groups_per_split, kernel=kernel).to(old.weight.device)))
    for name, module in staged:
        parent, attribute = name.rsplit(".", 1)
        setattr(block.get_submodule(parent), attribute, module)
    return [name for name, _ in staged]
