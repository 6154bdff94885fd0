"""W3 GEMV operator wrappers and the ``nn.Linear`` replacement for batch-1 decode.

Mirror of the reference's ``w3_lut_deployment`` module (reference file
``src/fluxbin_style/w3_lut_deployment.py``): same public names, argument meaning and
error behaviour, so code written against the reference runs unchanged.  What differs is
underneath: one ahead-of-time built sm_100a library reached through a C ABI instead of
per-row-tile JIT extensions.  ``row_tile``, ``groups_per_split`` and the ``workspace``
argument are still validated exactly as before but are advisory: the kernel chooses its
own tiling, reduces its K split internally and leaves a caller's workspace untouched
(the two-call form ``inline_main`` + ``finish`` does fill it, one row per group).
"""
from __future__ import annotations

from types import SimpleNamespace

import torch
from torch import nn
from torch.nn import functional as F

from . import _native
from .gptq_deployment import FIELDS, OPTIONAL_FIELDS, restore_planar_w3, validate_planar_w3

ROW_TILES = (256, 512, 1024)
EXPERIMENTAL_ROW_TILES = ROW_TILES + (2048,)
ARITHMETIC_MODES = ("structural", "decoded_bf16")
QWEN3_ROW_TILE_BY_SHAPE = {
    (4096, 4096): 256,
    (1024, 4096): 512,
    (12288, 4096): 1024,
    (4096, 12288): 1024,
}
_OBSERVED_EXACT_SPLIT = {(4096, 4096): 1, (1024, 4096): 1, (12288, 4096): 4, (4096, 12288): 2}


def _route_table(arithmetic: str, split_of=lambda shape: 1) -> dict:
    return {
        shape: {"row_tile": tile, "groups_per_split": split_of(shape), "arithmetic": arithmetic}
        for shape, tile in QWEN3_ROW_TILE_BY_SHAPE.items()
    }


QWEN3_W3_ROUTE_POLICIES = {
    "structural": _route_table("structural"),
    "fast_corrected": _route_table("decoded_bf16"),
    "observed_exact": _route_table("decoded_bf16", _OBSERVED_EXACT_SPLIT.__getitem__),
}


def w3_lut_extension_build(row_tile: int, uniform_index_probe: bool = False):
    """Describe the native build that serves ``row_tile``.

    The reference compiles one extension per row tile; here every row tile maps to the
    same prebuilt library, so the "build" is a description: ``(kwargs, contract)``.
    A timing-only wrong-result probe build does not exist in this library.
    """
    if row_tile not in EXPERIMENTAL_ROW_TILES:
        raise ValueError(f"row_tile must be one of {EXPERIMENTAL_ROW_TILES}")
    if uniform_index_probe:
        raise ValueError("the uniform-index timing probe is not part of this library")
    from .build import ARCH, COMMON, CSRC, EXTRA, LIBRARY

    kwargs = {
        "name": "fluxbin_b200",
        "sources": [str(CSRC / "fb_w3_gemv.cu")],
        "extra_cuda_cflags": [*ARCH, *COMMON, *EXTRA["fb_w3_gemv.cu"]],
    }
    contract = {"library": str(LIBRARY), "row_tile": row_tile, "row_tile_is_advisory": True}
    return kwargs, contract


def load_w3_lut_extension(row_tile: int, uniform_index_probe: bool = False):
    """Return an object with the reference extension's four entry points.

    ``inline_main``, ``inline_main_bf16_weight``, ``finish`` and ``m1_out`` take the same
    positional tensors as the reference's pybind functions (csrc/w3_lut.cu:334-339).
    """
    if row_tile not in EXPERIMENTAL_ROW_TILES:
        raise ValueError(f"row_tile must be one of {EXPERIMENTAL_ROW_TILES}")
    if uniform_index_probe:
        raise ValueError("the uniform-index timing probe is not part of this library")
    if not torch.cuda.is_available():
        raise RuntimeError("W3 LUT requires NVIDIA CUDA; no CPU/MPS substitution")
    _native.library()

    def _partials(x, planes, scales, perm, partial, corrected):
        _check_native_args(x, planes, scales, perm, partial, planes.shape[0])
        _native.w3_gemv(x, planes, scales, None, _perm_or_none(perm), partial,
                        decoded_bf16=corrected, group_partials=True)

    def inline_main(x, planes, scales, perm, partial):
        _partials(x, planes, scales, perm, partial, False)

    def inline_main_bf16_weight(x, planes, scales, perm, partial):
        _partials(x, planes, scales, perm, partial, True)

    def finish(partial, out):
        if partial.ndim != 2 or partial.dtype != torch.float32 or not partial.is_cuda:
            raise RuntimeError("partial must be CUDA FP32 [G,O]")
        if tuple(out.shape) != (1, partial.shape[1]) or out.dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError("out must be FP16/BF16 [1,O]")
        _native.w3_finish(partial, out)

    def m1_out(x, planes, scales, perm, partial, out, groups_per_split, dense_bf16_weight_semantics):
        groups = planes.shape[0]
        if not 0 < groups_per_split <= 255:
            raise RuntimeError("groups_per_split outside v1 bounds")
        _check_native_args(x, planes, scales, perm, partial, -(-groups // groups_per_split))
        if tuple(out.shape) != (1, planes.shape[2]) or out.dtype != x.dtype or out.device != x.device:
            raise RuntimeError("out must be contiguous same-device [1,O] with input dtype")
        _native.w3_gemv(x, planes, scales, None, _perm_or_none(perm), out,
                        decoded_bf16=bool(dense_bf16_weight_semantics))

    return SimpleNamespace(inline_main=inline_main, inline_main_bf16_weight=inline_main_bf16_weight,
                           finish=finish, m1_out=m1_out)


# perm tensors that were checked to be the identity: the kernel then skips the gather
_IDENTITY_PERMS: dict[tuple[int, int], bool] = {}


def _perm_or_none(perm: torch.Tensor):
    """``None`` when ``perm`` is the identity (decided once per tensor, outside capture)."""
    key = (perm.data_ptr(), perm.numel())
    known = _IDENTITY_PERMS.get(key)
    if known is None:
        if torch.cuda.is_current_stream_capturing():
            return perm  # cannot inspect values now; the general gather path is always valid
        known = bool(torch.equal(perm, torch.arange(perm.numel(), device=perm.device, dtype=perm.dtype)))
        if len(_IDENTITY_PERMS) > 4096:
            _IDENTITY_PERMS.clear()
        _IDENTITY_PERMS[key] = known
    return None if known else perm


def _check_native_args(x, planes, scales, perm, partial, splits) -> None:
    """The reference extension's argument contract (csrc/w3_lut.cu:191-226), as RuntimeError."""
    if not (x.is_cuda and x.is_contiguous() and x.ndim == 2 and x.shape[0] == 1):
        raise RuntimeError("CUDA x [1,K] required")
    for tensor in (planes, scales, perm, partial):
        if not (tensor.is_cuda and tensor.device == x.device and tensor.is_contiguous()):
            raise RuntimeError("all tensors must be contiguous on the input CUDA device")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("x must be FP16 or BF16")
    if planes.dtype != torch.uint8 or planes.ndim != 4 or planes.shape[1] != 3 or planes.shape[3] != 16:
        raise RuntimeError("planes must be uint8 [G,3,O,16]")
    groups, _, out_features, _ = planes.shape
    if not (0 < groups <= 255 and 0 < out_features <= 65536):
        raise RuntimeError("dimensions outside v1 bounds")
    if out_features % 32:
        raise RuntimeError("v1 requires O divisible by 32 for aligned plane rows")
    if x.shape[1] != groups * 128:
        raise RuntimeError("K mismatch")
    if scales.dtype not in (torch.bfloat16, torch.float16) or tuple(scales.shape) != (groups, out_features):
        raise RuntimeError("deployment scales must be BF16 [G,O]")
    if perm.dtype != torch.int16 or perm.ndim != 1 or perm.numel() != groups * 128:
        raise RuntimeError("perm must be int16 [K]")
    if partial.dtype != torch.float32 or tuple(partial.shape) != (splits, out_features):
        raise RuntimeError("partial has wrong FP32 [splits,O] shape")


def workspace_shape(out_features: int, in_features: int, groups_per_split: int = 1) -> tuple[int, int]:
    """Shape of the caller-owned FP32 workspace: one row per K split, ``O`` columns."""
    if not 1 <= out_features <= 65536 or not 128 <= in_features <= 32767 or in_features % 128:
        raise ValueError("invalid W3 LUT dimensions")
    groups = in_features // 128
    if not isinstance(groups_per_split, int) or not 1 <= groups_per_split <= groups:
        raise ValueError("groups_per_split must be an integer in [1,K/128]")
    return -(-groups // groups_per_split), out_features


def _layout_args(layout):
    return layout["planes"], layout["scales"], layout.get("zeros"), _perm_or_none(layout["perm"])


def inline_main(x, layout, workspace, *, row_tile: int, arithmetic: str = "structural") -> None:
    """First half of the two-call form: ``workspace[g, o]`` receives group ``g``'s scaled sum."""
    out_features, in_features = validate_planar_w3(layout, check_values=False)
    if x.shape != (1, in_features):
        raise ValueError("x must have shape [1,K]")
    if arithmetic not in ARITHMETIC_MODES:
        raise ValueError(f"arithmetic must be one of {ARITHMETIC_MODES}")
    if workspace.shape != workspace_shape(out_features, in_features) or workspace.dtype != torch.float32:
        raise ValueError("workspace must be FP32 [K/128,O]")
    if workspace.device != x.device or any(value.device != x.device for value in layout.values()):
        raise ValueError("x, layout and workspace must share a device")
    load_w3_lut_extension(row_tile)
    planes, scales, zeros, perm = _layout_args(layout)
    _native.w3_gemv(x, planes, scales, zeros, perm, workspace,
                    decoded_bf16=arithmetic == "decoded_bf16", group_partials=True)


def finish(workspace, out, *, row_tile: int):
    """Second half: ``out[0, o] = sum_g workspace[g, o]`` in ascending group order."""
    if workspace.ndim != 2 or workspace.dtype != torch.float32:
        raise ValueError("workspace must be FP32 [G,O]")
    if out.shape != (1, workspace.shape[1]) or out.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("out must be FP16/BF16 [1,O]")
    load_w3_lut_extension(row_tile).finish(workspace, out)
    return out


def w3_lut_m1_out(x, layout, out, workspace, *, row_tile: int, groups_per_split: int = 1,
                  arithmetic: str = "structural"):
    """Allocation-free M=1 GEMV on the current CUDA stream; returns ``out``.

    ``workspace`` must have the reference's shape for ``groups_per_split`` but is not
    written: the K split is reduced inside the kernel through a small per-stream scratch.
    """
    if out.dtype != x.dtype:
        raise ValueError("out dtype must match x dtype")
    if arithmetic not in ARITHMETIC_MODES:
        raise ValueError(f"arithmetic must be one of {ARITHMETIC_MODES}")
    out_features, in_features = validate_planar_w3(layout, check_values=False)
    if x.shape != (1, in_features) or out.shape != (1, out_features):
        raise ValueError("x/out shape mismatch")
    if workspace.shape != workspace_shape(out_features, in_features, groups_per_split) or workspace.dtype != torch.float32:
        raise ValueError("workspace must be FP32 [ceil(G/groups_per_split),O]")
    if workspace.device != x.device or out.device != x.device:
        raise ValueError("x, out and workspace must share a device")
    load_w3_lut_extension(row_tile)
    planes, scales, zeros, perm = _layout_args(layout)
    _native.w3_gemv(x, planes, scales, zeros, perm, out, decoded_bf16=arithmetic == "decoded_bf16")
    return out


def w3_lut_gemv_out(x, layout, out, *, arithmetic: str = "structural", kernel: str = "auto"):
    """Small-batch form (``x`` is ``[M,K]``, M = 1..16) of ``w3_lut_m1_out``; no reference counterpart.

    ``kernel``: ``"lut"`` is the table-lookup kernel (M <= 4, cost grows with M), ``"mma"`` the
    tensor-core kernel (M <= 16, cost independent of M; weights are rounded to the activation
    dtype, as the reference's dense fallback rounds them), ``"auto"`` picks ``"lut"`` up to M = 4
    (measured faster there on the Qwen3-8B shapes) and ``"mma"`` above.
    """
    out_features, in_features = validate_planar_w3(layout, check_values=False)
    if x.ndim != 2 or x.shape[1] != in_features or tuple(out.shape) != (x.shape[0], out_features):
        raise ValueError("x/out shape mismatch")
    if out.dtype != x.dtype or out.device != x.device:
        raise ValueError("out must match x in dtype and device")
    if kernel not in ("auto", "lut", "mma"):
        raise ValueError("kernel must be auto, lut or mma")
    rows = x.shape[0]
    if kernel == "auto":
        kernel = "lut" if rows <= 4 or arithmetic == "decoded_bf16" else "mma"
    if rows < 1 or rows > (4 if kernel == "lut" else 16):
        raise ValueError(f"the {kernel} kernel takes 1..{4 if kernel == 'lut' else 16} rows")
    planes, scales, zeros, perm = _layout_args(layout)
    if kernel == "mma":
        if arithmetic != "structural":
            raise ValueError("the tensor-core kernel has one arithmetic: weights rounded to the activation dtype")
        _native.w3_gemm_small(x, planes, scales, zeros, perm, out)
    else:
        _native.w3_gemv(x, planes, scales, zeros, perm, out, decoded_bf16=arithmetic == "decoded_bf16")
    return out


def qwen3_row_tile(out_features: int, in_features: int) -> int:
    try:
        return QWEN3_ROW_TILE_BY_SHAPE[(out_features, in_features)]
    except KeyError as exc:
        raise ValueError(f"unsupported Qwen3-8B W3 shape: {(out_features, in_features)}") from exc


def qwen3_w3_route(route: str, out_features: int, in_features: int) -> dict:
    if route not in QWEN3_W3_ROUTE_POLICIES:
        raise ValueError(f"unknown Qwen3-8B W3 route: {route}")
    try:
        return dict(QWEN3_W3_ROUTE_POLICIES[route][(out_features, in_features)])
    except KeyError as exc:
        raise ValueError(f"unsupported Qwen3-8B W3 shape: {(out_features, in_features)}") from exc


class PackedW3Linear(nn.Module):
    """Decode-only W3 ``Linear``: packed GEMV for one token, explicit dense fallback otherwise.

    Construction clones the layout into buffers.  A bound ("prepared") module owns one
    reusable ``[1,O]`` output and returns a view of it on every call, so a consumer must
    finish with it, on the same stream, before the next call; use is serial and batch-one,
    which is what a whole-sequence CUDA graph needs (no allocation per call).
    """

    def __init__(self, layout, *, bias=None, fallback: str = "error", row_tile: int | None = None,
                 groups_per_split: int = 1, arithmetic: str = "structural", route: str = "structural"):
        super().__init__()
        if fallback not in {"error", "dense"}:
            raise ValueError("fallback must be error or dense")
        self.out_features, self.in_features = validate_planar_w3(layout)
        self.row_tile = qwen3_row_tile(self.out_features, self.in_features) if row_tile is None else row_tile
        if self.row_tile not in ROW_TILES:
            raise ValueError(f"row_tile must be one of {ROW_TILES}")
        if arithmetic not in ARITHMETIC_MODES:
            raise ValueError(f"arithmetic must be one of {ARITHMETIC_MODES}")
        if arithmetic == "decoded_bf16" and "zeros" in layout:
            # the kernel's rounding correction covers code - zero = +/-3, the only inexact
            # products at zero points 3 and 4; other zero points have further inexact products
            zero_values = set(torch.unique(layout["zeros"]).tolist())
            if not zero_values <= {3, 4}:
                raise ValueError("decoded_bf16 arithmetic needs zero points 3 or 4")
        workspace_shape(self.out_features, self.in_features, groups_per_split)
        self.groups_per_split = groups_per_split
        self.arithmetic = arithmetic
        self.route = route
        self.fallback = fallback
        self.route_counts = {"packed_m1": 0, "dense_fallback": 0}
        self.last_route = "not_called"
        self._decode_binding = None
        self._decode_audit = False
        self._fields = tuple(name for name in FIELDS + OPTIONAL_FIELDS if name in layout)
        for name in self._fields:
            self.register_buffer(name, layout[name].detach().clone())
        self.register_buffer("bias", None if bias is None else bias.detach().clone())
        self.register_buffer("_workspace", None, persistent=False)
        self.register_buffer("_decode_output", None, persistent=False)

    def layout(self) -> dict[str, torch.Tensor]:
        return {name: getattr(self, name) for name in self._fields}

    def clear_prepared_decode(self) -> None:
        self._decode_binding = None
        self._decode_output = None
        self._workspace = None
        self._decode_audit = False

    def _apply(self, fn, recurse=True):
        # any device / dtype move invalidates the tensors a binding captured
        self.clear_prepared_decode()
        return super()._apply(fn, recurse=recurse)

    def bind_prepared_decode(self, dtype: torch.dtype) -> None:
        if self._decode_binding is not None:
            raise ValueError("decode already bound")
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("FP16/BF16 required")
        layout = self.layout()
        device = layout["planes"].device
        if device.type != "cuda":
            raise ValueError("prepared decode requires CUDA")
        validate_planar_w3(layout, check_values=False)
        load_w3_lut_extension(self.row_tile)
        planes, scales, zeros, perm = _layout_args(layout)
        corrected = self.arithmetic == "decoded_bf16"
        # The reference's workspace is kept (same shape contract) although the kernel does
        # not need it; the shared per-stream scratch is sized here, before any capture.
        self._workspace = torch.empty(
            workspace_shape(self.out_features, self.in_features, self.groups_per_split),
            device=device, dtype=torch.float32)
        _native.scratch_for(device, _native.w3_scratch_bytes(1, self.out_features, self.in_features))
        self._decode_output = torch.empty((1, self.out_features), device=device, dtype=dtype)
        output = self._decode_output
        shaped = output.view(1, 1, self.out_features)
        expected = (1, 1, self.in_features)
        in_features = self.in_features

        def apply(x: torch.Tensor) -> torch.Tensor:
            if torch.is_grad_enabled():
                raise RuntimeError("prepared decode is inference only")
            if tuple(x.shape) != expected or x.dtype != dtype or x.device != device or not x.is_contiguous():
                raise ValueError("prepared decode input shape/dtype/device/stride mismatch")
            if self._decode_audit:
                self.route_counts["packed_m1"] += 1
                self.last_route = "packed_m1"
            _native.w3_gemv(x.view(1, in_features), planes, scales, zeros, perm, output, decoded_bf16=corrected)
            if self.bias is not None:
                output.add_(self.bias)
            return shaped

        self._decode_binding = apply

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._decode_binding is not None:
            return self._decode_binding(x)
        if torch.is_grad_enabled():
            raise RuntimeError("packed inference requires no_grad/inference_mode")
        if x.ndim < 2 or x.shape[-1] != self.in_features:
            raise ValueError("expected [...,K] input")
        layout = self.layout()
        rows = x.numel() // self.in_features
        if rows != 1 or not x.is_cuda or x.dtype not in (torch.float16, torch.bfloat16):
            if self.fallback != "dense":
                raise ValueError("unsupported input; enable explicit dense fallback if needed")
            self.last_route = "dense_fallback"
            self.route_counts["dense_fallback"] += 1
            return F.linear(x, restore_planar_w3(layout, dtype=x.dtype), self.bias)
        self.last_route = "packed_m1"
        self.route_counts["packed_m1"] += 1
        shape = workspace_shape(self.out_features, self.in_features, self.groups_per_split)
        if self._workspace is None or self._workspace.device != x.device or tuple(self._workspace.shape) != shape:
            self._workspace = torch.empty(shape, device=x.device, dtype=torch.float32)
        output = torch.empty((1, self.out_features), device=x.device, dtype=x.dtype)
        w3_lut_m1_out(x.reshape(1, self.in_features).contiguous(), layout, output, self._workspace,
                      row_tile=self.row_tile, groups_per_split=self.groups_per_split, arithmetic=self.arithmetic)
        if self.bias is not None:
            output.add_(self.bias)
        return output.reshape(*x.shape[:-1], self.out_features)


def replace_w3_block_linears(block, layer_payload, *, fallback: str = "error",
                             row_tile_by_shape: dict[tuple[int, int], int] | None = None,
                             route: str = "structural") -> list[str]:
    """Swap the seven Linears of one Qwen3 decoder block; nothing is touched unless all seven validate."""
    from .qwen3 import QWEN3_LINEAR_MODULES

    fields_of = lambda name: [f for f in FIELDS + OPTIONAL_FIELDS if f"{name}.{f}" in layer_payload]  # noqa: E731
    required = {f"{module}.{field}" for module in QWEN3_LINEAR_MODULES for field in FIELDS}
    allowed = required | {f"{module}.{field}" for module in QWEN3_LINEAR_MODULES for field in OPTIONAL_FIELDS}
    if not required <= set(layer_payload) or not set(layer_payload) <= allowed:
        raise ValueError("layer must contain exactly seven complete W3 payloads")
    if route not in QWEN3_W3_ROUTE_POLICIES:
        raise ValueError(f"unknown Qwen3-8B W3 route: {route}")
    tiles = QWEN3_ROW_TILE_BY_SHAPE if row_tile_by_shape is None else row_tile_by_shape
    staged = []
    for name in QWEN3_LINEAR_MODULES:
        old = block.get_submodule(name)
        layout = {field: layer_payload[f"{name}.{field}"] for field in fields_of(name)}
        shape = validate_planar_w3(layout)
        if not isinstance(old, nn.Linear) or (old.out_features, old.in_features) != shape:
            raise ValueError(f"Linear shape/type mismatch: {name}")
        if shape not in tiles:
            raise ValueError(f"row-tile policy missing shape: {shape}")
        tile = tiles[shape]
        if row_tile_by_shape is None:
            policy = qwen3_w3_route(route, *shape)
            if policy["row_tile"] != tile:
                raise ValueError("route and row-tile policies disagree")
        else:
            policy = {"groups_per_split": 1, "arithmetic": "structural"}
        module = PackedW3Linear(layout, bias=old.bias, fallback=fallback, row_tile=tile,
                                groups_per_split=policy["groups_per_split"],
                                arithmetic=policy["arithmetic"], route=route).to(old.weight.device)
        staged.append((name, module))
    for name, module in staged:
        parent, attribute = name.rsplit(".", 1)
        setattr(block.get_submodule(parent), attribute, module)
    return [name for name, _ in staged]
