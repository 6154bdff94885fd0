"""Two-base binary-basis Linear with matrix-wide scales plus dense salient columns.

``W = diag(r_0) B_0 diag(c_0) + diag(r_1) B_1 diag(c_1) + S`` where ``B_b`` are {-1,+1} sign
matrices stored one bit per weight, ``r_b [O]`` / ``c_b [K]`` are fp16 and ``S`` is zero except
on ``n`` salient input columns, whose bf16 values are stored densely ``[O,n]``.  It is the
"one scale per row and per column, no refinement" case of the reference's two-base family
(the two-base part is what ``evaluation.py:59-95`` materialises with a single group), in the
configuration the decode benchmark is quoted on.  This module prepares the kernel layout
(planar codes ``[G,O,2,16]``, bit-exact permutation of the sign bits) and calls the kernel.
"""
from __future__ import annotations

import torch

from . import _native

FORMAT = "fluxbin-two-base-global-salient-m1-v1"
LAYOUT_FIELDS = ("codes", "row_scales", "column_scales", "salient_indices", "salient_values")


def pack_sign_planes(bases: torch.Tensor) -> torch.Tensor:
    """Signs ``[2,O,K]`` in {-1,+1} -> planar codes uint8 ``[K/128, O, 2, 16]`` (bit j of byte c = input 8c+j of the group, 1 = +1)."""
    if bases.ndim != 3 or bases.shape[0] != 2 or bases.shape[2] % 128:
        raise ValueError("bases must have shape [2, O, K] with K divisible by 128")
    if not bool(((bases == 1) | (bases == -1)).all()):
        raise ValueError("bases must contain only -1 and +1")
    _, o, k = bases.shape
    bits = (bases > 0).reshape(2, o, k // 128, 16, 8).to(torch.int32)
    weights = 2 ** torch.arange(8, dtype=torch.int32, device=bases.device)
    packed = (bits * weights).sum(-1).to(torch.uint8)  # [2, O, G, 16]
    return packed.permute(2, 1, 0, 3).contiguous()


def unpack_sign_planes(codes: torch.Tensor) -> torch.Tensor:
    """Inverse of ``pack_sign_planes``: int8 signs ``[2,O,K]``."""
    groups, o = codes.shape[:2]
    shifts = torch.arange(8, dtype=torch.int32, device=codes.device)
    bits = (codes.to(torch.int32).unsqueeze(-1) >> shifts) & 1  # [G,O,2,16,8]
    return (bits * 2 - 1).to(torch.int8).permute(2, 1, 0, 3, 4).reshape(2, o, groups * 128).contiguous()


def make_layout(bases, row_scales, column_scales, salient_indices, salient_values) -> dict[str, torch.Tensor]:
    _, o, k = bases.shape
    layout = {
        "codes": pack_sign_planes(bases),
        "row_scales": row_scales.to(torch.float16).contiguous(),
        "column_scales": column_scales.to(torch.float16).contiguous(),
        "salient_indices": salient_indices.to(torch.int32).contiguous(),
        "salient_values": salient_values.to(torch.bfloat16).contiguous(),
    }
    validate_layout(layout)
    return layout


def validate_layout(layout) -> tuple[int, int]:
    if set(layout) != set(LAYOUT_FIELDS):
        raise ValueError(f"expected exactly {LAYOUT_FIELDS}")
    codes = layout["codes"]
    if codes.dtype != torch.uint8 or codes.ndim != 4 or tuple(codes.shape[2:]) != (2, 16):
        raise ValueError("codes must be uint8 [G,O,2,16]")
    groups, o = codes.shape[:2]
    k = groups * 128
    n = layout["salient_indices"].numel()
    checks = (("row_scales", torch.float16, (2, o)), ("column_scales", torch.float16, (2, k)),
              ("salient_indices", torch.int32, (n,)), ("salient_values", torch.bfloat16, (o, n)))
    for name, dtype, shape in checks:
        value = layout[name]
        if value.dtype != dtype or tuple(value.shape) != shape or value.device != codes.device or not value.is_contiguous():
            raise ValueError(f"{name} must be contiguous {dtype} {list(shape)} on the codes' device")
    if n > 256:
        raise ValueError("at most 256 salient columns")
    return o, k


def materialize(layout, dtype=torch.float32) -> torch.Tensor:
    """Dense ``[O,K]`` weight: per base ``(sign * row) * column`` in fp32, base 0 then base 1, then the salient columns."""
    o, k = validate_layout(layout)
    signs = unpack_sign_planes(layout["codes"]).float()
    dense = torch.zeros(o, k, dtype=torch.float32, device=signs.device)
    for base in range(2):
        dense += (signs[base] * layout["row_scales"][base].float().unsqueeze(-1)) * layout["column_scales"][base].float().unsqueeze(0)
    dense[:, layout["salient_indices"].long()] += layout["salient_values"].float()
    return dense.to(dtype)


def workspace_bytes(out_features: int, in_features: int) -> int:
    return _native.bb_scratch_bytes(out_features, in_features, True)


def global_two_base_m1_out(x, layout, out):
    """``out[1,O] = x[1,K] . W^T`` on the current CUDA stream; allocation-free after warm-up."""
    o, k = validate_layout(layout)
    if tuple(x.shape) != (1, k) or tuple(out.shape) != (1, o) or out.dtype != x.dtype:
        raise ValueError("x/out shape or dtype mismatch")
    if not x.is_cuda or x.device != out.device or x.device != layout["codes"].device:
        raise ValueError("x, out and layout must share a CUDA device")
    n = layout["salient_indices"].numel()
    _native.bb_global_gemv(x, layout["codes"], layout["row_scales"], layout["column_scales"],
                           layout["salient_indices"] if n else None, layout["salient_values"] if n else None, out)
    return out
