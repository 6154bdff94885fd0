"""Dense materialisers of the two-base formats (oracles and prefill fallback) and hashing.

Mirror of the parts of the reference's ``evaluation`` module that the decode path uses
(``src/fluxbin_style/evaluation.py:19-34`` hashing, ``:59-175`` materialisers).  The
arithmetic order is kept: per base ``(sign * row_scale) * column_scale`` in fp32, base 0
then base 1 accumulated, refinement columns summed the same way and scatter-added last.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .packing import unpack_two_bases


def sha256_file(path: Path) -> str:
    digest = hashlib.sha256()
    with Path(path).open("rb") as stream:
        while True:
            chunk = stream.read(1 << 20)
            if not chunk:
                break
            digest.update(chunk)
    return digest.hexdigest()


def tensor_sha256(tensor: torch.Tensor) -> str:
    """Hash of dtype, shape and raw bytes (in that order)."""
    value = tensor.detach().cpu().contiguous()
    digest = hashlib.sha256()
    digest.update(str(value.dtype).encode("ascii"))
    digest.update(json.dumps(list(value.shape)).encode("ascii"))
    digest.update(value.view(torch.uint8).numpy().tobytes())
    return digest.hexdigest()


def _two_base_sum(signs, row, column):
    """``signs [2,O,G,W]``, ``row [2,O,G]``, ``column [2,G,W]`` -> fp32 ``[O,G,W]``."""
    total = torch.zeros(signs.shape[1:], dtype=torch.float32, device=signs.device)
    for base in range(2):
        term = signs[base].to(torch.float32)
        term = term * row[base].unsqueeze(-1)
        term = term * column[base].unsqueeze(0)
        total = total + term
    return total


def _check_scales(name, value, shape):
    if tuple(value.shape) != shape:
        raise ValueError(f"{name} shape drifted")
    if not value.is_floating_point() or not bool(torch.isfinite(value).all()):
        raise ValueError(f"{name} must be finite floating point")


def materialize_global_two_base_weight(sign_codes, row_scales, column_scales, *, group_size, device, output_dtype):
    """``W[o, g*S+j] = sum_b sign_b * row_b[o,g] * col_b[g,j]`` from packed sign codes."""
    if not isinstance(group_size, int) or group_size <= 0:
        raise ValueError("group_size must be positive")
    if sign_codes.ndim != 2 or sign_codes.dtype != torch.uint8:
        raise ValueError("global sign codes must be a uint8 matrix")
    out_features, in_features = sign_codes.shape[0], sign_codes.shape[1] * 4
    if in_features % group_size:
        raise ValueError("packed input width is not divisible by group_size")
    groups = in_features // group_size
    _check_scales("global row-scale", row_scales, (2, out_features, groups))
    _check_scales("global column-scale", column_scales, (2, groups, group_size))
    signs = unpack_two_bases(sign_codes.to(device)).reshape(2, out_features, groups, group_size)
    dense = _two_base_sum(signs, row_scales.to(device=device, dtype=torch.float32),
                          column_scales.to(device=device, dtype=torch.float32))
    return dense.reshape(out_features, in_features).to(output_dtype)


def materialize_hybrid_s8_weight(global_sign_codes, global_row_scales, global_column_scales, refinement_indices,
                                 refinement_sign_codes, refinement_row_scales, refinement_column_scales, *,
                                 group_size, columns_per_group, device, output_dtype):
    """Global two-base weight plus a two-base refinement on ``columns_per_group`` columns per group."""
    dense = materialize_global_two_base_weight(global_sign_codes, global_row_scales, global_column_scales,
                                               group_size=group_size, device=device, output_dtype=torch.float32)
    out_features, in_features = dense.shape
    groups = in_features // group_size
    if refinement_indices.dtype not in (torch.int16, torch.int32, torch.int64):
        raise TypeError("refinement indices must use an integer dtype")
    if tuple(refinement_indices.shape) != (groups, columns_per_group):
        raise ValueError("refinement indices have the wrong shape")
    indices = refinement_indices.to(device=device, dtype=torch.int64)
    if bool((indices < 0).any()) or bool((indices >= group_size).any()):
        raise ValueError("refinement indices are outside the group")
    if columns_per_group > 1 and bool((indices[:, 1:] <= indices[:, :-1]).any()):
        raise ValueError("refinement indices must be sorted and unique")
    if tuple(refinement_sign_codes.shape) != (out_features, groups * columns_per_group // 4):
        raise ValueError("refinement sign-code shape drifted")
    _check_scales("refinement row-scale", refinement_row_scales, (2, out_features, groups))
    _check_scales("refinement column-scale", refinement_column_scales, (2, groups, columns_per_group))
    signs = unpack_two_bases(refinement_sign_codes.to(device)).reshape(2, out_features, groups, columns_per_group)
    selected = _two_base_sum(signs, refinement_row_scales.to(device=device, dtype=torch.float32),
                             refinement_column_scales.to(device=device, dtype=torch.float32))
    grouped = dense.reshape(out_features, groups, group_size)
    grouped.scatter_add_(2, indices.unsqueeze(0).expand(out_features, -1, -1), selected)
    return grouped.reshape(out_features, in_features).to(output_dtype)
