"""Lossless two-bit storage of two {-1,+1} bases: four input positions per byte.

Mirror of the reference's ``packing`` module (``src/fluxbin_style/packing.py:14-49``): in
byte ``i`` of a row, bit ``2j`` is base 0 at position ``4i+j`` and bit ``2j+1`` is base 1,
with +1 stored as 1 and -1 as 0.
"""
from __future__ import annotations

import torch

TWO_BASE_PACKED_FORMAT = "fluxbin-two-base-interleaved-2bit-v1"


def pack_two_bases(bases: torch.Tensor) -> torch.Tensor:
    """``bases`` ``[2,O,K]`` in {-1,+1} -> ``uint8 [O,K/4]``."""
    if bases.ndim != 3 or bases.shape[0] != 2:
        raise ValueError("bases must have shape [2, out_features, in_features]")
    if bases.shape[-1] % 4:
        raise ValueError("in_features must be divisible by four")
    if not bool(((bases == 1) | (bases == -1)).all()):
        raise ValueError("bases must contain only -1 and +1")
    _, rows, cols = bases.shape
    # [O, K/4, 4 positions, 2 bases] -> bit index 2*position + base
    bit = (bases > 0).permute(1, 2, 0).reshape(rows, cols // 4, 8).to(torch.int32)
    weight = 2 ** torch.arange(8, dtype=torch.int32, device=bases.device)
    return (bit * weight).sum(-1).to(torch.uint8)


def unpack_two_bases(codes: torch.Tensor) -> torch.Tensor:
    """``uint8 [O,K/4]`` -> ``int8 [2,O,K]`` in {-1,+1}."""
    if codes.ndim != 2 or codes.dtype != torch.uint8:
        raise ValueError("codes must be a uint8 tensor shaped [out_features, K/4]")
    rows, quarter = codes.shape
    position = torch.arange(8, dtype=torch.int32, device=codes.device)
    bit = (codes.to(torch.int32).unsqueeze(-1) >> position) & 1  # [O, K/4, 8]
    signs = (bit * 2 - 1).to(torch.int8).reshape(rows, quarter * 4, 2)
    return signs.permute(2, 0, 1).contiguous()
