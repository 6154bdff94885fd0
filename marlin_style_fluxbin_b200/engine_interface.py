"""Engine-neutral backend protocol for the two-base M=1 Linear (no serving-framework imports).

Mirror of the reference's ``engine_interface`` (``src/fluxbin_style/engine_interface.py:15-60``).
A serving adapter owns weight loading, streams, workspaces and scheduling; the backend owns
layout conversion and the Linear operator only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Protocol

import torch

from .deployment import (FACTORED_KERNELS, FORMAT, KERNELS, PLANAR_FORMAT, PLANAR_KERNELS, convert_artifact, m1_out,
                         workspace_shape)


@dataclass(frozen=True)
class LinearContract:
    format: str = FORMAT
    supported_m: tuple[int, ...] = (1,)
    input_dtypes: tuple[torch.dtype, ...] = (torch.bfloat16, torch.float16)
    accumulation_dtype: torch.dtype = torch.float32
    scale_dtype: torch.dtype = torch.float32
    group_size: int = 128
    sparse_columns: int = 8
    arithmetic: str = "combined_weight_activation_dtype_v1"
    minimum_compute_capability: tuple[int, int] = (8, 0)
    fused_qkv: bool = False
    tensor_parallel: bool = False
    graph_capture_after_warmup: bool = True


class LinearBackend(Protocol):
    contract: LinearContract

    def convert(self, artifact: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]: ...
    def workspace_shape(self, out_features: int, in_features: int) -> tuple[int, ...]: ...
    def apply_out(self, x: torch.Tensor, layout: Mapping[str, torch.Tensor], out: torch.Tensor,
                  workspace: torch.Tensor) -> torch.Tensor: ...


class M1Backend:
    contract = LinearContract()

    def __init__(self, groups_per_split=8, *, kernel="v1"):
        if kernel not in KERNELS:
            raise ValueError(f"kernel must be one of {KERNELS}")
        if not isinstance(groups_per_split, int) or not 1 <= groups_per_split <= 1024:
            raise ValueError("groups_per_split must be 1..1024")
        self.kernel, self.groups_per_split = kernel, groups_per_split
        if kernel in FACTORED_KERNELS:
            self.contract = LinearContract(arithmetic="factored_fp32_v1",
                                           format=PLANAR_FORMAT if kernel in PLANAR_KERNELS else FORMAT)

    def convert(self, artifact):
        return convert_artifact(artifact, kernel=self.kernel)

    def workspace_shape(self, out_features, in_features):
        return workspace_shape(out_features, in_features, self.groups_per_split, kernel=self.kernel)

    def apply_out(self, x, layout, out, workspace):
        return m1_out(x, layout, out, workspace, groups_per_split=self.groups_per_split, kernel=self.kernel)
