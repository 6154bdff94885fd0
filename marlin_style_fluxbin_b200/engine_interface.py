"""Engine-neutral backend protocol for the two-base M=1 Linear (no serving-framework imports).

Same public surface as the reference's ``engine_interface``
(``src/fluxbin_style/engine_interface.py:15-60``): ``LinearContract`` describes what a backend
promises, ``LinearBackend`` is the structural type a serving adapter programs against and
``M1Backend`` is the one implementation.  A serving adapter owns weight loading, sharding,
streams, workspaces and scheduling; the backend owns layout conversion and the Linear operator
only.  Here the operator is the sm_100a binary-basis kernel behind ``deployment.m1_out``.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Mapping, Protocol, Tuple

import torch

from . import deployment as _dep

_Layout = Mapping[str, torch.Tensor]
_MAX_GROUPS_PER_SPLIT = 1024


@dataclass(frozen=True)
class LinearContract:
    """What a backend guarantees to the engine; field order and defaults follow the reference
    (``engine_interface.py:15-29``) so that positional construction and equality agree."""

    # artifact layout the backend's ``convert`` produces
    format: str = _dep.FORMAT
    # batch sizes the operator accepts (decode only)
    supported_m: Tuple[int, ...] = (1,)
    # activation / output dtypes
    input_dtypes: Tuple[torch.dtype, ...] = (torch.bfloat16, torch.float16)
    # dot products accumulate in fp32, scales are stored in fp32
    accumulation_dtype: torch.dtype = torch.float32
    scale_dtype: torch.dtype = torch.float32
    # quantisation geometry: inputs per scale group, dense salient columns per group
    group_size: int = 128
    sparse_columns: int = 8
    # name of the rounding scheme the oracle of this kernel family implements
    arithmetic: str = "combined_weight_activation_dtype_v1"
    # the reference's floor; this build itself needs (10, 0)
    minimum_compute_capability: Tuple[int, int] = (8, 0)
    # what the operator does NOT do for the engine
    fused_qkv: bool = False
    tensor_parallel: bool = False
    # a launch may be captured into a CUDA graph once the first call has run
    graph_capture_after_warmup: bool = True


class LinearBackend(Protocol):
    """Structural type of a backend (``engine_interface.py:32-39``)."""

    contract: LinearContract

    def convert(self, artifact: _Layout) -> dict[str, torch.Tensor]:
        """Quantisation artifact -> the kernel's device layout."""
        ...

    def workspace_shape(self, out_features: int, in_features: int) -> tuple[int, ...]:
        """Shape of the fp32 workspace ``apply_out`` needs for one Linear."""
        ...

    def apply_out(self, x: torch.Tensor, layout: _Layout, out: torch.Tensor,
                  workspace: torch.Tensor) -> torch.Tensor:
        """``out[:] = W @ x`` for one activation row; returns ``out``."""
        ...


def _contract_for(kernel: str) -> LinearContract:
    """The factored kernels accumulate scale-free sums in fp32 and apply the scales afterwards
    (a different rounding order, hence a different ``arithmetic`` tag); the planar ones also
    read the bit-plane layout (``engine_interface.py:47-49``)."""
    base = LinearContract()
    if kernel not in _dep.FACTORED_KERNELS:
        return base
    layout = _dep.PLANAR_FORMAT if kernel in _dep.PLANAR_KERNELS else _dep.FORMAT
    return replace(base, arithmetic="factored_fp32_v1", format=layout)


class M1Backend:
    """The batch-1 backend (``engine_interface.py:42-60``); error messages as the reference's."""

    contract = LinearContract()

    def __init__(self, groups_per_split=8, *, kernel="v1"):
        if kernel not in _dep.KERNELS:
            raise ValueError(f"kernel must be one of {_dep.KERNELS}")
        in_range = isinstance(groups_per_split, int) and 1 <= groups_per_split <= _MAX_GROUPS_PER_SPLIT
        if not in_range:
            raise ValueError("groups_per_split must be 1..1024")
        self.kernel = kernel
        self.groups_per_split = groups_per_split
        self.contract = _contract_for(kernel)

    def _options(self):
        return {"kernel": self.kernel}

    def convert(self, artifact):
        return _dep.convert_artifact(artifact, **self._options())

    def workspace_shape(self, out_features, in_features):
        return _dep.workspace_shape(out_features, in_features, self.groups_per_split, **self._options())

    def apply_out(self, x, layout, out, workspace):
        return _dep.m1_out(x, layout, out, workspace, groups_per_split=self.groups_per_split,
                           **self._options())
