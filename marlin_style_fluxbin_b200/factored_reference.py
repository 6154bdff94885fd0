"""High-precision structural reference for the two-base kernels (never a timed path).

Mirror of the reference's ``factored_reference`` (``src/fluxbin_style/factored_reference.py``):
fp32 payload coefficients promoted to fp64, one group's dense weights at a time.
"""
import torch

from .acceleration_checks import numerical_gate

REFERENCE = "hybrid-structural-fp64-v1"


def _signs(codes, positions, planar):
    """``codes`` of one group -> fp64 signs ``[O, positions, 2]``."""
    k = torch.arange(positions, device=codes.device)
    if planar:
        per_base = [((codes[:, b, :][:, k // 8].long() >> (k % 8)) & 1) * 2 - 1 for b in range(2)]
    else:
        pair = codes[:, k // 4].long() >> (2 * (k % 4))
        per_base = [(pair & 1) * 2 - 1, ((pair >> 1) & 1) * 2 - 1]
    return torch.stack(per_base, dim=-1).double()


@torch.no_grad()
def structural_reference(x, layout):
    """``[1,O]`` fp64 result of the factored form on a kernel layout (planar or interleaved)."""
    groups, o = layout["codes"].shape[:2]
    if tuple(x.shape) != (1, groups * 128):
        raise ValueError("expected [1,G*128]")
    planar = layout["codes"].ndim == 4
    total = torch.zeros(o, device=x.device, dtype=torch.float64)
    for g in range(groups):
        weight = (_signs(layout["codes"][g], 128, planar) * layout["rows"][g].double()[:, None, :]
                  * layout["columns"][g].double()[None, :, :]).sum(-1)
        delta = (_signs(layout["sparse_codes"][g], 8, planar) * layout["sparse_rows"][g].double()[:, None, :]
                 * layout["sparse_columns"][g].double()[None, :, :]).sum(-1)
        weight[:, layout["indices"][g].long()] += delta
        total += weight @ x[0, g * 128:(g + 1) * 128].double()
    return total[None, :]


def structural_gate(actual, expected):
    """The numerical gate against the fp64 structural output (bf16: factor 0.02, NRMSE limit 0.005)."""
    gate = numerical_gate(actual, expected)
    if actual.dtype == torch.bfloat16 and gate.get("reference_rms") is not None:
        rms = gate["reference_rms"]
        error = (actual.double() - expected).abs()
        gate.update(elementwise_tolerance_factor=0.02, normalized_rmse_limit=0.005,
                    passed=bool((error <= 0.02 * (rms + expected.abs()) + 1e-6).all()) and gate["normalized_rmse"] <= 0.005)
    gate["reference"] = REFERENCE
    return gate
