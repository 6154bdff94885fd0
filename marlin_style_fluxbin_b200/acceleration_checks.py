"""Numerical gate and paired CUDA timing used to judge a packed kernel against a baseline.

Same contract as the reference's ``acceleration_checks`` module
(``src/fluxbin_style/acceleration_checks.py:7-64``): the gate combines an element-wise
bound ``|e| <= tol*(rms(ref) + |ref|) + 1e-6`` with ``NRMSE <= tol/4`` (tol 0.02 for a
bf16 reference, 0.002 otherwise); timing interleaves the arms round by round.
"""
from __future__ import annotations

import statistics

import torch


def numerical_gate(actual, expected):
    if actual.shape != expected.shape:
        return {"passed": False, "reason": "shape mismatch"}
    got, want = actual.detach().double(), expected.detach().double()
    if not bool(torch.isfinite(got).all()) or not bool(torch.isfinite(want).all()):
        return {"passed": False, "reason": "nonfinite output"}
    rms = float(want.square().mean().sqrt())
    error = got - want
    nrmse = float(error.square().mean().sqrt()) / max(rms, 1e-12)
    tol = 0.02 if expected.dtype == torch.bfloat16 else 0.002
    within = bool((error.abs() <= tol * (rms + want.abs()) + 1e-6).all())
    return {
        "passed": within and nrmse <= tol / 4,
        "max_abs_error": float(error.abs().max()),
        "reference_rms": rms,
        "normalized_rmse": nrmse,
        "elementwise_tolerance_factor": tol,
        "normalized_rmse_limit": tol / 4,
    }


def stepwise_nrmse(actual, expected):
    """NRMSE per decode step of a ``[1,steps,vocab]`` logits trace (report only), else None."""
    if actual.shape != expected.shape or actual.ndim != 3 or actual.shape[0] != 1:
        return None
    got, want = actual.detach().double(), expected.detach().double()
    if not bool(torch.isfinite(got).all()) or not bool(torch.isfinite(want).all()):
        return None
    rms = want.square().mean(dim=-1).sqrt().clamp_min(1e-12)
    return [float(v) for v in ((got - want).square().mean(dim=-1).sqrt() / rms)[0]]


def paired_cuda_timing(functions, *, warmup=20, repeats=100, rounds=7):
    """Median microseconds per call of each named function, arms alternated every round.

    ``stable`` is true when (max - min) / median over the rounds is at most 10 %.
    """
    if warmup < 1 or repeats < 1 or rounds < 3:
        raise ValueError("positive warmup/repeats and at least three rounds required")
    for fn in functions.values():
        for _ in range(warmup):
            fn()
    torch.cuda.synchronize()
    order = list(functions)
    samples = {name: [] for name in order}
    for index in range(rounds):
        for name in order if index % 2 == 0 else reversed(order):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            for _ in range(repeats):
                functions[name]()
            end.record()
            end.synchronize()
            samples[name].append(begin.elapsed_time(end) * 1000 / repeats)
    report = {}
    for name, values in samples.items():
        median = statistics.median(values)
        spread = (max(values) - min(values)) / median if median > 0 else float("inf")
        report[name] = {"microseconds_per_call": values, "median_us": median,
                        "relative_range": spread, "stable": spread <= 0.10}
    return report
