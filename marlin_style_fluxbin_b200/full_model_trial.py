"""HF cached-decode protocol shared by the decode runner and its tests.

Same functions and result keys as the reference's ``full_model_trial``
(``src/fluxbin_style/full_model_trial.py:10-93``): a dynamic-KV reference trace (prefill once, then
``steps`` single-token calls), the trace comparison (numerical gate, greedy tokens, fed tokens,
log-probability bound) and the route coverage check.  Organised here around two small tools, a
region clock (host wall time and, on a GPU, CUDA events) and a context manager that moves the
packed modules between their prefill policy (dense fallback allowed) and their decode policy
(packed path or error).
"""
from __future__ import annotations

import time
from contextlib import contextmanager

import torch

from .acceleration_checks import numerical_gate, stepwise_nrmse
from .deployment import PackedHybridLinear
from .w3_lut_deployment import PackedW3Linear

_PACKED_TYPES = (PackedHybridLinear, PackedW3Linear)


def packed_modules(model):
    """All packed Linear replacements of ``model`` by qualified name."""
    return {name: module for name, module in model.named_modules() if isinstance(module, _PACKED_TYPES)}


class RegionClock:
    """Times one region: host wall-clock milliseconds always, device milliseconds when ``device`` is a GPU."""

    def __init__(self, device: torch.device):
        self.gpu = device.type == "cuda"
        self.device = device
        self.wall_ms = None
        self._events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) if self.gpu else None

    def __enter__(self):
        if self.gpu:
            torch.cuda.synchronize(self.device)
        self._start = time.perf_counter()
        if self.gpu:
            self._events[0].record()
        return self

    def __exit__(self, *exc):
        if self.gpu:
            self._events[1].record()
            self._events[1].synchronize()
        self.wall_ms = (time.perf_counter() - self._start) * 1000
        return False

    @property
    def device_ms(self):
        return self._events[0].elapsed_time(self._events[1]) if self.gpu else None


@contextmanager
def _route_accounting(modules):
    """Fresh route counters, dense fallback for the prefill; ``decode_only()`` (the yielded function)
    switches every module to fail on anything but the packed path.  Policies are restored on exit."""
    before = {name: module.fallback for name, module in modules.items()}
    for module in modules.values():
        module.route_counts = {"packed_m1": 0, "dense_fallback": 0}
        module.fallback = "dense"

    def decode_only():
        for module in modules.values():
            module.fallback = "error"

    try:
        yield decode_only
    finally:
        for name, module in modules.items():
            module.fallback = before[name]


def _cache_length(cache) -> int:
    length = cache.get_seq_length()
    return int(length.item()) if isinstance(length, torch.Tensor) else int(length)


@torch.inference_mode()
def decode_trace(model, input_ids, *, steps, forced_tokens=None):
    """Prefill, then exactly ``steps`` M=1 calls on one growing dynamic KV cache.

    Returns ``steps+1`` next-token predictions (the first is the prefill's).  ``forced_tokens``
    ``[1,steps]`` fixes the fed tokens so that two models see identical contexts.  During the
    prefill packed modules use their dense fallback; during decode they must not.
    """
    if input_ids.ndim != 2 or input_ids.shape[0] != 1 or input_ids.shape[1] < 2 or steps < 1:
        raise ValueError("batch1, prompt length>=2 and positive decode steps required")
    if forced_tokens is not None and tuple(forced_tokens.shape) != (1, steps):
        raise ValueError("forced continuation shape must be [1,steps]")
    device = input_ids.device
    script = None if forced_tokens is None else forced_tokens.to(device)
    modules = packed_modules(model)
    logits, fed = [], []

    def advance(**call):
        """One model call; keeps the last-position logits and returns (cache, greedy token)."""
        output = model(use_cache=True, logits_to_keep=1, **call)
        logits.append(output.logits[:, -1, :].detach())
        return output.past_key_values, logits[-1].argmax(-1, keepdim=True)

    with _route_accounting(modules) as decode_only:
        with RegionClock(device) as prefill_clock:
            cache, token = advance(input_ids=input_ids)
        decode_only()
        step_clocks = []
        with RegionClock(device) as decode_clock:
            for index in range(steps):
                fed.append(token if script is None else script[:, index:index + 1])
                # per-step device time from a pair of events; the host does not wait between steps
                marks = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) if decode_clock.gpu else None
                if marks:
                    marks[0].record()
                cache, token = advance(input_ids=fed[-1], past_key_values=cache)
                if marks:
                    marks[1].record()
                    step_clocks.append(marks)
        length = _cache_length(cache)
        if length != input_ids.shape[1] + steps:
            raise RuntimeError("KV cache length drift")
        routes = {name: dict(module.route_counts) for name, module in modules.items()}
    return {
        "logits": torch.stack(logits, dim=1).cpu(),
        "predictions": torch.cat([row.argmax(-1, keepdim=True) for row in logits], dim=1).cpu(),
        "fed_tokens": torch.cat(fed, dim=1).cpu(),
        "cache_length": length,
        "prefill_wall_ms": prefill_clock.wall_ms,
        "decode_wall_ms": decode_clock.wall_ms,
        "prefill_device_ms": prefill_clock.device_ms,
        "decode_device_ms": decode_clock.device_ms,
        "step_device_ms": [first.elapsed_time(second) for first, second in step_clocks],
        "routes": routes,
    }


def compare_trace(candidate, reference, *, logprob_tolerance):
    """A candidate trace passes when its logits pass the numerical gate, its greedy tokens and fed
    tokens equal the reference's, and no log-probability moved by more than ``logprob_tolerance``."""
    if logprob_tolerance < 0:
        raise ValueError("negative logprob tolerance")
    ours, theirs = candidate["logits"], reference["logits"]
    if ours.shape != theirs.shape:
        return {"passed": False, "reason": "shape drift"}
    report = {
        "logits": numerical_gate(ours, theirs),
        "greedy_tokens_equal": torch.equal(candidate["predictions"], reference["predictions"]),
        "fed_tokens_equal": torch.equal(candidate["fed_tokens"], reference["fed_tokens"]),
        "logprob_tolerance": logprob_tolerance,
        "stepwise_normalized_rmse": stepwise_nrmse(ours, theirs),
    }
    moved = (ours.float().log_softmax(-1) - theirs.float().log_softmax(-1)).abs()
    report["max_abs_logprob_error"] = float(moved.max())
    within = bool(torch.isfinite(moved).all()) and report["max_abs_logprob_error"] <= logprob_tolerance
    report["passed"] = bool(report["logits"]["passed"] and report["greedy_tokens_equal"] and report["fed_tokens_equal"] and within)
    return report


def validate_routes(trace, *, expected_linears, steps):
    """Every packed Linear ran densely exactly once (the prefill) and packed exactly ``steps`` times."""
    wanted = {"dense_fallback": 1, "packed_m1": steps}
    routes = trace["routes"]
    return len(routes) == expected_linears and all(counts == wanted for counts in routes.values())
