"""HF cached-decode protocol shared by the decode runner and its tests.

Mirror of the reference's ``full_model_trial`` (``src/fluxbin_style/full_model_trial.py:10-93``):
a dynamic-KV reference trace (prefill once, then ``steps`` single-token calls), the trace
comparison (numerical gate, greedy tokens, fed tokens, log-probability bound) and the route
coverage check.
"""
from __future__ import annotations

import time

import torch

from .acceleration_checks import numerical_gate, stepwise_nrmse
from .deployment import PackedHybridLinear
from .w3_lut_deployment import PackedW3Linear


def packed_modules(model):
    """All packed Linear replacements of ``model`` by qualified name."""
    return {name: m for name, m in model.named_modules() if isinstance(m, (PackedHybridLinear, PackedW3Linear))}


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
    forced = None if forced_tokens is None else forced_tokens.to(input_ids.device)
    modules = packed_modules(model)
    saved_fallback = {name: m.fallback for name, m in modules.items()}
    for m in modules.values():
        m.route_counts = {"packed_m1": 0, "dense_fallback": 0}
        m.fallback = "dense"
    on_gpu = input_ids.is_cuda

    def sync():
        if on_gpu:
            torch.cuda.synchronize(input_ids.device)

    def event():
        return torch.cuda.Event(enable_timing=True) if on_gpu else None

    logits, predictions, fed, step_events = [], [], [], []
    try:
        sync()
        wall = time.perf_counter()
        pre_begin, pre_end = event(), event()
        if on_gpu:
            pre_begin.record()
        output = model(input_ids=input_ids, use_cache=True, logits_to_keep=1)
        cache = output.past_key_values
        logits.append(output.logits[:, -1, :].detach())
        current = logits[-1].argmax(-1, keepdim=True)
        predictions.append(current)
        if on_gpu:
            pre_end.record()
        sync()
        prefill_wall = (time.perf_counter() - wall) * 1000
        for m in modules.values():
            m.fallback = "error"
        dec_begin, dec_end = event(), event()
        wall = time.perf_counter()
        if on_gpu:
            dec_begin.record()
        for i in range(steps):
            token = current if forced is None else forced[:, i:i + 1]
            fed.append(token)
            begin, end = event(), event()
            if on_gpu:
                begin.record()
            output = model(input_ids=token, past_key_values=cache, use_cache=True, logits_to_keep=1)
            cache = output.past_key_values
            logits.append(output.logits[:, -1, :].detach())
            current = logits[-1].argmax(-1, keepdim=True)
            predictions.append(current)
            if on_gpu:
                end.record()
                step_events.append((begin, end))
        if on_gpu:
            dec_end.record()
        sync()
        decode_wall = (time.perf_counter() - wall) * 1000
        length = cache.get_seq_length()
        length = int(length.item()) if isinstance(length, torch.Tensor) else int(length)
        if length != input_ids.shape[1] + steps:
            raise RuntimeError("KV cache length drift")
        return {
            "logits": torch.stack(logits, dim=1).cpu(),
            "predictions": torch.cat(predictions, dim=1).cpu(),
            "fed_tokens": torch.cat(fed, dim=1).cpu(),
            "cache_length": length,
            "prefill_wall_ms": prefill_wall,
            "decode_wall_ms": decode_wall,
            "prefill_device_ms": pre_begin.elapsed_time(pre_end) if on_gpu else None,
            "decode_device_ms": dec_begin.elapsed_time(dec_end) if on_gpu else None,
            "step_device_ms": [a.elapsed_time(b) for a, b in step_events],
            "routes": {name: dict(m.route_counts) for name, m in modules.items()},
        }
    finally:
        for name, m in modules.items():
            m.fallback = saved_fallback[name]


def compare_trace(candidate, reference, *, logprob_tolerance):
    if logprob_tolerance < 0:
        raise ValueError("negative logprob tolerance")
    gate = numerical_gate(candidate["logits"], reference["logits"])
    if candidate["logits"].shape != reference["logits"].shape:
        return {"passed": False, "reason": "shape drift"}
    tokens_equal = torch.equal(candidate["predictions"], reference["predictions"])
    contexts_equal = torch.equal(candidate["fed_tokens"], reference["fed_tokens"])
    delta = (candidate["logits"].float().log_softmax(-1) - reference["logits"].float().log_softmax(-1)).abs()
    worst, finite = float(delta.max()), bool(torch.isfinite(delta).all())
    return {
        "passed": gate["passed"] and tokens_equal and contexts_equal and finite and worst <= logprob_tolerance,
        "logits": gate, "greedy_tokens_equal": tokens_equal, "fed_tokens_equal": contexts_equal,
        "max_abs_logprob_error": worst, "logprob_tolerance": logprob_tolerance,
        "stepwise_normalized_rmse": stepwise_nrmse(candidate["logits"], reference["logits"]),
    }


def validate_routes(trace, *, expected_linears, steps):
    return len(trace["routes"]) == expected_linears and all(
        r == {"dense_fallback": 1, "packed_m1": steps} for r in trace["routes"].values())
