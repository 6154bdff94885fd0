"""Teacher-forced perplexity through the packed batch-1 route: every transition of every block
is scored by a ONE-token cached forward call, so the number the quality gate sees is produced by
exactly the kernels the decode benchmark times.

Counterpart of the scoring core of the reference's protocol
(``scripts/run_qwen3_8b_w3_packed_m1_ppl.py:167-312``: ``packed_route_smoke``, ``score_m1_ppl``,
``comparison``; the dataset, tokenizer and checkpoint handling of that script stay with the
caller, who passes token blocks).  A block is a list of token ids; the model sees token ``t`` with
the KV cache of tokens ``< t`` and is scored on token ``t + 1``; negative log-likelihoods are taken
on fp32 logits and summed in fp64 per block, the block totals with ``math.fsum``.
"""
from __future__ import annotations

import hashlib
import math
import time

import torch

from .full_model_trial import packed_modules
from .static_decode import prepared_linears

ROUTE_OF_ONE_CALL = {"packed_m1": 1, "dense_fallback": 0}


def _kv_length(cache) -> int:
    value = cache.get_seq_length()
    return int(value.item()) if isinstance(value, torch.Tensor) else int(value)


def _perplexity(mean_nll):
    """exp(mean_nll), or None when it is not a finite number."""
    if mean_nll is None or not math.isfinite(mean_nll):
        return None
    try:
        value = math.exp(mean_nll)
    except OverflowError:
        return None
    return value if math.isfinite(value) else None


@torch.inference_mode()
def packed_route_smoke(model, token: int, device, *, expected_packed_linears: int):
    """One single-token call with route counting on: every packed Linear must take its packed path
    exactly once and never its dense fallback.  None for a model without packed Linears."""
    modules = packed_modules(model)
    if not modules:
        return None
    for module in modules.values():
        module.route_counts = {"packed_m1": 0, "dense_fallback": 0}
        module._decode_audit = True
    try:
        model(input_ids=torch.tensor([[token]], dtype=torch.long, device=device), use_cache=True, logits_to_keep=1)
    finally:
        for module in modules.values():
            module._decode_audit = False
    if len(modules) != expected_packed_linears or any(dict(m.route_counts) != ROUTE_OF_ONE_CALL for m in modules.values()):
        raise RuntimeError("packed M=1 route smoke failed")
    return {"passed": True, "linear_count": len(modules), "calls_per_linear": 1}


def _score_block(model, tokens: torch.Tensor):
    """fp32 NLL of tokens[1:] given the growing prefix, one cached single-token call per transition."""
    nll = torch.empty(tokens.numel() - 1, dtype=torch.float32, device=tokens.device)
    cache = None
    for position in range(tokens.numel() - 1):
        output = model(input_ids=tokens[position:position + 1].view(1, 1), past_key_values=cache, use_cache=True, logits_to_keep=1)
        cache = output.past_key_values
        logits = output.logits[0, -1].float()
        nll[position] = torch.logsumexp(logits, dim=0) - logits[tokens[position + 1]]
    if _kv_length(cache) != tokens.numel() - 1:
        raise RuntimeError("KV cache length drifted during M=1 PPL")
    return nll, str(output.logits.dtype)


@torch.inference_mode()
def score_m1_ppl(model, blocks, *, arm: str, device, expected_packed_linears: int, progress_every: int = 5) -> dict:
    """Perplexity of ``blocks`` (lists of token ids, at least two each) under teacher forcing, one token
    per model call, packed Linears bound for decode and forbidden from falling back to dense."""
    if model.training:
        raise ValueError("PPL model must be in eval mode")
    device = torch.device(device)
    on_gpu = device.type == "cuda"
    if on_gpu:
        torch.cuda.reset_peak_memory_stats(device)
        torch.cuda.synchronize(device)
    began = time.monotonic()
    totals, digests, failed_blocks, transitions, logits_dtype = [], [], [], 0, None
    with prepared_linears(model, torch.bfloat16) as modules:
        if len(modules) != expected_packed_linears:
            raise RuntimeError(f"packed Linear count drifted for {arm}: {len(modules)} != {expected_packed_linears}")
        smoke = packed_route_smoke(model, blocks[0][0], device, expected_packed_linears=expected_packed_linears)
        for index, block in enumerate(blocks):
            if len(block) < 2:
                raise ValueError("PPL block must contain at least two tokens")
            nll, logits_dtype = _score_block(model, torch.tensor(block, dtype=torch.long, device=device))
            total = float(nll.double().sum())
            if not math.isfinite(total):
                failed_blocks.append(index)
                break
            totals.append(total)
            digests.append(hashlib.sha256(nll.cpu().numpy().tobytes()).hexdigest())
            transitions += len(block) - 1
            if progress_every and ((index + 1) % progress_every == 0 or index + 1 == len(blocks)):
                print(f"FLUXBIN_{arm.upper()}_M1_PPL_PROGRESS={index + 1}/{len(blocks)}", flush=True)
    if on_gpu:
        torch.cuda.synchronize(device)
    total_nll = None if failed_blocks else math.fsum(totals)
    mean_nll = None if total_nll is None else total_nll / transitions
    perplexity = _perplexity(mean_nll)
    valid = perplexity is not None and not failed_blocks
    return {
        "arm": arm, "status": "completed" if valid else "invalid", "execution": "teacher_forced_cached_decode_m1",
        "tokens_per_model_call": 1, "block_count": len(totals), "scored_transition_count": transitions,
        "total_nll": total_nll, "mean_nll": mean_nll, "perplexity": perplexity, "metrics_valid": valid,
        "nonfinite_block_indices": failed_blocks, "block_nll_sha256": digests,
        "logits_dtype": logits_dtype, "nll_logits_dtype": "torch.float32",
        "elapsed_seconds": time.monotonic() - began,
        "peak_allocated_bytes": torch.cuda.max_memory_allocated(device) if on_gpu else None,
        "packed_route_smoke": smoke, "packed_linear_count": len(packed_modules(model)),
        "dense_fallback_permitted_during_scoring": False,
    }


def comparison(candidate: dict, baseline: dict) -> dict:
    """How far a candidate arm's perplexity is from a baseline arm's."""
    return {
        "candidate": candidate["arm"], "baseline": baseline["arm"],
        "ppl_delta": candidate["perplexity"] - baseline["perplexity"],
        "ppl_relative_percent": (candidate["perplexity"] / baseline["perplexity"] - 1.0) * 100.0,
        "mean_nll_delta": candidate["mean_nll"] - baseline["mean_nll"],
    }
