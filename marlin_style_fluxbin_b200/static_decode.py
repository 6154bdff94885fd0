"""Prepared static-cache Qwen3 decode with whole-sequence CUDA-graph capture.

Same public surface as the reference's ``static_decode`` (``src/fluxbin_style/static_decode.py:15-138``:
``prepared_linears`` and ``StaticDecodeSession`` with ``reset / run / set_audit / routes / trace / audit /
capture / measure``).  The static KV cache grows through a fixed (teacher-forced) continuation; one
graph holds every decode step, embedding, attention, LM head and argmax included.  Prefill, restoring
the prefix KV, capture and audits stay outside the timed region.

The session is assembled from three parts: a snapshot of the prompt's KV rows that can be put back
into the static cache (``_PromptKV``), the per-step constant inputs (``_StepInputs``: token view,
position and boolean mask, all built once so that the loop neither builds masks nor reads a device
length on the host) and the region clock shared with the dynamic-cache trace.
"""
from __future__ import annotations

from contextlib import contextmanager

import torch
from transformers import StaticCache

from . import _native
from .full_model_trial import RegionClock, packed_modules

_MODES = ("prepared_eager", "sequence_graph")


@contextmanager
def prepared_linears(model, dtype):
    """Bind every packed Linear of ``model`` for serial decode; always unbind on exit."""
    modules = packed_modules(model)
    if any(module._decode_binding is not None for module in modules.values()):
        raise ValueError("prepared decode contexts cannot overlap")
    try:
        for module in modules.values():
            module.bind_prepared_decode(dtype)
        yield modules
    finally:
        for module in modules.values():
            module.clear_prepared_decode()


class _PromptKV:
    """The first ``length`` cache rows of every layer, copied out after the prefill."""

    def __init__(self, cache, length: int):
        self.cache, self.length = cache, length
        self.rows = [(layer.keys[:, :, :length].clone(), layer.values[:, :, :length].clone()) for layer in cache.layers]

    def restore(self):
        """Cache = prompt rows followed by zeros, bookkeeping set to the prompt length."""
        for layer, (keys, values) in zip(self.cache.layers, self.rows):
            for target, source in ((layer.keys, keys), (layer.values, values)):
                target.zero_()
                target[:, :, :self.length].copy_(source)
            counter = getattr(layer, "cumulative_length", None)  # absent, an int or a tensor, depending on the transformers version
            if isinstance(counter, torch.Tensor):
                counter.fill_(self.length)
            elif counter is not None:
                layer.cumulative_length = self.length


class _StepInputs:
    """What step ``i`` feeds the model besides the cache: token ``[1,1]``, position, and a mask over the whole cache."""

    def __init__(self, tokens: torch.Tensor, first_position: int):
        device, steps = tokens.device, tokens.shape[1]
        self.total = first_position + steps
        self.tokens = tokens
        self.positions = torch.arange(first_position, self.total, device=device).view(1, -1)
        slots = torch.arange(self.total, device=device)
        self.masks = [(slots <= position).view(1, 1, 1, -1) for position in range(first_position, self.total)]  # True = attend

    def __len__(self):
        return self.tokens.shape[1]

    def of(self, index: int) -> dict:
        at = slice(index, index + 1)
        return {"input_ids": self.tokens[:, at], "position_ids": self.positions[:, at], "cache_position": self.positions[0, at],
                "attention_mask": {"full_attention": self.masks[index]}}


class StaticDecodeSession:
    def __init__(self, model, input_ids, forced_tokens):
        for tensor, floor, message in ((input_ids, 2, "batch1 nonempty real prefix required"), (forced_tokens, 1, "batch1 continuation required")):
            if tensor.ndim != 2 or tensor.shape[0] != 1 or tensor.shape[1] < floor:
                raise ValueError(message)
        if model.training:
            raise ValueError("eval model required")
        if any(module._decode_binding is not None for module in packed_modules(model).values()):
            raise ValueError("prepare real prefix before binding decode-only linears")
        if set(model.config.layer_types) != {"full_attention"}:
            raise ValueError("this protocol supports full-attention Qwen3 only")
        self.model, self.ids = model, input_ids
        self.tokens = forced_tokens.to(input_ids.device).contiguous()
        self.steps, self.prefix_length = self.tokens.shape[1], input_ids.shape[1]
        self.maximum_length = self.prefix_length + self.steps
        self.inputs = _StepInputs(self.tokens, self.prefix_length)
        self.cache = StaticCache(config=model.config, max_cache_len=self.maximum_length)
        with torch.inference_mode():
            prefill = model(input_ids=input_ids, past_key_values=self.cache, use_cache=True, logits_to_keep=1)
            self.prefill_logits = prefill.logits[:, -1, :].detach().clone()
            self.prompt_kv = _PromptKV(self.cache, self.prefix_length)
        self.graph = self.graph_outputs = self.capture_routes = None

    # ---- the decode loop and its bookkeeping ----
    @torch.inference_mode()
    def reset(self):
        self.prompt_kv.restore()

    @torch.inference_mode()
    def run(self):
        """The whole continuation, eagerly; per step ``(logits [1,V], greedy token [1,1])``."""
        produced = []
        for index in range(len(self.inputs)):
            row = self.model(past_key_values=self.cache, use_cache=True, logits_to_keep=1, **self.inputs.of(index)).logits[:, -1, :]
            produced.append((row, row.argmax(-1, keepdim=True)))
        return produced

    def set_audit(self, enabled):
        for module in packed_modules(self.model).values():
            module._decode_audit = enabled
            module.route_counts = {"dense_fallback": 0, "packed_m1": 0}

    def routes(self):
        return {name: dict(module.route_counts) for name, module in packed_modules(self.model).items()}

    def trace(self, outputs):
        """Host-side record of a finished run, the prefill's prediction first."""
        rows = [self.prefill_logits] + [logits for logits, _ in outputs]
        choices = [self.prefill_logits.argmax(-1, keepdim=True)] + [choice for _, choice in outputs]
        logits = torch.stack(rows, dim=1).detach().cpu()
        if not bool(torch.isfinite(logits).all()):
            raise RuntimeError("nonfinite static decode logits")
        return {"logits": logits, "predictions": torch.cat(choices, dim=1).cpu(), "fed_tokens": self.tokens.cpu(),
                "cache_length": self.maximum_length, "routes": self.routes()}

    @contextmanager
    def _auditing(self):
        self.set_audit(True)
        try:
            yield
        finally:
            self.set_audit(False)

    @torch.inference_mode()
    def audit(self):
        """One eager run with route counting switched on."""
        self.reset()
        with self._auditing():
            return self.trace(self.run())

    # ---- graph capture and timing ----
    @torch.inference_mode()
    def capture(self):
        """Two eager warm-up runs on a side stream, then the whole continuation into one CUDA graph
        (route counters record what the capture pass launched); replays it once and returns its trace."""
        if self.ids.device.type != "cuda":
            raise RuntimeError("CUDA Graph requires NVIDIA CUDA")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.reset()
                self.run()
        torch.cuda.current_stream().wait_stream(side)
        self.reset()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with self._auditing():
            with torch.cuda.graph(graph, stream=side):
                outputs = self.run()
            self.capture_routes = self.routes()
        self.graph, self.graph_outputs = graph, outputs
        self.reset()
        graph.replay()
        _native.check_status(self.ids.device)  # synchronises; raises if a bounded device-side wait gave up
        return self.trace(outputs)

    @torch.inference_mode()
    def measure(self, mode):
        """``(timing, trace)`` of one run from the restored prompt: eager, or a replay of the captured graph."""
        if mode not in _MODES:
            raise ValueError("unknown mode")
        if mode == "sequence_graph" and self.graph is None:
            raise ValueError("capture first")
        self.reset()
        with RegionClock(self.ids.device) as clock:
            if mode == "sequence_graph":
                self.graph.replay()
                outputs = self.graph_outputs
            else:
                outputs = self.run()
        if clock.gpu:
            _native.check_status(self.ids.device)
        return {"wall_ms": clock.wall_ms, "device_ms": clock.device_ms}, self.trace(outputs)
