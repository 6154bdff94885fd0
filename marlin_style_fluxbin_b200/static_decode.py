"""Prepared static-cache Qwen3 decode with whole-sequence CUDA-graph capture.

Mirror of the reference's ``static_decode`` (``src/fluxbin_style/static_decode.py:15-138``).
The static KV cache grows through a fixed (teacher-forced) continuation; one graph holds every
decode step, embedding, attention, LM head and argmax included.  Prefill, restoring the prefix
KV, capture and audits stay outside the timed region.
"""
from __future__ import annotations

import time
from contextlib import contextmanager

import torch
from transformers import StaticCache

from .full_model_trial import packed_modules


@contextmanager
def prepared_linears(model, dtype):
    """Bind every packed Linear of ``model`` for serial decode; always unbind on exit."""
    modules = packed_modules(model)
    if any(m._decode_binding is not None for m in modules.values()):
        raise ValueError("prepared decode contexts cannot overlap")
    try:
        for m in modules.values():
            m.bind_prepared_decode(dtype)
        yield modules
    finally:
        for m in modules.values():
            m.clear_prepared_decode()


class StaticDecodeSession:
    def __init__(self, model, input_ids, forced_tokens):
        if input_ids.ndim != 2 or input_ids.shape[0] != 1 or input_ids.shape[1] < 2:
            raise ValueError("batch1 nonempty real prefix required")
        if forced_tokens.ndim != 2 or forced_tokens.shape[0] != 1 or forced_tokens.shape[1] < 1:
            raise ValueError("batch1 continuation required")
        if model.training:
            raise ValueError("eval model required")
        if any(m._decode_binding is not None for m in packed_modules(model).values()):
            raise ValueError("prepare real prefix before binding decode-only linears")
        if set(model.config.layer_types) != {"full_attention"}:
            raise ValueError("this protocol supports full-attention Qwen3 only")
        self.model, self.ids = model, input_ids
        self.tokens = forced_tokens.to(input_ids.device).contiguous()
        self.steps = self.tokens.shape[1]
        self.prefix_length = input_ids.shape[1]
        self.maximum_length = self.prefix_length + self.steps
        self.cache = StaticCache(config=model.config, max_cache_len=self.maximum_length)
        with torch.inference_mode():
            out = model(input_ids=input_ids, past_key_values=self.cache, use_cache=True, logits_to_keep=1)
            self.prefill_logits = out.logits[:, -1, :].detach().clone()
            self.prefix = [(layer.keys[:, :, :self.prefix_length].clone(), layer.values[:, :, :self.prefix_length].clone())
                           for layer in self.cache.layers]
        device = input_ids.device
        self.positions = torch.arange(self.prefix_length, self.maximum_length, device=device).view(1, -1)
        # Boolean SDPA masks (True = attend), one per step, built once: no dynamic mask
        # construction and no device-to-host read of a sequence length inside the loop.
        columns = torch.arange(self.maximum_length, device=device)
        self.masks = [(columns <= p).view(1, 1, 1, -1) for p in range(self.prefix_length, self.maximum_length)]
        self.graph = self.graph_outputs = self.capture_routes = None

    @torch.inference_mode()
    def reset(self):
        for layer, (k, v) in zip(self.cache.layers, self.prefix):
            layer.keys.zero_()
            layer.values.zero_()
            layer.keys[:, :, :self.prefix_length].copy_(k)
            layer.values[:, :, :self.prefix_length].copy_(v)
            if hasattr(layer, "cumulative_length"):
                if isinstance(layer.cumulative_length, torch.Tensor):
                    layer.cumulative_length.fill_(self.prefix_length)
                else:
                    layer.cumulative_length = self.prefix_length

    @torch.inference_mode()
    def run(self):
        outputs = []
        for i in range(self.steps):
            out = self.model(input_ids=self.tokens[:, i:i + 1], past_key_values=self.cache,
                             position_ids=self.positions[:, i:i + 1], cache_position=self.positions[0, i:i + 1],
                             attention_mask={"full_attention": self.masks[i]}, use_cache=True, logits_to_keep=1)
            logits = out.logits[:, -1, :]
            outputs.append((logits, logits.argmax(-1, keepdim=True)))
        return outputs

    def set_audit(self, enabled):
        for m in packed_modules(self.model).values():
            m._decode_audit = enabled
            m.route_counts = {"dense_fallback": 0, "packed_m1": 0}

    def routes(self):
        return {name: dict(m.route_counts) for name, m in packed_modules(self.model).items()}

    def trace(self, outputs):
        logits = torch.stack([self.prefill_logits] + [p[0] for p in outputs], dim=1).detach().cpu()
        predictions = torch.cat([self.prefill_logits.argmax(-1, keepdim=True)] + [p[1] for p in outputs], dim=1).cpu()
        if not bool(torch.isfinite(logits).all()):
            raise RuntimeError("nonfinite static decode logits")
        return dict(logits=logits, predictions=predictions, fed_tokens=self.tokens.cpu(),
                    cache_length=self.maximum_length, routes=self.routes())

    @torch.inference_mode()
    def audit(self):
        self.reset()
        self.set_audit(True)
        try:
            return self.trace(self.run())
        finally:
            self.set_audit(False)

    @torch.inference_mode()
    def capture(self):
        if self.ids.device.type != "cuda":
            raise RuntimeError("CUDA Graph requires NVIDIA CUDA")
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):
                self.reset()
                self.run()
        torch.cuda.current_stream().wait_stream(stream)
        self.reset()
        torch.cuda.synchronize()
        self.set_audit(True)
        graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(graph, stream=stream):
                outputs = self.run()
            self.capture_routes = self.routes()
        finally:
            self.set_audit(False)
        self.graph, self.graph_outputs = graph, outputs
        self.reset()
        graph.replay()
        torch.cuda.synchronize()
        return self.trace(outputs)

    @torch.inference_mode()
    def measure(self, mode):
        if mode not in ("prepared_eager", "sequence_graph"):
            raise ValueError("unknown mode")
        if mode == "sequence_graph" and self.graph is None:
            raise ValueError("capture first")
        self.reset()
        on_gpu = self.ids.device.type == "cuda"
        if on_gpu:
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
        wall = time.perf_counter()
        if on_gpu:
            begin.record()
        if mode == "sequence_graph":
            self.graph.replay()
            outputs = self.graph_outputs
        else:
            outputs = self.run()
        if on_gpu:
            end.record()
            end.synchronize()
        wall_ms = (time.perf_counter() - wall) * 1000
        return dict(wall_ms=wall_ms, device_ms=begin.elapsed_time(end) if on_gpu else None), self.trace(outputs)
