"""Benchmark of the batch-1 packed-Linear decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[1]): all seven Qwen3-8B Linear shapes as W3 group-128
GEMVs at M=1, for 36 layers of DISTINCT synthetic weights (2.8 GB, far larger than L2, so
every weight byte comes from HBM), value distributions as configs[0] states (uniform codes,
fp16 scales U(0.005,0.02), zero points in {3,4}, x ~ N(0,1) bf16).  One step = one pass over
all 252 GEMVs = the Linear work of one decoded token, replayed from a CUDA graph.

Metric: HBM GB/s on the algorithmic bytes (stored planes + scales + zero points + x + y).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = (  # name, out_features, in_features (Qwen3-8B)
    ("q_proj", 4096, 4096), ("k_proj", 1024, 4096), ("v_proj", 1024, 4096), ("o_proj", 4096, 4096),
    ("gate_proj", 12288, 4096), ("up_proj", 12288, 4096), ("down_proj", 4096, 12288),
)
LAYERS = 36
NOMINAL_HBM_GBS = 8000.0
DRAM_TRAFFIC_RATIO = 20.203 / 20.087
METRIC = "W3 GEMV HBM GB/s (% of 8 TB/s) per Qwen3-8B shape; batch-1 decode tokens/s"


def gemv_bytes(o: int, k: int, zeros: bool = True) -> int:
    """Algorithmic bytes of one M=1 GEMV: planes, fp16 scales, uint8 zero points, x and y."""
    g = k // 128
    return 3 * o * k // 8 + 2 * g * o + (g * o if zeros else 0) + 2 * k + 2 * o


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()

    def summary(self):
        good = [r for r in self.rows if len(r) == 6 and r[0].isdigit()]
        if not good:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        mhz = sorted(int(r[0]) for r in good)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in good)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(good[0][1]), "reasons": reasons, "samples": len(good)}


def synthetic_layout(torch, o, k, device, gen):
    g = k // 128
    return {
        "planes": torch.randint(0, 256, (g, 3, o, 16), dtype=torch.uint8, device=device, generator=gen),
        "scales": (torch.rand(g, o, device=device, generator=gen) * 0.015 + 0.005).half(),
        "zeros": torch.randint(3, 5, (g, o), dtype=torch.uint8, device=device, generator=gen),
        "perm": torch.arange(k, dtype=torch.int16, device=device),
    }


def run_ours(args, rank, world, local_rank):
    import torch

    from marlin_style_fluxbin_b200.w3_lut_deployment import PackedW3Linear

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    gen = torch.Generator(device=device).manual_seed(20260916 + rank)
    with torch.inference_mode():
        modules = []  # LAYERS x 7 bound modules, distinct weights
        for _ in range(LAYERS):
            for name, o, k in SHAPES:
                module = PackedW3Linear(synthetic_layout(torch, o, k, device, gen), row_tile=1024 if max(o, k) > 4096 else 256)
                module.bind_prepared_decode(torch.bfloat16)
                modules.append((name, module))
        x_dev = {k: torch.randn(1, 1, k, device=device, generator=gen).bfloat16() for k in (4096, 12288)}
        x_host = {k: v.cpu().pin_memory() for k, v in x_dev.items()}
        last = [m for _, m in modules[-len(SHAPES):]]
        out_host = [torch.empty(1, 1, m.out_features, dtype=torch.bfloat16).pin_memory() for m in last]

        def one_pass():
            for _, module in modules:
                module(x_dev[module.in_features])

        stream = torch.cuda.Stream(device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):
                one_pass()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                one_pass()

            def e2e_step():
                for k in x_dev:
                    x_dev[k].copy_(x_host[k], non_blocking=True)
                graph.replay()
                for host, module in zip(out_host, last):
                    host.copy_(module._decode_output.view(1, 1, -1), non_blocking=True)
                stream.synchronize()

            def barrier():
                stream.synchronize()
                if world > 1:
                    torch.distributed.barrier()
                stream.synchronize()

            for _ in range(max(args.warmup, 3)):
                graph.replay()
            barrier()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with ClockSampler(local_rank) as clocks:
                begin.record(stream)
                for _ in range(args.steps):
                    graph.replay()
                end.record(stream)
                barrier()
                # the K timed steps last tens of milliseconds: keep the same graph running for
                # about a second under the sampler, so that the clock record holds samples taken
                # under this very load (reported beside the number, not instead of it)
                # (not in the --headline-only form, which profiling commands run)
                held = 1 if args.headline_only else max(1, int(1000.0 / max(begin.elapsed_time(end) / args.steps, 1e-3)))
                hold_begin, hold_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                hold_begin.record(stream)
                for _ in range(held):
                    graph.replay()
                hold_end.record(stream)
                barrier()
            step_ms = begin.elapsed_time(end) / args.steps
            held_ms = hold_begin.elapsed_time(hold_end) / held

            # per-shape: the same protocol on 36 distinct weights of one shape
            per_shape = {}
            for name, o, k in SHAPES:
                if args.headline_only or name in ("v_proj", "up_proj", "o_proj"):
                    continue
                mods = [m for n, m in modules if n == name]
                shape_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(shape_graph, stream=stream):
                    for m in mods:
                        m(x_dev[k])
                for _ in range(3):
                    shape_graph.replay()
                stream.synchronize()
                begin.record(stream)
                for _ in range(20):
                    shape_graph.replay()
                end.record(stream)
                stream.synchronize()
                us = begin.elapsed_time(end) * 1000 / (20 * len(mods))
                gbs = gemv_bytes(o, k) / us / 1e3
                per_shape[f"{o}x{k}"] = {"us": round(us, 3), "gbs": round(gbs, 1), "bytes": gemv_bytes(o, k),
                                         "bytes_zeros_as_fp16": gemv_bytes(o, k) + (k // 128) * o}

            # the same seven Linears as the decode engine launches them: q/k/v and gate/up share a
            # launch, so a layer is four launches; and the M sweep of configs[1] on two shapes
            extras = world == 1 and not args.headline_only
            fused = fused_layer_pass(torch, modules, x_dev, stream, begin, end) if extras else None
            sweep = m_sweep(torch, modules, device, stream, begin, end) if extras else None

            for _ in range(3):
                e2e_step()
            barrier()
            t0 = time.perf_counter()
            begin.record(stream)
            for _ in range(args.steps):
                e2e_step()
            end.record(stream)
            barrier()
            e2e_ms = max(begin.elapsed_time(end), (time.perf_counter() - t0) * 1e3) / args.steps

    if world > 1:
        t = torch.tensor([step_ms, e2e_ms], device=device, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        step_ms, e2e_ms = float(t[0]), float(t[1])
    step_bytes = LAYERS * sum(gemv_bytes(o, k) for _, o, k in SHAPES)
    return {
        "step_ms": step_ms, "e2e_ms": e2e_ms, "step_bytes": step_bytes, "per_shape": per_shape, "fused": fused, "m_sweep": sweep,
        "clocks": dict(clocks.summary(), sampled_over_steps=args.steps + held, ms_per_step_while_sampled=round(held_ms, 4)),
        "launches": len(modules) * args.steps,
        "h2d": sum(v.numel() * 2 for v in x_host.values()), "d2h": sum(v.numel() * 2 for v in out_host),
    }


def _graph_time(torch, fn, stream, begin, end, launches, repeats=20):
    graph = torch.cuda.CUDAGraph()
    fn()
    stream.synchronize()
    with torch.cuda.graph(graph, stream=stream):
        fn()
    for _ in range(3):
        graph.replay()
    stream.synchronize()
    begin.record(stream)
    for _ in range(repeats):
        graph.replay()
    end.record(stream)
    stream.synchronize()
    return begin.elapsed_time(end) * 1000 / (repeats * launches)


def fused_layer_pass(torch, modules, x_dev, stream, begin, end):
    """Four launches per layer (q/k/v, o, gate/up, down) over the weights of the headline step."""
    from marlin_style_fluxbin_b200 import _native

    by_layer = [dict(modules[i:i + len(SHAPES)]) for i in range(0, len(modules), len(SHAPES))]
    scratch = torch.zeros(_native.w3_scratch_bytes(1, 2 * 12288, 4096) + (1 << 20), dtype=torch.uint8, device=x_dev[4096].device)
    plan = []
    for layer in by_layer:
        for names in (("q_proj", "k_proj", "v_proj"), ("o_proj",), ("gate_proj", "up_proj"), ("down_proj",)):
            mods = [layer[n] for n in names]
            outs = [torch.empty(1, m.out_features, device=scratch.device, dtype=torch.bfloat16) for m in mods]
            entries = [(m.planes, m.scales, getattr(m, "zeros", None), o, None) for m, o in zip(mods, outs)]
            plan.append((_native.w3_matrix_list(entries), len(mods), sum(m.out_features for m in mods), mods[0].in_features, entries))

    def run():
        for array, n, total, k, _ in plan:
            _native.w3_gemv_multi(x_dev[k].view(1, k), array, n, total, torch.float16, None, scratch=scratch)

    us = _graph_time(torch, run, stream, begin, end, len(by_layer))
    layer_bytes = sum(gemv_bytes(o, k) for _, o, k in SHAPES)
    return {"launches_per_layer": 4, "us_per_layer": round(us, 2), "gbs": round(layer_bytes / us / 1e3, 1)}


def m_sweep(torch, modules, device, stream, begin, end):
    """M in {1,2,4,8,16} on q_proj and gate_proj: table-lookup kernel (M <= 4), tensor-core kernel, cuBLAS bf16."""
    from marlin_style_fluxbin_b200 import _native
    from marlin_style_fluxbin_b200.gptq_deployment import restore_planar_w3

    out = {}
    scratch = {kind: torch.zeros(8 << 20, dtype=torch.uint8, device=device) for kind in ("lut", "mma")}
    for name in ("q_proj", "gate_proj"):
        mods = [m for n, m in modules if n == name][:12]
        o, k = mods[0].out_features, mods[0].in_features
        dense = [restore_planar_w3(m.layout(), dtype=torch.bfloat16) for m in mods[:4]]
        for rows in (1, 2, 4, 8, 16):
            x = torch.randn(rows, k, device=device).bfloat16()
            y = torch.empty(rows, o, device=device, dtype=torch.bfloat16)
            entry = {}
            if rows <= 4:
                entry["lut_us"] = round(_graph_time(torch, lambda: [_native.w3_gemv(x, m.planes, m.scales, getattr(m, "zeros", None), None, y, scratch=scratch["lut"]) for m in mods], stream, begin, end, len(mods)), 2)
            entry["mma_us"] = round(_graph_time(torch, lambda: [_native.w3_gemm_small(x, m.planes, m.scales, getattr(m, "zeros", None), None, y, scratch=scratch["mma"]) for m in mods], stream, begin, end, len(mods)), 2)
            entry["cublas_bf16_us"] = round(_graph_time(torch, lambda: [torch.mm(x, w.t(), out=y) for w in dense], stream, begin, end, len(dense)), 2)
            best = min(v for key, v in entry.items() if key != "cublas_bf16_us")
            entry["packed_gbs"] = round(gemv_bytes(o, k) / best / 1e3, 1)
            out[f"{o}x{k} M={rows}"] = entry
        del dense
    return out


def bb_bytes(o: int, k: int, n_salient: int = 32) -> int:
    """Algorithmic bytes of one two-base GEMV with matrix-wide scales (BASELINE.json configs[2])."""
    return 2 * o * k // 8 + 4 * o + 4 * k + 2 * n_salient * o + 4 * n_salient + 2 * k + 2 * o


def run_binary_basis(torch, device):
    """configs[2]: the two-base binary-basis GEMV (1 bit per weight and base, fp16 row / column scales,
    32 dense bf16 salient columns) on the seven shapes, 12 distinct weight sets per shape."""
    from marlin_style_fluxbin_b200 import _native
    from marlin_style_fluxbin_b200.binary_global import global_two_base_m1_out

    gen = torch.Generator(device=device).manual_seed(20260917)
    stream = torch.cuda.Stream(device)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    table, total_us, total_bytes = {}, 0.0, 0
    with torch.inference_mode(), torch.cuda.stream(stream):
        for name, o, k in SHAPES:
            key = f"{o}x{k}"
            if key in table:
                total_us += table[key]["us"]
                total_bytes += table[key]["bytes"]
                continue
            layouts = []
            for _ in range(12):
                layouts.append({
                    "codes": torch.randint(0, 256, (k // 128, o, 2, 16), device=device, generator=gen, dtype=torch.uint8),
                    "row_scales": (torch.randn(2, o, device=device, generator=gen) * 0.02).abs().half(),
                    "column_scales": (torch.randn(2, k, device=device, generator=gen) * 0.02).abs().half(),
                    "salient_indices": torch.randperm(k, device=device, generator=gen)[:32].sort().values.int(),
                    "salient_values": (torch.randn(o, 32, device=device, generator=gen) * 0.05).bfloat16(),
                })
            x = torch.randn(1, k, device=device, generator=gen).bfloat16()
            y = torch.empty(1, o, device=device, dtype=torch.bfloat16)
            scratch = torch.zeros(_native.bb_scratch_bytes(o, k, True), dtype=torch.uint8, device=device)

            def run():
                for layout in layouts:
                    _native.bb_global_gemv(x, layout["codes"], layout["row_scales"], layout["column_scales"],
                                           layout["salient_indices"], layout["salient_values"], y, scratch=scratch)

            global_two_base_m1_out(x, layouts[0], y)  # the public call, once, validates the layout
            us = _graph_time(torch, run, stream, begin, end, len(layouts))
            table[key] = {"us": round(us, 3), "bytes": bb_bytes(o, k), "gbs": round(bb_bytes(o, k) / us / 1e3, 1)}
            total_us += us
            total_bytes += bb_bytes(o, k)
            del layouts
    return table, total_us, total_bytes


def run_decode(torch, shape_name, prompt, steps, rank, world, local_rank, arms=("bf16", "w3"), repeats=5, tp_push=None):
    """Full-model batch-1 decode (BASELINE.json configs[3] / [4]): random-init Qwen3 shape, all Linears
    W3 g128, LM head bf16; prefill `prompt` random ids, then `steps` tokens from ONE CUDA graph.  The
    BF16 arm runs the same engine with dense dequantised weights through cuBLAS.  Tensor parallel
    over `world` ranks when world > 1."""
    from marlin_style_fluxbin_b200.decode_engine import QWEN3_8B, QWEN3_32B, DecodeEngine

    shape = {"qwen3-8b": QWEN3_8B, "qwen3-32b": QWEN3_32B}[shape_name]
    device = torch.device("cuda", local_rank)
    ids = torch.randint(0, shape.vocab, (1, prompt), generator=torch.Generator().manual_seed(1))
    out, forced, reference = {}, None, None
    for arm in arms:
        engine = DecodeEngine(shape, device=device, max_positions=prompt + steps + 8, arm=arm,
                              tp_rank=rank, tp_size=world, tp_push=tp_push)
        first = engine.prefill(ids).argmax(-1)
        fed, greedy, logits = engine.decode(first, prompt, steps, forced=forced)
        engine.prefill(ids)
        graph, predictions, _ = engine.capture(first, prompt, steps, forced=forced)
        engine.prefill(ids)
        graph.replay()
        torch.cuda.synchronize(device)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        times = []
        for _ in range(repeats):
            if world > 1:
                torch.distributed.barrier()
            begin.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize(device)
            times.append(begin.elapsed_time(end))
        ms = sorted(times)[len(times) // 2]
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t[0])
        entry = {"tokens_per_s": round(steps / ms * 1e3, 1), "ms_per_token": round(ms / steps, 4),
                 "launches_per_token": engine.launches_per_step, "graph_equals_eager": bool(torch.equal(predictions, greedy))}
        if forced is None:
            forced, reference = fed, (greedy, logits)
        else:
            a, b = logits.double(), reference[1].double()
            entry["greedy_agreement_forced"] = round(float((greedy == reference[0]).float().mean()), 4)
            entry["logits_nrmse_vs_bf16_arm"] = round(float((a - b).square().mean().sqrt() / b.square().mean().sqrt()), 5)
            # a disagreement is a near-tie when the bf16 arm's margin between its own choice and the
            # packed arm's choice is within four times the rms difference of the two arms' logits
            rms = float((a - b).square().mean().sqrt())
            differ = (greedy != reference[0]).nonzero().flatten().tolist()
            margins = [float(b[i, reference[0][i]] - b[i, greedy[i]]) for i in differ]
            entry["disagreements"] = len(differ)
            entry["disagreements_outside_near_ties"] = sum(1 for v in margins if v > 4 * rms)
        if arm == "w3":
            tp_forced, tp_greedy, tp_logits = fed, greedy, logits
        out[arm] = entry
        del engine, graph
        torch.cuda.empty_cache()
    if world > 1 and "w3" in out:
        # the sharded engine against an unsharded engine with the same weights, on rank 0:
        # the allreduce changes the summation order, nothing else
        if rank == 0:
            single = DecodeEngine(shape, device=device, max_positions=prompt + steps + 8, arm="w3", tp_rank=0, tp_size=1)
            first_single = single.prefill(ids).argmax(-1)
            _, greedy_single, logits_single = single.decode(first_single, prompt, min(steps, 8), forced=tp_forced[:min(steps, 8)])
            a, b = tp_logits[:min(steps, 8)].double(), logits_single.double()
            out["w3"]["tp_vs_single_logits_nrmse"] = round(float((a - b).square().mean().sqrt() / b.square().mean().sqrt()), 5)
            out["w3"]["tp_vs_single_greedy_agreement"] = round(float((tp_greedy[:min(steps, 8)] == greedy_single).float().mean()), 4)
            del single
            torch.cuda.empty_cache()
        torch.distributed.barrier()
    if "w3" in out and "bf16" in out:
        out["w3_over_bf16"] = round(out["w3"]["tokens_per_s"] / out["bf16"]["tokens_per_s"], 3)
    exchange = "none" if world == 1 else ("nccl allreduce" if tp_push is False else "pushed from the GEMV epilogue into peer buffers (packed arm)")
    out["config"] = {"model": shape_name, "prompt_tokens": prompt, "decode_tokens": steps, "tensor_parallel": world, "exchange": exchange,
                     "graph": "whole continuation, teacher-forced from the bf16 arm's greedy tokens"}
    return out


def cpu_reference(steps: int, warmup: int):
    """The reference's CPU path (dequantise, then fp32 matmul) restated in the oracle, timed
    on the host cores over ONE layer's seven Linears per step (a bounded sample)."""
    import numpy as np

    from oracle import oracle as orc

    # all the host cores this process may use (torchrun exports OMP_NUM_THREADS=1 to its ranks)
    orc.set_num_threads(len(os.sched_getaffinity(0)))
    rng = np.random.default_rng(20260916)
    layer = []
    t_dequant = 0.0
    for _, o, k in SHAPES:
        g = k // 128
        planes = rng.integers(0, 256, (g, 3, o, 16), dtype=np.uint8)
        scales = (rng.random((g, o), dtype=np.float32) * 0.015 + 0.005).astype(np.float16).view(np.uint16)
        zeros = rng.integers(3, 5, (g, o), dtype=np.uint8)
        t0 = time.perf_counter()
        dense = orc.w3_dequant(planes, scales, orc.F16, zeros, None, orc.F32)
        t_dequant += time.perf_counter() - t0
        layer.append((dense, rng.standard_normal((1, k), dtype=np.float32)))
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        for dense, x in layer:
            orc.dense_gemv_f32(dense, x)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    step_s = sum(times) / len(times)
    nbytes = sum(gemv_bytes(o, k) for _, o, k in SHAPES)
    return {"value": nbytes / step_s / 1e9, "cores": orc.num_threads(), "step_ms": step_s * 1e3,
            "dequant_s_per_layer": t_dequant,
            "sample": (f"one layer (7 Linears, {nbytes} packed bytes) per step: fp32 matmul on weights dequantised once "
                       f"outside the timer ({t_dequant:.2f} s per layer when redone every call)")}


def small_case(args):
    """A few launches of one shape on distinct weights (larger than L2 together): the
    small, self-ending program that profiler captures are taken on."""
    import torch

    from marlin_style_fluxbin_b200.w3_lut_deployment import w3_lut_gemv_out, w3_lut_m1_out, workspace_shape

    o, k = (int(v) for v in args.case.lower().split("x"))
    device = torch.device("cuda", 0)
    gen = torch.Generator(device=device).manual_seed(1)
    layouts = [synthetic_layout(torch, o, k, device, gen) for _ in range(args.copies)]
    x = torch.randn(args.rows, k, device=device, generator=gen).bfloat16()
    out = torch.empty(args.rows, o, device=device, dtype=torch.bfloat16)
    workspace = torch.empty(workspace_shape(o, k), device=device)
    for _ in range(2):
        for layout in layouts:
            if args.rows == 1:
                w3_lut_m1_out(x, layout, out, workspace, row_tile=256)
            else:  # the tensor-core small-batch kernel
                w3_lut_gemv_out(x, layout, out, kernel="mma")
    torch.cuda.synchronize()
    print(json.dumps({"case": args.case, "rows": args.rows, "copies": args.copies, "launches": 2 * args.copies,
                      "bytes_per_launch": gemv_bytes(o, k), "checksum": float(out.float().abs().sum())}))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--workload", default="gemv", choices=("gemv", "decode-8b", "tp-decode-32b", "binary-basis"),
                        help="gemv (default): the seven Linear shapes plus the 8B decode; tp-decode-32b: tensor-parallel decode over --gpus ranks")
    parser.add_argument("--case", default=None, metavar="OxK",
                        help="profiling helper: launch the GEMV of one shape on --copies distinct weights and exit")
    parser.add_argument("--prompt-tokens", type=int, default=512, help="decode-8b: prompt length")
    parser.add_argument("--decode-tokens", type=int, default=32, help="decode-8b: tokens decoded in the graph")
    parser.add_argument("--packed-arm-only", action="store_true", help="decode-8b: skip the BF16 arm (for profiler launch lists)")
    parser.add_argument("--tp-exchange", default="push", choices=("push", "nccl"),
                        help="tp-decode-32b: exchange after the row-split GEMVs (fused push, or NCCL allreduce)")
    parser.add_argument("--copies", type=int, default=8)
    parser.add_argument("--rows", type=int, default=1, help="with --case: activation rows (above 1 runs the tensor-core kernel)")
    parser.add_argument("--headline-only", action="store_true",
                        help="time only the headline step (no per-shape table, sweeps, decode or CPU leg): for profiler launch lists")
    args = parser.parse_args()
    if args.case:
        return small_case(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {
        "workload": "qwen3-8b all seven Linear shapes, W3 g128 GEMV, M=1, 36 layers of distinct weights (configs[1])",
        "shapes": [f"{o}x{k}" for _, o, k in SHAPES], "layers": LAYERS, "gemvs_per_step": LAYERS * len(SHAPES),
        "cache": "inputs larger than L2 (2.8 GB of weights per pass), no flush needed",
        "zero_points": "uint8 per (group,row), counted at their stored size", "parallelism": f"replicas x{world}",
    }

    if args.impl == "reference":
        if rank != 0:
            return
        ref = cpu_reference(args.steps, min(args.warmup, 1))
        line = {
            "impl": "reference", "metric": METRIC, "value": round(ref["value"], 3), "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ref["step_ms"], 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "cpu_baseline": {"value": round(ref["value"], 3), "unit": "GB/s", "cores": ref["cores"], "kind": "port", "sample": ref["sample"]},
            "e2e": {"value": round(ref["value"], 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
        print(json.dumps(line))
        return

    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the packed kernels have no CPU path")
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if args.workload == "tp-decode-32b":
        torch.cuda.set_device(local_rank)
        decode = run_decode(torch, "qwen3-32b", 1024, 64, rank, world, local_rank, arms=("w3",) if world > 1 else ("bf16", "w3"),
                            tp_push=False if args.tp_exchange == "nccl" else None)
        if rank == 0:
            print(json.dumps({"metric": "batch-1 decode tokens/s, Qwen3-32B-shaped W3 g128, tensor parallel", "unit": "tokens/s",
                              "value": decode["w3"]["tokens_per_s"], "n_gpus": world, "higher_is_better": True, "scaling": "strong",
                              "data": "synthetic", "dtype": "f32", "decode": decode}))
        if world > 1:
            torch.distributed.barrier()
            torch.distributed.destroy_process_group()
        return
    if args.workload == "decode-8b":
        torch.cuda.set_device(local_rank)
        decode = run_decode(torch, "qwen3-8b", args.prompt_tokens, args.decode_tokens, 0, 1, local_rank,
                            arms=("w3",) if args.packed_arm_only else ("bf16", "w3"))
        if rank == 0:
            print(json.dumps({"metric": "batch-1 decode tokens/s, Qwen3-8B random init, W3 g128 (configs[3])", "unit": "tokens/s",
                              "value": decode["w3"]["tokens_per_s"], "n_gpus": 1, "higher_is_better": True, "data": "synthetic",
                              "dtype": "f32", "decode": decode}))
        return
    if args.workload == "binary-basis":
        torch.cuda.set_device(local_rank)
        table, total_us, total_bytes = run_binary_basis(torch, torch.device("cuda", local_rank))
        peak, peak_kind = measured_peak()
        if rank == 0:
            print(json.dumps({"metric": "two-base binary-basis GEMV HBM GB/s per Qwen3-8B shape (configs[2])", "unit": "GB/s",
                              "value": round(total_bytes / total_us / 1e3, 1), "n_gpus": 1, "higher_is_better": True, "data": "synthetic",
                              "dtype": "f32", "us_per_layer": round(total_us, 2), "per_shape": table,
                              "roofline": {"bound": "hbm", "achieved": round(total_bytes / total_us / 1e3, 1), "peak": peak, "unit": "GB/s",
                                           "frac": round(total_bytes / total_us / 1e3 / peak, 4), "peak_kind": peak_kind, "traffic": None}}))
        return
    result = run_ours(args, rank, world, local_rank)
    decode = None
    if world == 1 and not args.headline_only:
        torch.cuda.empty_cache()
        decode = run_decode(torch, "qwen3-8b", 512, 32, 0, 1, local_rank)
    if rank == 0:
        peak, peak_kind = measured_peak()
        total_bytes = result["step_bytes"] * world
        value = total_bytes / (result["step_ms"] * 1e-3) / 1e9
        per_gpu = value / world
        e2e = total_bytes / (result["e2e_ms"] * 1e-3) / 1e9
        for entry in result["per_shape"].values():
            entry["pct_of_8TBps"] = round(100 * entry["gbs"] / NOMINAL_HBM_GBS, 1)
            entry["pct_of_measured"] = round(100 * entry["gbs"] / peak, 1)
            # the same time against the byte count with zero points held as fp16, as the config words them
            entry["gbs_zeros_as_fp16"] = round(entry["gbs"] * (1 + (entry["bytes_zeros_as_fp16"] - entry["bytes"]) / entry["bytes"]), 1)
        cpu = cpu_reference(3, 1) if world == 1 and not args.headline_only else None
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(result["step_ms"], 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "pct_of_8TBps": round(100 * per_gpu / NOMINAL_HBM_GBS, 1),
            "linear_tokens_per_s": round(world * 1e3 / result["step_ms"], 1),
            "per_shape": result["per_shape"], "fused_launches": result["fused"], "m_sweep": result["m_sweep"], "clocks": result["clocks"],
            "e2e": {"value": round(e2e, 1), "unit": "GB/s", "h2d_bytes_per_step": result["h2d"] * world, "d2h_bytes_per_step": result["d2h"] * world},
            "gpu_launches": result["launches"] * world,  # whole job: every rank launches the same graph
            "roofline": {"bound": "hbm", "achieved": round(per_gpu, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(per_gpu / peak, 4), "traffic": None, "peak_kind": peak_kind,
                         "kernel": "w3_gemv_kernel<1,false>", "bytes_per_launch_avg": result["step_bytes"] // (LAYERS * len(SHAPES))},
        }
        # DRAM bytes per launch: ncu measured 20.203 MB for the 12288x4096 launch against 20.087 MB
        # algorithmic (profiles/w3_gemv_12288x4096_m1.md); traffic grows with the bytes a launch
        # streams, so the average launch of this mixed-shape step is scaled by the same ratio.
        line["roofline"]["traffic"] = int(DRAM_TRAFFIC_RATIO * line["roofline"]["bytes_per_launch_avg"])
        if decode is not None:
            line["decode"] = decode
        if cpu is not None:
            line["cpu_baseline"] = {"value": round(cpu["value"], 3), "unit": "GB/s", "cores": cpu["cores"], "kind": "port", "sample": cpu["sample"]}
        print(json.dumps(line))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
