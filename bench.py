"""Benchmark of the batch-1 packed-Linear decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: all seven Qwen3-8B Linear shapes as W3 group-128 GEMVs at M=1, for 36 layers of
DISTINCT synthetic weights (2.8 GB, far larger than L2, so every weight byte comes from HBM):
uniform codes, fp16 scales U(0.005,0.02), zero points in {3,4}, x ~ N(0,1) bf16.  One step = one
pass over all 252 GEMVs = the Linear work of one decoded token, replayed from a CUDA graph.

One GPU: one launch per Linear through the module interface.  Several GPUs (torchrun): the same
252 GEMVs sharded tensor-parallel, q/k/v/gate/up by output rows, o/down by input groups, each
row-split GEMV followed by its exchange (results pushed from the GEMV epilogue into every rank's
buffer over NVLink, summed by a polling kernel): strong scaling of one token's Linear work.

Metric: HBM GB/s on the algorithmic bytes (stored planes + scales + zero points + x + y).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
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
# DRAM bytes over algorithmic bytes of a 12288x4096 launch, from one profiler capture of that launch;
# traffic grows with the bytes a launch streams, so other launches are scaled by the same ratio.
DRAM_TRAFFIC_RATIO = 20.219 / 20.087
METRIC = "W3 GEMV HBM GB/s (% of 8 TB/s) per Qwen3-8B shape; batch-1 decode tokens/s"


def gemv_bytes(o: int, k: int, zeros: bool = True) -> int:
    """Algorithmic bytes of one M=1 GEMV: planes, fp16 scales, uint8 zero points, x and y."""
    g = k // 128
    return 3 * o * k // 8 + 2 * g * o + (g * o if zeros else 0) + 2 * k + 2 * o


def bb_bytes(o: int, k: int, n_salient: int = 32) -> int:
    """Algorithmic bytes of one two-base GEMV with matrix-wide scales: two sign planes, fp16 row and
    column scales, 32 dense bf16 salient columns with their indices, x and y."""
    return 2 * o * k // 8 + 4 * o + 4 * k + 2 * n_salient * o + 4 * n_salient + 2 * k + 2 * o


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


def capture(torch, fn, stream):
    """Run ``fn`` once eagerly on ``stream`` (sizes scratch, sets kernel attributes), then capture it."""
    fn()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        fn()
    return graph


def paired_rounds(torch, graphs, launches, stream, *, warmup=20, repeats=100, rounds=7):
    """The reference's timing protocol (acceleration_checks.py:42-64, run_w3_lut_benchmark.py:278-285) on
    CUDA graphs: ``warmup`` replays of every arm, then ``rounds`` rounds of ``repeats`` replays each,
    the order of the arms reversed every other round.  Per arm: median microseconds per LAUNCH,
    (max - min) / median over the rounds, and ``stable`` when that is at most 10 %."""
    for graph in graphs.values():
        for _ in range(warmup):
            graph.replay()
    stream.synchronize()
    order = list(graphs)
    samples = {name: [] for name in order}
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for index in range(rounds):
        for name in order if index % 2 == 0 else reversed(order):
            begin.record(stream)
            for _ in range(repeats):
                graphs[name].replay()
            end.record(stream)
            stream.synchronize()
            samples[name].append(begin.elapsed_time(end) * 1000 / (repeats * launches[name]))
    report = {}
    for name, values in samples.items():
        median = statistics.median(values)
        spread = (max(values) - min(values)) / median if median > 0 else float("inf")
        report[name] = {"us": round(median, 3), "relative_range": round(spread, 4), "stable": spread <= 0.10}
    return report


def clock_note(us, clocks):
    """time x median SM MHz: the same kernel at another clock scales by this product."""
    mhz = clocks.get("sm_mhz")
    return None if mhz is None else round(us * mhz, 1)


def run_single_gpu(args, local_rank):
    """One GPU: 252 launches, one per Linear, through ``PackedW3Linear`` (the reference's module surface)."""
    import torch

    from marlin_style_fluxbin_b200 import _native
    from marlin_style_fluxbin_b200.gptq_deployment import restore_planar_w3
    from marlin_style_fluxbin_b200.w3_lut_deployment import PackedW3Linear

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    gen = torch.Generator(device=device).manual_seed(20260916)
    with torch.inference_mode():
        modules = []  # LAYERS x 7 bound modules, distinct weights
        for _ in range(LAYERS):
            for name, o, k in SHAPES:
                module = PackedW3Linear(synthetic_layout(torch, o, k, device, gen), row_tile=1024 if max(o, k) > 4096 else 256)
                module.bind_prepared_decode(torch.bfloat16)
                modules.append((name, module))
        # activations as a decoder layer hands them over: q/k/v read one buffer, o another, gate/up a third, down a
        # fourth (Linears that follow one another on the same buffer do not wait for one another: FB_W3_SAME_INPUT)
        inputs = {"attn_in": 4096, "o_in": 4096, "mlp_in": 4096, "down_in": 12288}
        role = {"q_proj": "attn_in", "k_proj": "attn_in", "v_proj": "attn_in", "o_proj": "o_in", "gate_proj": "mlp_in",
                "up_proj": "mlp_in", "down_proj": "down_in"}
        x_in = {name: torch.randn(1, 1, k, device=device, generator=gen).bfloat16() for name, k in inputs.items()}
        x_dev = {4096: x_in["attn_in"], 12288: x_in["down_in"]}
        # a second buffer per width: single-shape timings alternate between the two, so that no launch there
        # follows one on the same buffer and every launch waits for the one ahead, as a lone Linear does
        x_alt = {k: (x_dev[k], torch.randn(1, 1, k, device=device, generator=gen).bfloat16()) for k in (4096, 12288)}
        x_host = {name: v.cpu().pin_memory() for name, v in x_in.items()}
        last = [m for _, m in modules[-len(SHAPES):]]
        out_host = [torch.empty(1, 1, m.out_features, dtype=torch.bfloat16).pin_memory() for m in last]

        def one_pass():
            for name, module in modules:
                module(x_in[role[name]])

        stream = torch.cuda.Stream(device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            one_pass()
            graph = capture(torch, one_pass, stream)

            def e2e_step():
                for name in x_in:
                    x_in[name].copy_(x_host[name], non_blocking=True)
                graph.replay()
                for host, module in zip(out_host, last):
                    host.copy_(module._decode_output.view(1, 1, -1), non_blocking=True)
                stream.synchronize()

            for _ in range(max(args.warmup, 3)):
                graph.replay()
            stream.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with ClockSampler(local_rank) as clocks:
                begin.record(stream)
                for _ in range(args.steps):
                    graph.replay()
                end.record(stream)
                stream.synchronize()
                # the K timed steps last tens of milliseconds: the protocol rounds below keep the same
                # graph running for about a second under the sampler, so that the clock record holds
                # samples taken under this very load
                protocol = None if args.headline_only else paired_rounds(torch, {"step": graph}, {"step": 1}, stream, warmup=3)["step"]
            step_ms = begin.elapsed_time(end) / args.steps
            clock_summary = clocks.summary()

            per_shape = {}
            if not args.headline_only:
                for name, o, k in SHAPES:
                    if name in ("v_proj", "up_proj", "o_proj"):
                        continue
                    mods = [m for n, m in modules if n == name]
                    dense = [restore_planar_w3(m.layout(), dtype=torch.bfloat16) for m in mods[:6]]  # 6 x 100 MB > L2 for the large shapes
                    y = torch.empty(1, o, device=device, dtype=torch.bfloat16)
                    x2 = x_dev[k].view(1, k)
                    graphs = {"w3": capture(torch, lambda: [m(x_alt[k][i % 2]) for i, m in enumerate(mods)], stream),
                              "cublas_bf16": capture(torch, lambda: [torch.mm(x2, w.t(), out=y) for w in dense], stream)}
                    report = paired_rounds(torch, graphs, {"w3": len(mods), "cublas_bf16": len(dense)}, stream)
                    us = report["w3"]["us"]
                    per_shape[f"{o}x{k}"] = {
                        "us": us, "relative_range": report["w3"]["relative_range"], "stable": report["w3"]["stable"],
                        "gbs": round(gemv_bytes(o, k) / us / 1e3, 1), "bytes": gemv_bytes(o, k),
                        "bytes_zeros_as_fp16": gemv_bytes(o, k) + (k // 128) * o,
                        "us_x_sm_mhz": clock_note(us, clock_summary),
                        "cublas_bf16_dense_us": report["cublas_bf16"]["us"], "speedup_over_cublas_bf16": round(report["cublas_bf16"]["us"] / us, 2)}
                    del dense, graphs

            extras = not args.headline_only
            fused = fused_layer_pass(torch, modules, x_dev, stream) if extras else None
            sweep = m_sweep(torch, modules, device, stream) if extras else None

            for _ in range(3):
                e2e_step()
            stream.synchronize()
            t0 = time.perf_counter()
            begin.record(stream)
            for _ in range(args.steps):
                e2e_step()
            end.record(stream)
            stream.synchronize()
            e2e_ms = max(begin.elapsed_time(end), (time.perf_counter() - t0) * 1e3) / args.steps
            status = _native.status_word(device)

    step_bytes = LAYERS * sum(gemv_bytes(o, k) for _, o, k in SHAPES)
    return {
        "step_ms": step_ms, "e2e_ms": e2e_ms, "step_bytes": step_bytes, "per_shape": per_shape, "fused": fused, "m_sweep": sweep,
        "protocol": protocol, "clocks": dict(clock_summary, sampled_over="the timed steps and the protocol rounds of the same graph"),
        "launches": len(modules) * args.steps, "status": status,
        "h2d": sum(v.numel() * 2 for v in x_host.values()), "d2h": sum(v.numel() * 2 for v in out_host),
    }


def fused_layer_pass(torch, modules, x_dev, stream):
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

    report = paired_rounds(torch, {"layer": capture(torch, run, stream)}, {"layer": len(by_layer)}, stream, warmup=5, repeats=30)["layer"]
    layer_bytes = sum(gemv_bytes(o, k) for _, o, k in SHAPES)
    return {"launches_per_layer": 4, "us_per_layer": report["us"], "relative_range": report["relative_range"], "stable": report["stable"],
            "gbs": round(layer_bytes / report["us"] / 1e3, 1), "status": int(scratch[:4].view(torch.int32)[0])}


def m_sweep(torch, modules, device, stream):
    """M in {1,2,4,8,16} on q_proj and gate_proj: table-lookup kernel (M <= 4), tensor-core kernel, cuBLAS bf16."""
    from marlin_style_fluxbin_b200 import _native
    from marlin_style_fluxbin_b200.gptq_deployment import restore_planar_w3

    out = {}
    scratch = {kind: torch.zeros(8 << 20, dtype=torch.uint8, device=device) for kind in ("lut", "mma")}
    for name in ("q_proj", "gate_proj"):
        mods = [m for n, m in modules if n == name][:12]
        o, k = mods[0].out_features, mods[0].in_features
        dense = [restore_planar_w3(m.layout(), dtype=torch.bfloat16) for m in mods[:6]]
        for rows in (1, 2, 4, 8, 16):
            x = torch.randn(rows, k, device=device).bfloat16()
            y = torch.empty(rows, o, device=device, dtype=torch.bfloat16)
            graphs, launches = {}, {}
            if rows <= 4:
                graphs["lut_us"] = capture(torch, lambda: [_native.w3_gemv(x, m.planes, m.scales, getattr(m, "zeros", None), None, y, scratch=scratch["lut"]) for m in mods], stream)
                launches["lut_us"] = len(mods)
            graphs["mma_us"] = capture(torch, lambda: [_native.w3_gemm_small(x, m.planes, m.scales, getattr(m, "zeros", None), None, y, scratch=scratch["mma"]) for m in mods], stream)
            launches["mma_us"] = len(mods)
            graphs["cublas_bf16_us"] = capture(torch, lambda: [torch.mm(x, w.t(), out=y) for w in dense], stream)
            launches["cublas_bf16_us"] = len(dense)
            report = paired_rounds(torch, graphs, launches, stream, warmup=5, repeats=30, rounds=5)
            entry = {key: value["us"] for key, value in report.items()}
            entry["stable"] = all(value["stable"] for value in report.values())
            best = min(v for key, v in entry.items() if key in ("lut_us", "mma_us"))
            entry["packed_gbs"] = round(gemv_bytes(o, k) / best / 1e3, 1)
            out[f"{o}x{k} M={rows}"] = entry
        del dense
    return out


def run_binary_basis(torch, device):
    """The two-base binary-basis GEMV (1 bit per weight and base, fp16 row / column scales, 32 dense
    bf16 salient columns) on the seven shapes, 12 distinct weight sets per shape."""
    from marlin_style_fluxbin_b200 import _native
    from marlin_style_fluxbin_b200.binary_global import global_two_base_m1_out

    gen = torch.Generator(device=device).manual_seed(20260917)
    stream = torch.cuda.Stream(device)
    stream.wait_stream(torch.cuda.current_stream())
    table, total_us, total_bytes, status = {}, 0.0, 0, 0
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
            report = paired_rounds(torch, {"bb": capture(torch, run, stream)}, {"bb": len(layouts)}, stream, warmup=5, repeats=50)["bb"]
            table[key] = {"us": report["us"], "relative_range": report["relative_range"], "stable": report["stable"],
                          "bytes": bb_bytes(o, k), "gbs": round(bb_bytes(o, k) / report["us"] / 1e3, 1)}
            total_us += report["us"]
            total_bytes += bb_bytes(o, k)
            status |= int(scratch[:4].view(torch.int32)[0])
            del layouts
    torch.cuda.current_stream().wait_stream(stream)
    return table, total_us, total_bytes, status


def run_tensor_parallel(args, rank, world, local_rank):
    """Several GPUs: the 252 GEMVs of one token sharded tensor-parallel (one process per GPU).

    q/k/v/gate/up keep a slice of their output rows and need no exchange; o/down keep a slice of
    their input groups, and their partial rows are pushed from the GEMV epilogue into every rank's
    exchange buffer (plain peer stores over NVLink) and summed there by a polling kernel.  One step
    = the 252 sharded GEMVs + 72 exchanges; the step time is the maximum over the ranks."""
    import torch
    import torch.distributed._symmetric_memory as symm

    from marlin_style_fluxbin_b200 import _native
    from marlin_style_fluxbin_b200.decode_engine import shard_groups, shard_rows

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    gen = torch.Generator(device=device).manual_seed(20260916)  # the same draws on every rank: every rank shards the same weights
    hidden, f16 = 4096, torch.float16
    with torch.inference_mode():
        x_dev = {k: torch.randn(1, k, device=device, generator=gen).bfloat16() for k in (4096, 12288)}
        x_host = {k: v.cpu().pin_memory() for k, v in x_dev.items()}
        header = 64
        xchg = symm.empty(2 * (header + 2 * world * hidden), dtype=torch.float32, device=device)
        xchg.zero_()
        handle = symm.rendezvous(xchg, torch.distributed.group.WORLD.group_name)
        bases = [int(ptr) for ptr in handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        torch.distributed.barrier()
        sites = []
        for site in range(2):
            data = 8 * (header + site * world * hidden)
            sites.append({"push": _native.w3_push_descriptor([base + data + 8 * rank * hidden for base in bases]), "parts": bases[rank] + data})
        scratch = torch.zeros(_native.w3_scratch_bytes(1, 12288, 12288), dtype=torch.uint8, device=device)
        residual = torch.zeros(1, hidden, device=device, dtype=torch.bfloat16)
        plan, keep, outs_last = [], [], []
        for _ in range(LAYERS):
            exchanges = 0
            for name, o, k in SHAPES:
                full = synthetic_layout(torch, o, k, device, gen)
                row_split = name in ("o_proj", "down_proj")
                shard = shard_groups(full, rank, world) if row_split else shard_rows(full, rank, world)
                del full
                out = torch.empty(1, shard["planes"].shape[2], device=device, dtype=torch.bfloat16)
                matrix = _native.w3_matrix_list([(shard["planes"], shard["scales"], shard["zeros"], out, None)])
                k_local = shard["planes"].shape[0] * 128
                x_local = x_dev[k][:, rank * k_local:(rank + 1) * k_local].contiguous() if row_split else x_dev[k]
                plan.append((row_split, sites[exchanges % 2] if row_split else None, matrix, x_local, k_local, out))
                exchanges += int(row_split)
                keep.append(shard)
            outs_last = [entry[5] for entry in plan[-len(SHAPES):]]
        out_host = [torch.empty_like(o, device="cpu").pin_memory() for o in outs_last]

        def one_pass():
            for row_split, site, matrix, x_local, k_local, out in plan:
                if row_split:
                    _native.w3_gemv_push(x_local, 0, None, 0.0, matrix, k_local, f16, site["push"], scratch=scratch)
                    _native.tp_reduce(site["parts"], world, residual, out, bases[rank])
                else:
                    _native.w3_gemv_multi(x_local, matrix, 1, out.shape[1], f16, None, scratch=scratch)

        stream = torch.cuda.Stream(device)
        stream.wait_stream(torch.cuda.current_stream())

        def barrier():
            stream.synchronize()
            torch.distributed.barrier()
            stream.synchronize()

        with torch.cuda.stream(stream):
            one_pass()
            barrier()
            graph = capture(torch, one_pass, stream)
            barrier()

            def e2e_step():
                for k in x_dev:
                    x_dev[k].copy_(x_host[k], non_blocking=True)
                graph.replay()
                for host, out in zip(out_host, outs_last):
                    host.copy_(out, non_blocking=True)
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
                # about half a second more under the sampler; every rank must replay the same number
                # of times (each replay waits for the peers' contributions), so the count is agreed on
                pace = torch.tensor([begin.elapsed_time(end) / args.steps], device=device, dtype=torch.float64)
                torch.distributed.all_reduce(pace, op=torch.distributed.ReduceOp.MAX)
                for _ in range(max(1, int(500.0 / max(float(pace[0]), 1e-3)))):
                    graph.replay()
                barrier()
            step_ms = begin.elapsed_time(end) / args.steps
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
            status = int(scratch[:4].view(torch.int32)[0]) | int(xchg[:1].view(torch.int32)[0])
        times = torch.tensor([step_ms, e2e_ms, float(status)], device=device, dtype=torch.float64)
        torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
    return {
        "step_ms": float(times[0]), "e2e_ms": float(times[1]), "status": int(times[2]),
        "step_bytes": LAYERS * sum(gemv_bytes(o, k) for _, o, k in SHAPES),
        "clocks": clocks.summary(), "launches": (len(plan) + 2 * LAYERS) * args.steps,
        "exchange_bytes_per_step": 2 * LAYERS * hidden * 8 * (world - 1),
        "h2d": sum(v.numel() * 2 for v in x_host.values()), "d2h": sum(v.numel() * 2 for v in out_host),
    }


def nrmse(a, b):
    a, b = a.double(), b.double()
    return round(float((a - b).square().mean().sqrt() / b.square().mean().sqrt()), 5)


def run_decode(torch, shape_name, prompt, steps, rank, world, local_rank, arms=("bf16", "w3"), repeats=5, tp_push=None, truth=True):
    """Full-model batch-1 decode: random-init Qwen3 shape, all Linears W3 g128, LM head bf16; prefill
    `prompt` random ids, then `steps` tokens from ONE CUDA graph.  The BF16 arm runs the same engine
    with dense dequantised weights through cuBLAS.  All arms are fed the BF16 arm's greedy tokens, and
    (unsharded) each arm's logits are measured against the same model run in fp32.  Tensor parallel
    over `world` ranks when world > 1."""
    from marlin_style_fluxbin_b200.decode_engine import QWEN3_8B, QWEN3_32B, DecodeEngine

    shape = {"qwen3-8b": QWEN3_8B, "qwen3-32b": QWEN3_32B}[shape_name]
    device = torch.device("cuda", local_rank)
    ids = torch.randint(0, shape.vocab, (1, prompt), generator=torch.Generator().manual_seed(1))
    out, forced, traces, truth_logits = {}, None, {}, None
    for arm in arms:
        engine_arm, arithmetic = ("w3", "decoded_bf16") if arm == "w3_decoded" else (arm, "structural")
        engine = DecodeEngine(shape, device=device, max_positions=prompt + steps + 8, arm=engine_arm, arithmetic=arithmetic,
                              tp_rank=rank, tp_size=world, tp_push=tp_push)
        first = engine.prefill(ids).argmax(-1)
        fed, greedy, logits = engine.decode(first, prompt, steps, forced=forced)
        engine.prefill(ids)
        engine.keep_logits = False  # the timed graph is a greedy decode: the logits stay on the chip
        graph, predictions, _ = engine.capture(first, prompt, steps, forced=forced)
        engine.prefill(ids)
        graph.replay()
        torch.cuda.synchronize(device)
        engine.check_status()
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
        engine.check_status()
        ms = sorted(times)[len(times) // 2]
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t[0])
        entry = {"tokens_per_s": round(steps / ms * 1e3, 1), "ms_per_token": round(ms / steps, 4),
                 "launches_per_token": engine.launches_per_step,  # in the graph only the first step gathers its embedding row
                 "graph_equals_eager": bool(torch.equal(predictions, greedy)), "status": 0}
        if forced is None:
            forced = fed
            if truth and world == 1:
                truth_logits = engine.truth_logits(ids, fed)
        traces[arm] = (greedy, logits)
        if truth_logits is not None:
            entry["logits_nrmse_vs_fp32"] = nrmse(logits, truth_logits)
            entry["greedy_agreement_with_fp32"] = round(float((greedy == truth_logits.argmax(-1)).float().mean()), 4)
            entry["steps_differing_from_fp32"] = (greedy != truth_logits.argmax(-1)).nonzero().flatten().tolist()
        if arm != arms[0]:
            entry["greedy_agreement_forced"] = round(float((greedy == traces[arms[0]][0]).float().mean()), 4)
            entry[f"steps_differing_from_{arms[0]}_arm"] = (greedy != traces[arms[0]][0]).nonzero().flatten().tolist()
            entry[f"logits_nrmse_vs_{arms[0]}_arm"] = nrmse(logits, traces[arms[0]][1])
        if engine_arm == "bf16":
            weights = sum(v.numel() * 2 for layer in engine.layers for v in layer.dense.values()) + engine.lm_head.numel() * 2
            entry["weight_bytes_per_token"] = weights
            entry["weight_gbs"] = round(weights / (ms / steps) / 1e6, 1)
        out[arm] = entry
        last_engine_fed = fed
        del engine, graph
        torch.cuda.empty_cache()
    packed = [a for a in arms if a.startswith("w3")]
    if world > 1 and packed:
        # the sharded engine against an unsharded engine with the same weights, on rank 0:
        # the exchange changes the summation order, nothing else
        if rank == 0:
            single = DecodeEngine(shape, device=device, max_positions=prompt + steps + 8, arm="w3", tp_rank=0, tp_size=1)
            single.prefill(ids)
            few = min(steps, 8)
            _, greedy_single, logits_single = single.decode(last_engine_fed[:1], prompt, few, forced=last_engine_fed[:few])
            out[packed[0]]["tp_vs_single_logits_nrmse"] = nrmse(traces[packed[0]][1][:few], logits_single)
            out[packed[0]]["tp_vs_single_greedy_agreement"] = round(float((traces[packed[0]][0][:few] == greedy_single).float().mean()), 4)
            del single
            torch.cuda.empty_cache()
        torch.distributed.barrier()
    if "w3" in out and "bf16" in out:
        out["w3_over_bf16"] = round(out["w3"]["tokens_per_s"] / out["bf16"]["tokens_per_s"], 3)
    if truth_logits is not None:
        out["fp32_yardstick"] = ("one causal forward pass of prompt + fed tokens with fp32 activations and fp32 dequantised weights; "
                                 "every arm is fed the first arm's greedy tokens")
    exchange = "none" if world == 1 else ("nccl allreduce" if tp_push is False else "pushed from the GEMV epilogue into peer buffers (packed arm)")
    out["config"] = {"model": shape_name, "prompt_tokens": prompt, "decode_tokens": steps, "tensor_parallel": world, "exchange": exchange,
                     "graph": "whole continuation, teacher-forced from the first arm's greedy tokens, logits kept on the chip"}
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
    passes = 64  # a step is 64 passes over the layer (about half a second): ten seconds or so of timed CPU work at the default 20 steps
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        for _ in range(passes):
            for dense, x in layer:
                orc.dense_gemv_f32(dense, x)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    step_s = sum(times) / len(times) / passes
    nbytes = sum(gemv_bytes(o, k) for _, o, k in SHAPES)
    return {"value": nbytes / step_s / 1e9, "cores": orc.num_threads(), "step_ms": step_s * 1e3,
            "dequant_s_per_layer": t_dequant,
            "sample": (f"one layer (7 Linears, {nbytes} packed bytes), {passes} passes per step, {sum(times):.1f} s timed: fp32 matmul on "
                       f"weights dequantised once outside the timer ({t_dequant:.2f} s per layer when redone every call)")}


def small_case(args):
    """A few launches of one shape on distinct weights (larger than L2 together): the
    small, self-ending program that profiler captures are taken on."""
    import torch

    from marlin_style_fluxbin_b200.w3_lut_deployment import w3_lut_gemv_out, w3_lut_m1_out, workspace_shape

    device = torch.device("cuda", 0)
    gen = torch.Generator(device=device).manual_seed(1)
    if args.case.lower().startswith("lm_head:"):  # the fused LM head on a VxK bf16 weight, a few launches
        from marlin_style_fluxbin_b200 import _native

        v, k = (int(n) for n in args.case.split(":")[1].lower().split("x"))
        weight = (torch.randn(v, k, device=device, generator=gen) * 0.02).bfloat16()
        x = torch.randn(1, k, device=device, generator=gen).bfloat16()
        norm = torch.ones(k, device=device, dtype=torch.bfloat16)
        best = torch.zeros(1, dtype=torch.long, device=device)
        scratch = torch.zeros(_native.lm_head_scratch_bytes(), dtype=torch.uint8, device=device)
        for _ in range(args.copies):
            _native.lm_head_argmax(x, norm, 1e-6, weight, best, scratch=scratch)
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "launches": args.copies, "bytes_per_launch": v * k * 2, "choice": int(best[0])}))
        return
    o, k = (int(v) for v in args.case.lower().split("x"))
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
                        help="gemv (default): the seven Linear shapes (plus, on one GPU, the two-base kernel and the 8B decode; "
                             "on several, the tensor-parallel 32B-shaped decode); the others run one part alone")
    parser.add_argument("--case", default=None, metavar="OxK",
                        help="profiling helper: launch the GEMV of one shape on --copies distinct weights and exit "
                             "(lm_head:VxK launches the fused LM head --copies times instead)")
    parser.add_argument("--prompt-tokens", type=int, default=512, help="decode-8b: prompt length")
    parser.add_argument("--decode-tokens", type=int, default=32, help="decode-8b: tokens decoded in the graph")
    parser.add_argument("--packed-arm-only", action="store_true", help="decode-8b: skip the BF16 arm (for profiler launch lists)")
    parser.add_argument("--tp-exchange", default="push", choices=("push", "nccl"),
                        help="tp-decode-32b: exchange after the row-split GEMVs (fused push, or NCCL allreduce)")
    parser.add_argument("--copies", type=int, default=8)
    parser.add_argument("--rows", type=int, default=1, help="with --case: activation rows (above 1 runs the tensor-core kernel)")
    parser.add_argument("--headline-only", action="store_true",
                        help="time only the headline step (no per-shape table, sweeps, decode or CPU leg): for profiler launch lists")
    parser.add_argument("--no-tp-decode", action="store_true", help="several GPUs: skip the 32B-shaped decode")
    args = parser.parse_args()
    if args.case:
        return small_case(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {
        "workload": "qwen3-8b all seven Linear shapes, W3 g128 GEMV, M=1, 36 layers of distinct weights",
        "shapes": [f"{o}x{k}" for _, o, k in SHAPES], "layers": LAYERS, "gemvs_per_step": LAYERS * len(SHAPES),
        "cache": "inputs larger than L2 (2.8 GB of weights per pass), no flush needed",
        "zero_points": "uint8 per (group,row), counted at their stored size",
        "parallelism": "single GPU" if world == 1 else f"tensor-parallel x{world}, exchange: push",
    }

    if args.impl == "reference":
        if rank != 0:
            return
        ref = cpu_reference(args.steps, min(args.warmup, 1))
        line = {
            "impl": "reference", "metric": METRIC, "value": round(ref["value"], 3), "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ref["step_ms"], 3), "higher_is_better": True,
            "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
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
    peak, peak_kind = measured_peak()
    if args.workload == "tp-decode-32b":
        torch.cuda.set_device(local_rank)
        decode = run_decode(torch, "qwen3-32b", 1024, 64, rank, world, local_rank, arms=("w3",) if world > 1 else ("bf16", "w3"),
                            tp_push=False if args.tp_exchange == "nccl" else None, truth=False)
        if rank == 0:
            print(json.dumps({"metric": "batch-1 decode tokens/s, Qwen3-32B-shaped W3 g128, tensor parallel", "unit": "tokens/s",
                              "value": decode["w3"]["tokens_per_s"], "n_gpus": world, "higher_is_better": True, "scaling": "strong",
                              "data": "synthetic", "dtype": "bf16", "decode": decode}))
        if world > 1:
            torch.distributed.barrier()
            torch.distributed.destroy_process_group()
        return
    if args.workload == "decode-8b":
        torch.cuda.set_device(local_rank)
        decode = run_decode(torch, "qwen3-8b", args.prompt_tokens, args.decode_tokens, 0, 1, local_rank,
                            arms=("w3",) if args.packed_arm_only else ("bf16", "w3", "w3_decoded"), truth=not args.packed_arm_only)
        if rank == 0:
            print(json.dumps({"metric": "batch-1 decode tokens/s, Qwen3-8B random init, W3 g128", "unit": "tokens/s",
                              "value": decode["w3"]["tokens_per_s"], "n_gpus": 1, "higher_is_better": True, "data": "synthetic",
                              "dtype": "bf16", "decode": decode}))
        return
    if args.workload == "binary-basis":
        torch.cuda.set_device(local_rank)
        table, total_us, total_bytes, status = run_binary_basis(torch, torch.device("cuda", local_rank))
        if rank == 0:
            print(json.dumps({"metric": "two-base binary-basis GEMV HBM GB/s per Qwen3-8B shape", "unit": "GB/s",
                              "value": round(total_bytes / total_us / 1e3, 1), "n_gpus": 1, "higher_is_better": True, "data": "synthetic",
                              "dtype": "bf16", "us_per_layer": round(total_us, 2), "per_shape": table, "status": status,
                              "roofline": {"bound": "hbm", "achieved": round(total_bytes / total_us / 1e3, 1), "peak": peak, "unit": "GB/s",
                                           "frac": round(total_bytes / total_us / 1e3 / peak, 4), "peak_kind": peak_kind, "traffic": None}}))
        return

    result = run_single_gpu(args, local_rank) if world == 1 else run_tensor_parallel(args, rank, world, local_rank)
    extras = {}
    if not args.headline_only:
        torch.cuda.empty_cache()
        if world == 1:
            table, total_us, total_bytes, status = run_binary_basis(torch, torch.device("cuda", local_rank))
            extras["binary_basis"] = {"us_per_layer": round(total_us, 2), "gbs": round(total_bytes / total_us / 1e3, 1),
                                      "frac": round(total_bytes / total_us / 1e3 / peak, 4), "per_shape": table, "status": status}
            torch.cuda.empty_cache()
            extras["decode"] = run_decode(torch, "qwen3-8b", 512, 32, 0, 1, local_rank, arms=("bf16", "w3", "w3_decoded"))
        elif not args.no_tp_decode:
            push = run_decode(torch, "qwen3-32b", 1024, 64, rank, world, local_rank, arms=("w3",), truth=False)
            nccl = run_decode(torch, "qwen3-32b", 1024, 64, rank, world, local_rank, arms=("w3",), tp_push=False, truth=False)
            extras["tp_decode"] = {"push": push, "nccl_allreduce": nccl}
    if rank == 0:
        total_bytes = result["step_bytes"]  # one token's Linear work, whatever the number of ranks
        value = total_bytes / (result["step_ms"] * 1e-3) / 1e9
        per_gpu = value / world
        e2e = total_bytes / (result["e2e_ms"] * 1e-3) / 1e9
        for entry in result.get("per_shape", {}).values():
            entry["pct_of_8TBps"] = round(100 * entry["gbs"] / NOMINAL_HBM_GBS, 1)
            entry["pct_of_measured"] = round(100 * entry["gbs"] / peak, 1)
            # the same time against the byte count with zero points held as fp16
            entry["gbs_zeros_as_fp16"] = round(entry["gbs"] * entry["bytes_zeros_as_fp16"] / entry["bytes"], 1)
        cpu = cpu_reference(20, 2) if world == 1 and not args.headline_only else None
        launches_per_step = result["launches"] // args.steps
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(result["step_ms"], 4), "higher_is_better": True,
            "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
            "pct_of_8TBps": round(100 * per_gpu / NOMINAL_HBM_GBS, 1),
            "linear_tokens_per_s": round(1e3 / result["step_ms"], 1), "status": result["status"],
            "clocks": result["clocks"],
            "e2e": {"value": round(e2e, 1), "unit": "GB/s", "h2d_bytes_per_step": result["h2d"] * world, "d2h_bytes_per_step": result["d2h"] * world},
            "gpu_launches": result["launches"] * world,  # whole job: every rank launches its own graph
            "roofline": {"bound": "hbm", "achieved": round(per_gpu, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(per_gpu / peak, 4), "peak_kind": peak_kind, "kernel": "w3_gemv_kernel<1,false>",
                         "bytes_per_launch_avg": result["step_bytes"] // world // (LAYERS * len(SHAPES)),
                         "traffic": int(DRAM_TRAFFIC_RATIO * (result["step_bytes"] // world // (LAYERS * len(SHAPES)))),
                         "note": "per GPU: each rank streams 1/N of the bytes" if world > 1 else
                                 "one launch per Linear; k/v behind q and up behind gate read the same activations and do not wait for the Linear ahead"},
        }
        if world == 1:
            line.update({"protocol": result["protocol"], "per_shape": result["per_shape"], "fused_launches": result["fused"], "m_sweep": result["m_sweep"]})
        else:
            line["tensor_parallel"] = {"launches_per_step_per_rank": launches_per_step, "exchanges_per_step": 2 * LAYERS,
                                       "nvlink_bytes_sent_per_rank_per_step": result["exchange_bytes_per_step"],
                                       "limiter": "launch chain: each rank still runs 324 dependent launches per step while its bytes shrink by 1/N"}
        line.update(extras)
        if cpu is not None:
            line["cpu_baseline"] = {"value": round(cpu["value"], 3), "unit": "GB/s", "cores": cpu["cores"], "kind": "port", "sample": cpu["sample"]}
        print(json.dumps(line))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
