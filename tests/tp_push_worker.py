"""Worker of tests/test_tp_push_gpu.py (one process per GPU under torchrun): a small Qwen3-shaped
model decoded with the exchange fused into the row-split GEMVs, with the NCCL allreduce, and
unsharded; prints one line of figures on rank 0 and exits non-zero on a failed check."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from marlin_style_fluxbin_b200.decode_engine import DecodeEngine, ModelShape  # noqa: E402


def nrmse(a, b):
    a, b = a.double(), b.double()
    return float((a - b).square().mean().sqrt() / b.square().mean().sqrt())


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    shape = ModelShape(layers=4, hidden=1024, q_heads=8, kv_heads=4, head_dim=128, intermediate=2048, vocab=4096)
    prompt, steps = 24, 6
    ids = torch.randint(0, shape.vocab, (1, prompt), generator=torch.Generator().manual_seed(3))
    results = {}
    for label, push in (("nccl", False), ("push", True)):
        engine = DecodeEngine(shape, device=f"cuda:{rank}", max_positions=prompt + steps + 8, arm="w3", tp_rank=rank, tp_size=world, tp_push=push)
        first = engine.prefill(ids).argmax(-1)
        fed, greedy, logits = engine.decode(first, prompt, steps, forced=results["nccl"][0] if results else None)
        engine.prefill(ids)
        graph, predictions, _ = engine.capture(first, prompt, steps, forced=fed)
        engine.prefill(ids)
        dist.barrier()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(predictions, greedy), f"{label}: graph replay differs from eager decode"
        if push:
            assert int(engine._xchg[0:1].view(torch.int32)) == 0, "a bounded wait of the reduce kernel expired"
        results[label] = (fed, greedy, logits)
        del engine, graph
        torch.cuda.empty_cache()
    if rank == 0:
        single = DecodeEngine(shape, device="cuda:0", max_positions=prompt + steps + 8, arm="w3")
        first = single.prefill(ids).argmax(-1)
        _, greedy_single, logits_single = single.decode(first, prompt, steps, forced=results["nccl"][0])
        push_gap, nccl_gap = nrmse(results["push"][2], logits_single), nrmse(results["nccl"][2], logits_single)
        print(f"push vs unsharded {push_gap:.4f}; nccl vs unsharded {nccl_gap:.4f}", flush=True)
        assert push_gap <= 0.03 and nccl_gap <= 0.05, (push_gap, nccl_gap)
        assert torch.equal(results["push"][1], greedy_single)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
