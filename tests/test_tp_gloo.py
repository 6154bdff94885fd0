"""Tensor-parallel sharding of the packed layouts, checked with two CPU ranks over gloo:
column-parallel shards (output rows) concatenate, row-parallel shards (input groups) sum through an
allreduce, and both reproduce the unsharded dequantise-then-matmul result; the keys of the
vocabulary-split LM head pick torch.argmax's row."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from marlin_style_fluxbin_b200.decode_engine import head_key, head_key_row, shard_groups, shard_rows, synthetic_w3
from marlin_style_fluxbin_b200.gptq_deployment import restore_planar_w3, validate_planar_w3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, failures):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(11)  # every rank draws the same full matrices
        col = synthetic_w3(256, 512, "cpu", gen)   # q/k/v/gate/up style
        row = synthetic_w3(128, 1024, "cpu", gen)  # o/down style
        x = torch.randn(1, 512, generator=gen).bfloat16()
        # column parallel: full x, rows split; gather of the shards equals the full product
        mine = shard_rows(col, rank, world)
        assert validate_planar_w3(mine) == (256 // world, 512)
        y_local = x.float() @ restore_planar_w3(mine).float().T
        parts = [torch.empty_like(y_local) for _ in range(world)]
        dist.all_gather(parts, y_local)
        full = x.float() @ restore_planar_w3(col).float().T
        assert torch.equal(torch.cat(parts, dim=1), full)
        # row parallel: x split by groups, partial sums allreduced
        mine = shard_groups(row, rank, world)
        assert validate_planar_w3(mine) == (128, 1024 // world)
        x2 = torch.randn(1, 1024, generator=gen).bfloat16()
        lo, hi = rank * 1024 // world, (rank + 1) * 1024 // world
        partial = x2[:, lo:hi].double() @ restore_planar_w3(mine).double().T
        dist.all_reduce(partial)
        want = x2.double() @ restore_planar_w3(row).double().T
        torch.testing.assert_close(partial, want, rtol=1e-12, atol=1e-12)
        # vocabulary-split LM head: every rank keys the best row of its shard, all ranks take the largest key;
        # the choice equals torch.argmax of the whole logits, ties (planted across the two shards) included
        logits = torch.randn(640, generator=gen).bfloat16()
        logits[7] = logits[400] = logits[401] = 9.0
        logits[100] = -0.0
        rows = 640 // world
        mine = max(head_key(float(logits[r]), r) for r in range(rank * rows, (rank + 1) * rows))
        keys = [None] * world
        dist.all_gather_object(keys, mine)
        assert head_key_row(max(keys)) == int(torch.argmax(logits.float())) == 7
        order = sorted(range(640), key=lambda r: head_key(float(logits[r]), r), reverse=True)
        assert order == sorted(range(640), key=lambda r: (-float(logits[r]), r))  # descending logit, ascending row
    except Exception as exc:  # pragma: no cover - reported to the parent
        failures.put(f"rank {rank}: {exc!r}")
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded():
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, failures)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert failures.empty(), failures.get()
