"""The fused LM head (final RMSNorm + dense 16-bit GEMV + argmax + next token's embedding row) against
plain tensor math.  The reference runs this step as the stock Linear plus ``torch.argmax``
(docs/performance/NONLINEAR_FUSION.md:100); the oracle is therefore fp32 tensor arithmetic on the CPU
copy of the same bits.

Tolerance: logits are 16-bit outputs of an fp32-accumulated dot product, so they may differ from
another summation order by one 16-bit ulp; the chosen index must be a row whose oracle logit (rounded
to 16 bits) ties with the oracle's maximum, and with exactly representable data it must equal
``torch.argmax`` including its lowest-index tie rule.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def run_head(x, weight, *, norm=None, logits=True, forced=None, embedding=None):
    from marlin_style_fluxbin_b200 import _native

    v, k = weight.shape
    best = torch.full((1,), -1, dtype=torch.long, device="cuda")
    out = torch.full((1, v), float("nan"), device="cuda", dtype=x.dtype) if logits else None
    scratch = torch.zeros(_native.lm_head_scratch_bytes(), dtype=torch.uint8, device="cuda")
    nxt = torch.zeros(1, k, device="cuda", dtype=x.dtype) if embedding is not None else None
    for _ in range(2):  # twice: the control words must come back to zero
        _native.lm_head_argmax(x, norm, 1e-6, weight, best, logits=out, forced_next=forced, embedding=embedding, next_hidden=nxt,
                               scratch=scratch)
    torch.cuda.synchronize()
    assert int(scratch.view(torch.int64).abs().sum()) == 0
    return int(best[0]), out, nxt


@pytest.mark.parametrize("vocab,k", ((151936, 4096), (151936, 5120), (1000, 264)))
@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
def test_logits_and_choice_against_tensor_math(vocab, k, dtype):
    gen = torch.Generator().manual_seed(vocab + k)
    weight = (torch.randn(vocab, k, generator=gen) * 0.02).to(dtype)
    x = torch.randn(1, k, generator=gen).to(dtype)
    norm = (1 + 0.1 * torch.randn(k, generator=gen)).to(dtype)
    xf = x.float()
    normed = (norm.float() * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(dtype).float()).to(dtype)
    want = (normed.double() @ weight.double().t()).float()
    best, logits, _ = run_head(x.cuda(), weight.cuda(), norm=norm.cuda())
    got = logits.float().cpu()
    ulp = want.abs().clamp_min(1e-3) * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10)
    assert bool(((got - want).abs() <= ulp + 1e-4).all())
    # the choice is the argmax of the kernel's own 16-bit logits with torch's tie rule ...
    assert best == int(torch.argmax(logits, dim=-1))
    # ... and a row that the oracle also puts within one 16-bit ulp of its maximum
    assert float(want[0, best]) >= float(want.max()) - float(ulp[0, best]) - 1e-4
    # without the logits buffer the choice is the same
    assert run_head(x.cuda(), weight.cuda(), norm=norm.cuda(), logits=False)[0] == best


def test_exact_ties_go_to_the_lowest_index_and_next_embedding_row():
    """Integer-valued data: every product and sum is exact, so the logits equal torch's bit for bit;
    three rows are planted with the same maximal logit."""
    vocab, k = 20000, 1024
    gen = torch.Generator().manual_seed(3)
    weight = torch.randint(-2, 3, (vocab, k), generator=gen).float()
    x = torch.randint(-1, 2, (1, k), generator=gen).float()
    top = weight.abs().sum(-1).max() + 5  # above every other row's logit
    for row in (17321, 905, 12000):
        weight[row] = 0
        picks = (x[0] != 0).nonzero().flatten()[: int(top)]
        weight[row, picks] = x[0, picks]  # logit = number of picks
    weight, x = weight.bfloat16(), x.bfloat16()
    want_logits = torch.nn.functional.linear(x.float(), weight.float()).bfloat16()
    embedding = torch.randn(vocab, k, generator=gen).bfloat16().cuda()
    best, logits, nxt = run_head(x.cuda(), weight.cuda(), embedding=embedding)
    assert torch.equal(logits.cpu(), want_logits)
    assert best == int(torch.argmax(want_logits, dim=-1)) == 905
    assert torch.equal(nxt[0], embedding[905])
    forced = torch.tensor([4242], device="cuda")
    _, _, nxt = run_head(x.cuda(), weight.cuda(), embedding=embedding, forced=forced)
    assert torch.equal(nxt[0], embedding[4242])


def test_embed_row_and_rejections():
    from marlin_style_fluxbin_b200 import _native

    table = torch.randn(300, 256).bfloat16().cuda()
    out = torch.zeros(1, 256, device="cuda", dtype=torch.bfloat16)
    _native.embed_row(table, torch.tensor([123], device="cuda"), out)
    assert torch.equal(out[0], table[123])
    best = torch.zeros(1, dtype=torch.long, device="cuda")
    with pytest.raises(_native.NativeError, match="scratch"):
        _native.lm_head_argmax(out, None, 0.0, table, best, scratch=torch.zeros(16, dtype=torch.uint8, device="cuda"))
    with pytest.raises(_native.NativeError, match="multiple of 8"):
        _native.lm_head_argmax(out[:, :100], None, 0.0, table[:, :100].contiguous(), best,
                               scratch=torch.zeros(256, dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("world", (2, 8))
def test_vocabulary_shards_agree_through_the_key_exchange(world):
    """The LM head split by rows over `world` ranks, all of them emulated on one device (the shard launches
    complete before the receiving launches start, so no kernel waits on a later one): every rank's receiving
    kernel names the row that the unsplit kernel names, the shards' logits tile the unsplit logits bit for bit,
    the key slots come back to zero, and the planted tie across two shards goes to the lower row."""
    from marlin_style_fluxbin_b200 import _native

    vocab, k, dtype = 4096, 512, torch.bfloat16
    gen = torch.Generator().manual_seed(world)
    weight = torch.randint(-2, 3, (vocab, k), generator=gen).float()
    x = torch.randint(-2, 3, (1, k), generator=gen).float()
    top = float((x @ weight.t()).max()) + 8
    pattern = torch.zeros(k)
    pattern[0] = 1.0
    x[0, 0] = 1.0
    for row in (vocab // world + 3, 5):  # the same maximal logit in shard 1 and in shard 0: the lower row wins
        weight[row] = 0
        weight[row, 0] = top
    weight, x = weight.to(dtype).cuda(), x.to(dtype).cuda()
    embedding = torch.randn(vocab, k, generator=gen).to(dtype).cuda()
    whole_best, whole_logits, _ = run_head(x, weight)
    assert whole_best == 5

    rows = vocab // world
    keys = torch.zeros(world, world, dtype=torch.int64, device="cuda")  # [receiving rank][sending rank]
    descriptor = _native.w3_push_descriptor([keys[r].data_ptr() for r in range(world)])
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    logits = torch.full((1, vocab), float("nan"), device="cuda", dtype=dtype)
    scratch = torch.zeros(_native.lm_head_scratch_bytes(), dtype=torch.uint8, device="cuda")
    for rank in range(world):
        _native.lm_head_shard(x, None, 1e-6, weight[rank * rows:(rank + 1) * rows], rank * rows, descriptor, rank,
                              logits_shard=logits[:, rank * rows:(rank + 1) * rows], scratch=scratch)
    forced = torch.tensor([77], dtype=torch.long, device="cuda")
    for rank in range(world):
        best = torch.full((1,), -1, dtype=torch.long, device="cuda")
        hidden = torch.zeros(1, k, device="cuda", dtype=dtype)
        _native.tp_argmax(keys[rank].data_ptr(), world, best, status.data_ptr(), forced_next=forced if rank % 2 else None, embedding=embedding,
                          next_hidden=hidden)
        torch.cuda.synchronize()
        assert int(best[0]) == whole_best
        assert torch.equal(hidden[0], embedding[77 if rank % 2 else whole_best])
    assert torch.equal(logits, whole_logits)
    assert int(keys.abs().sum()) == 0 and int(status[0]) == 0 and int(scratch.view(torch.int64).abs().sum()) == 0
    # a key that never arrives: the bounded poll gives up, reports status 6 and the launch ends
    keys[0, 0] = 12345
    best = torch.full((1,), -1, dtype=torch.long, device="cuda")
    _native.tp_argmax(keys[0].data_ptr(), world, best, status.data_ptr(), wait_ns=5_000_000)
    torch.cuda.synchronize()
    assert int(status[0]) == 6 and int(keys[0].abs().sum()) == 0
