"""The B200 decode engine: its glue kernels against plain tensor math, the packed arm against
the dense BF16 arm through the same glue, graph replay against eager execution."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def small_shape():
    from marlin_style_fluxbin_b200.decode_engine import ModelShape

    return ModelShape(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=128, intermediate=512, vocab=640)


def nrmse(a, b):
    a, b = a.double(), b.double()
    return float((a - b).square().mean().sqrt() / b.square().mean().sqrt())


def test_glue_kernels_match_tensor_math():
    """prefill(T) + one engine step must equal prefill(T+1) at the last position (dense arm):
    that exercises RMSNorm, q/k-norm + RoPE + cache write, attention, SwiGLU and the residuals."""
    from marlin_style_fluxbin_b200.decode_engine import DecodeEngine

    engine = DecodeEngine(small_shape(), device="cuda", max_positions=64, arm="bf16", seed=5)
    ids = torch.randint(0, 640, (1, 24), generator=torch.Generator().manual_seed(1))
    want = engine.prefill(ids).float()
    engine.k_cache.zero_()
    engine.v_cache.zero_()
    engine.prefill(ids[:, :23])
    engine.step(ids[0, 23:24].cuda(), 23)
    got = engine.logits.float()
    assert nrmse(got, want) < 0.02, nrmse(got, want)
    assert int(got.argmax()) == int(want.argmax()) or float(want.max() - want.flatten()[got.argmax()]) < 0.02 * float(want.abs().max())


def test_packed_arm_matches_dense_arm_and_graph_replays_exactly():
    from marlin_style_fluxbin_b200.decode_engine import DecodeEngine

    shape, steps, prompt = small_shape(), 6, 20
    ids = torch.randint(0, 640, (1, prompt), generator=torch.Generator().manual_seed(2))
    arms = {}
    for arm in ("bf16", "w3"):
        engine = DecodeEngine(shape, device="cuda", max_positions=64, arm=arm, seed=7)
        first = engine.prefill(ids).argmax(-1)
        arms[arm] = (engine, first)
    dense, first = arms["bf16"]
    fed, greedy, logits = dense.decode(first, prompt, steps)
    packed, first_packed = arms["w3"]
    assert torch.equal(first, first_packed)  # identical dense prefill in both arms
    fed_p, greedy_p, logits_p = packed.decode(first, prompt, steps, forced=fed)
    # same weights (the dense arm holds the dequantised packed weights): 16-bit-level agreement
    assert nrmse(logits_p, logits) < 0.02, nrmse(logits_p, logits)
    agree = (greedy_p == greedy).float().mean()
    assert agree >= 0.8, (greedy_p, greedy)
    # whole-continuation graph, teacher-forced: bit-identical to eager
    packed.prefill(ids)
    graph, predictions, last = packed.capture(first, prompt, steps, forced=fed)
    packed.prefill(ids)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(predictions, greedy_p)
    assert torch.equal(last, logits_p[-1:])
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(predictions, greedy_p)
    # greedy feedback inside the graph follows the engine's own choices
    packed.prefill(ids)
    _, own, _ = packed.decode(first, prompt, steps)
    packed.prefill(ids)
    graph2, predictions2, _ = packed.capture(first, prompt, steps)
    packed.prefill(ids)
    graph2.replay()
    torch.cuda.synchronize()
    assert torch.equal(predictions2, own)


def test_both_arms_against_the_fp32_yardstick_and_decoded_weight_arithmetic():
    """Neither 16-bit arm is the truth: both are measured against the same model run with fp32
    activations and fp32 dequantised weights.  The packed arm with the dequantised-weight
    arithmetic must not be further from it than the dense arm (whose weights carry one more
    rounding, fp16 product to bf16)."""
    from marlin_style_fluxbin_b200.decode_engine import DecodeEngine

    shape, steps, prompt = small_shape(), 6, 20
    ids = torch.randint(0, 640, (1, prompt), generator=torch.Generator().manual_seed(4))
    dense = DecodeEngine(shape, device="cuda", max_positions=64, arm="bf16", seed=9)
    first = dense.prefill(ids).argmax(-1)
    fed, _, logits_dense = dense.decode(first, prompt, steps)
    truth = dense.truth_logits(ids, fed)
    assert tuple(truth.shape) == (steps, shape.vocab) and truth.dtype == torch.float32
    gaps = {"bf16": nrmse(logits_dense, truth)}
    for arithmetic in ("structural", "decoded_bf16"):
        packed = DecodeEngine(shape, device="cuda", max_positions=64, arm="w3", seed=9, arithmetic=arithmetic)
        packed.prefill(ids)
        _, _, logits_packed = packed.decode(first, prompt, steps, forced=fed)
        gaps[arithmetic] = nrmse(logits_packed, truth)
        packed.check_status()
    assert max(gaps.values()) < 0.02, gaps
    assert gaps["decoded_bf16"] <= 1.25 * gaps["bf16"], gaps


def test_fused_input_launches_match_separate_glue_kernels():
    """Six launches per layer (RMSNorm and the SwiGLU gate inside the GEMVs) against nine."""
    from marlin_style_fluxbin_b200.decode_engine import DecodeEngine

    shape, prompt = small_shape(), 20
    ids = torch.randint(0, 640, (1, prompt), generator=torch.Generator().manual_seed(3))
    logits = {}
    for fuse in (True, False):
        engine = DecodeEngine(shape, device="cuda", max_positions=64, arm="w3", seed=7, fuse_inputs=fuse)
        first = engine.prefill(ids).argmax(-1)
        _, _, logits[fuse] = engine.decode(first, prompt, 4)
        assert engine.launches_per_step == 2 + shape.layers * (5 if fuse else 8)  # gather, layers, fused LM head
    assert nrmse(logits[True], logits[False]) < 5e-3, nrmse(logits[True], logits[False])


@pytest.mark.parametrize("position", (0, 5, 63, 200, 1500))
@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
def test_fused_attention_equals_the_two_launch_form(position, dtype):
    """q/k-norm + RoPE + cache write inside the attention launch: outputs and cache rows are
    bit-identical to fb_qknorm_rope_cache followed by fb_attn_decode."""
    from marlin_style_fluxbin_b200 import _native

    q_heads, kv_heads, dim, max_positions = 8, 2, 128, 1536
    gen = torch.Generator().manual_seed(position + 1)
    rnd = lambda *shape: torch.randn(*shape, generator=gen).to(dtype).cuda()  # noqa: E731
    q, k, v = rnd(1, q_heads * dim), rnd(1, kv_heads * dim), rnd(1, kv_heads * dim)
    q_weight, k_weight = (1 + 0.1 * rnd(dim)), (1 + 0.1 * rnd(dim))
    angle = torch.rand(dim // 2, generator=gen) * 6.28
    cos, sin = torch.cat([angle.cos()] * 2).to(dtype).cuda(), torch.cat([angle.sin()] * 2).to(dtype).cuda()
    caches = [rnd(kv_heads, max_positions, dim) for _ in range(2)]
    scale = dim ** -0.5
    scratch = torch.zeros(_native.attn_scratch_bytes(q_heads), dtype=torch.uint8, device="cuda")

    k_a, v_a = caches[0].clone(), caches[1].clone()
    q_rot, out_a = torch.empty_like(q), torch.empty_like(q)
    _native.qknorm_rope_cache(q, k, v, q_weight, k_weight, cos, sin, q_rot, k_a, v_a, position, 1e-6)
    _native.attn_decode(q_rot, k_a, v_a, out_a, position + 1, scale, scratch)

    k_b, v_b = caches[0].clone(), caches[1].clone()
    out_b = torch.full_like(q, float("nan"))
    _native.attn_decode_fused(q, k, v, q_weight, k_weight, cos, sin, k_b, v_b, out_b, position, 1e-6, scale, scratch)
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b)
    assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
    # and against plain tensor math (fp32 softmax over the 16-bit cache)
    keys, values = k_a[:, :position + 1].float(), v_a[:, :position + 1].float()
    heads = q_rot.view(q_heads, dim).float()
    group = q_heads // kv_heads
    scores = torch.einsum("hd,hpd->hp", heads, keys.repeat_interleave(group, dim=0)) * scale
    want = torch.einsum("hp,hpd->hd", scores.softmax(-1), values.repeat_interleave(group, dim=0)).reshape(1, -1)
    assert (out_b.float() - want).abs().max() <= 2e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("position", (0, 63, 200, 530, 1500))
@pytest.mark.parametrize("dtype,heads", ((torch.bfloat16, (8, 2)), (torch.float16, (8, 2)), (torch.bfloat16, (5, 1))))
def test_attention_pieces_merged_by_the_consuming_gemv(position, dtype, heads):
    """The attention launch that stops at per-split pieces, merged inside the o-projection GEMV's table
    build, gives the output of fb_attn_decode_fused followed by the plain GEMV bit for bit (cache rows too)."""
    from marlin_style_fluxbin_b200 import _native
    from marlin_style_fluxbin_b200.decode_engine import synthetic_w3

    (q_heads, kv_heads), dim, max_positions, hidden = heads, 128, 1536, 384  # five heads: an odd number of groups in the GEMV
    gen = torch.Generator().manual_seed(position + 11)
    rnd = lambda *shape: torch.randn(*shape, generator=gen).to(dtype).cuda()  # noqa: E731
    q, k, v = rnd(1, q_heads * dim), rnd(1, kv_heads * dim), rnd(1, kv_heads * dim)
    q_weight, k_weight = (1 + 0.1 * rnd(dim)), (1 + 0.1 * rnd(dim))
    angle = torch.rand(dim // 2, generator=gen) * 6.28
    cos, sin = torch.cat([angle.cos()] * 2).to(dtype).cuda(), torch.cat([angle.sin()] * 2).to(dtype).cuda()
    caches = [rnd(kv_heads, max_positions, dim) for _ in range(2)]
    scale = dim ** -0.5
    layout = synthetic_w3(hidden, q_heads * dim, torch.device("cuda"), torch.Generator(device="cuda").manual_seed(5))
    residual = rnd(1, hidden)

    def project(run_attention):
        k_cache, v_cache = caches[0].clone(), caches[1].clone()
        scratch = torch.zeros(_native.attn_scratch_bytes(q_heads), dtype=torch.uint8, device="cuda")
        out = torch.full((1, hidden), float("nan"), device="cuda", dtype=dtype)
        matrices = _native.w3_matrix_list([(layout["planes"], layout["scales"], layout.get("zeros"), out, residual)])
        run_attention(k_cache, v_cache, scratch, matrices)
        torch.cuda.synchronize()
        _native.check_status(torch.device("cuda"))
        return out, k_cache, v_cache

    def whole(k_cache, v_cache, scratch, matrices):
        attn = torch.empty_like(q)
        _native.attn_decode_fused(q, k, v, q_weight, k_weight, cos, sin, k_cache, v_cache, attn, position, 1e-6, scale, scratch)
        _native.w3_gemv_multi(attn, matrices, 1, hidden, layout["scales"].dtype, None)

    def pieces(k_cache, v_cache, scratch, matrices):
        splits = _native.attn_decode_partial(q, k, v, q_weight, k_weight, cos, sin, k_cache, v_cache, position, 1e-6, scale, scratch)
        assert 1 <= splits <= 8 and (splits > 1) == (position + 1 > 80)
        _native.w3_gemv_attn_merge(scratch, splits, dtype, q_heads * dim, matrices, 1, hidden, layout["scales"].dtype)

    want, k_a, v_a = project(whole)
    got, k_b, v_b = project(pieces)
    assert torch.isfinite(want.float()).all()
    assert torch.equal(got, want)
    assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
