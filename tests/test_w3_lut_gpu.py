"""Parity of the CUDA W3 GEMV (through the C ABI) with the CPU oracle and the reference's
golden fixtures.  Cases follow the reference's tests/test_w3_lut_correctness.py (small
shapes with tails, fp16/bf16, every row tile, NaN-filled workspace, repeat-exact and
CUDA-graph-replay-exact) and add the benchmark shapes, zero points, fp16 scales, the
desc_act permutation and M = 1..4.

Tolerance (stated by the task for this floating-point path): max |y - ref| / max |ref|
<= 1e-2 on the 16-bit outputs against dequantise-then-matmul with fp32 accumulation;
the reference's combined numerical gate must pass as well.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2


def make_case(o, k, *, seed=0, zeros=False, perm=False, scale_dtype=torch.float16, act_dtype=torch.bfloat16, m=1):
    """Synthetic Linear as the benchmark configs draw it: uniform codes, scales U(0.005,0.02),
    zero points in {3,4}, x ~ N(0,1)."""
    gen = torch.Generator().manual_seed(seed)
    groups = k // 128
    layout = {
        "planes": torch.randint(0, 256, (groups, 3, o, 16), generator=gen, dtype=torch.uint8),
        "scales": (torch.rand(groups, o, generator=gen) * 0.015 + 0.005).to(scale_dtype),
        "perm": (torch.randperm(k, generator=gen) if perm else torch.arange(k)).to(torch.int16),
    }
    if zeros:
        layout["zeros"] = torch.randint(3, 5, (groups, o), generator=gen, dtype=torch.uint8)
    x = torch.randn(m, k, generator=gen).to(act_dtype)
    return layout, x


def oracle_outputs(layout, x):
    args = (orc.bits(x), orc.tag(x.dtype), layout["planes"].numpy(), orc.bits(layout["scales"]),
            orc.tag(layout["scales"].dtype), layout["zeros"].numpy() if "zeros" in layout else None,
            layout["perm"].numpy())
    return orc.w3_gemv_dequant(*args), orc.w3_gemv_structural(*args)


def assert_parity(out, reference, *, tol=REL_TOL):
    from marlin_style_fluxbin_b200.acceleration_checks import numerical_gate

    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    rel = np.abs(got - reference).max() / np.abs(reference).max()
    assert rel <= tol, rel
    # The gate's bf16 thresholds apply whatever the output dtype: the distance to the
    # dequantised-weight product is set by the 16-bit rounding of scale*(+/-3), not by the output.
    gate = numerical_gate(out.cpu(), torch.from_numpy(reference).to(torch.bfloat16))
    assert gate["passed"], gate


def to_cuda(layout):
    return {k: v.cuda() for k, v in layout.items()}


def run(layout_gpu, x_gpu, *, arithmetic="structural", gps=1, row_tile=256, nan_workspace=True):
    from marlin_style_fluxbin_b200.w3_lut_deployment import w3_lut_m1_out, workspace_shape

    o, k = layout_gpu["planes"].shape[2], x_gpu.shape[1]
    out = torch.full((1, o), float("nan"), device="cuda", dtype=x_gpu.dtype)
    workspace = torch.full(workspace_shape(o, k, gps), float("nan"), device="cuda")
    w3_lut_m1_out(x_gpu, layout_gpu, out, workspace, row_tile=row_tile, groups_per_split=gps, arithmetic=arithmetic)
    return out, workspace


@pytest.mark.parametrize("case", ("w3_k256_o64", "w3_k512_o256", "w3_k384_o288"))
def test_reference_fixtures_through_cuda(golden, case):
    """Layouts produced by the reference's converter, outputs of the reference's oracles."""
    from marlin_style_fluxbin_b200.w3_lut_deployment import ROW_TILES

    g = golden(case)
    layout = to_cuda({"planes": torch.from_numpy(g["planes"]), "scales": orc.unbits(g["scales_bf16"], torch.bfloat16),
                      "perm": torch.from_numpy(g["perm"])})
    x = orc.unbits(g["x_bf16"], torch.bfloat16).cuda()
    for row_tile in ROW_TILES:
        out, _ = run(layout, x, row_tile=row_tile)
        torch.testing.assert_close(out.float().cpu(), torch.from_numpy(g["structural"]), rtol=0.02, atol=0.02)
        assert_parity(out, g["dequant_matmul"])
    corrected, _ = run(layout, x, arithmetic="decoded_bf16")
    torch.testing.assert_close(corrected.float().cpu(), torch.from_numpy(g["bf16_weight_semantics"]).bfloat16().float(), rtol=0.005, atol=0.02)
    # the correction moves the result towards the dense-weight product
    e_plain = np.abs(run(layout, x)[0].float().cpu().numpy() - g["dequant_matmul"]).mean()
    e_corr = np.abs(corrected.float().cpu().numpy() - g["dequant_matmul"]).mean()
    assert e_corr <= e_plain


@pytest.mark.parametrize("o,k", ((32, 128), (64, 256), (288, 384)))
@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16))
def test_small_shapes_repeat_and_graph_exact(o, k, dtype):
    from marlin_style_fluxbin_b200.w3_lut_deployment import ROW_TILES, w3_lut_m1_out, workspace_shape

    layout, x = make_case(o, k, seed=20260916, perm=True, scale_dtype=torch.bfloat16, act_dtype=dtype)
    reference, structural = oracle_outputs(layout, x)
    lg, xg = to_cuda(layout), x.cuda()
    for row_tile in ROW_TILES:
        for gps in (1, k // 128):
            out, workspace = run(lg, xg, row_tile=row_tile, gps=gps)
            assert_parity(out, reference)
            torch.testing.assert_close(out.float().cpu(), torch.from_numpy(structural), rtol=0.02, atol=0.02)
            saved = out.clone()
            w3_lut_m1_out(xg, lg, out, workspace, row_tile=row_tile, groups_per_split=gps)
            assert torch.equal(out, saved)
            for _ in range(3):
                w3_lut_m1_out(xg, lg, out, workspace, row_tile=row_tile, groups_per_split=gps)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                w3_lut_m1_out(xg, lg, out, workspace, row_tile=row_tile, groups_per_split=gps)  # sizes this stream's scratch
            torch.cuda.current_stream().wait_stream(stream)
            with torch.cuda.graph(graph, stream=stream):
                w3_lut_m1_out(xg, lg, out, workspace, row_tile=row_tile, groups_per_split=gps)
            out.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, saved)


QWEN3_SHAPES = {"q_proj": (4096, 4096), "k_proj": (1024, 4096), "gate_proj": (12288, 4096), "down_proj": (4096, 12288)}


@pytest.mark.parametrize("name", sorted(QWEN3_SHAPES))
def test_benchmark_shapes_with_zero_points(name):
    o, k = QWEN3_SHAPES[name]
    layout, x = make_case(o, k, seed=7, zeros=True)
    reference, _ = oracle_outputs(layout, x)
    lg, xg = to_cuda(layout), x.cuda()
    out, _ = run(lg, xg, row_tile=1024)
    assert_parity(out, reference)
    # size-independent properties: scaling by two (exact in every fp32 step; the K split is
    # combined in fixed point with steps of 2^-26, which can move a 16-bit rounding boundary in
    # a rare row, by one ulp), exact under a shift of the rows by a whole 32-row unit, and zero
    # for all-zero signed codes
    doubled, _ = run(lg, (x * 2).cuda(), row_tile=1024)
    twice = out.float() * 2
    differing = doubled.float() != twice
    assert float(differing.float().mean()) <= 2e-3
    assert float((doubled.float() - twice).abs().max()) <= float(twice.abs().max()) * 2.0 ** -7
    rolled = dict(lg, planes=lg["planes"].roll(32, dims=2), scales=lg["scales"].roll(32, dims=1), zeros=lg["zeros"].roll(32, dims=1))
    assert torch.equal(run(rolled, xg, row_tile=1024)[0], out.roll(32, dims=1))
    flat = dict(lg)
    flat["planes"] = torch.zeros_like(lg["planes"])  # stored planes 0,0,0 = code 4
    flat.pop("zeros")
    assert float(run(flat, xg, row_tile=1024)[0].abs().max()) == 0.0


def test_desc_act_permutation_and_fp16_everything():
    layout, x = make_case(1024, 1024, seed=3, zeros=True, perm=True, act_dtype=torch.float16)
    reference, _ = oracle_outputs(layout, x)
    out, _ = run(to_cuda(layout), x.cuda())
    assert_parity(out, reference)


@pytest.mark.parametrize("m", (1, 2, 3, 4))
def test_small_batch_rows(m):
    from marlin_style_fluxbin_b200.w3_lut_deployment import w3_lut_gemv_out

    layout, x = make_case(2048, 1024, seed=11 + m, zeros=(m % 2 == 0), m=m)
    reference, _ = oracle_outputs(layout, x)
    out = torch.empty(m, 2048, device="cuda", dtype=torch.bfloat16)
    w3_lut_gemv_out(x.cuda(), to_cuda(layout), out, kernel="lut")
    for row in range(m):
        assert_parity(out[row:row + 1], reference[row:row + 1])
    single = torch.empty(1, 2048, device="cuda", dtype=torch.bfloat16)
    w3_lut_gemv_out(x[:1].cuda(), to_cuda(layout), single, kernel="lut")
    assert torch.equal(single[0], out[0])  # a row's result does not depend on its neighbours


@pytest.mark.parametrize("o,k,m,dtype,scale_dtype,zeros,perm", (
    (2048, 1024, 16, torch.bfloat16, torch.float16, True, False),
    (2048, 1024, 5, torch.float16, torch.float16, False, False),
    (96, 384, 8, torch.bfloat16, torch.bfloat16, True, False),     # a partial 128-row tile, an odd group count
    (160, 128, 3, torch.bfloat16, torch.float16, False, False),    # one group: no K split
    (1024, 1024, 16, torch.float16, torch.bfloat16, True, True),   # desc_act gather
    (4096, 4096, 16, torch.bfloat16, torch.float16, True, False),  # q_proj
    (4096, 12288, 8, torch.bfloat16, torch.float16, True, False),  # down_proj
))
def test_tensor_core_small_batch(o, k, m, dtype, scale_dtype, zeros, perm):
    """The tcgen05 form (M = 1..16) against dequantise-then-matmul, its oracle: the reference has no
    packed path for M > 1.  Weights are rounded to the activation dtype before the product, as in
    the reference's dense fallback, so the distance to the fp32 oracle is that of a 16-bit Linear."""
    from marlin_style_fluxbin_b200.w3_lut_deployment import w3_lut_gemv_out

    layout, x = make_case(o, k, seed=3 * m + o % 7, zeros=zeros, perm=perm, scale_dtype=scale_dtype, act_dtype=dtype, m=m)
    reference, _ = oracle_outputs(layout, x)
    lg, xg = to_cuda(layout), x.cuda()
    out = torch.full((m, o), float("nan"), device="cuda", dtype=dtype)
    w3_lut_gemv_out(xg, lg, out, kernel="mma")
    torch.cuda.synchronize()
    for row in range(m):
        assert_parity(out[row:row + 1], reference[row:row + 1])
    again = torch.full_like(out, float("nan"))
    w3_lut_gemv_out(xg, lg, again, kernel="mma")
    assert torch.equal(again, out)  # repeat-exact
    single = torch.empty(1, o, device="cuda", dtype=dtype)
    w3_lut_gemv_out(xg[:1].contiguous(), lg, single, kernel="mma")
    assert torch.equal(single[0], out[0])  # a row's result does not depend on its neighbours
    # close to the table-lookup kernel's answer for the same row (different roundings of the weights)
    lut = torch.empty(1, o, device="cuda", dtype=dtype)
    w3_lut_gemv_out(xg[:1].contiguous(), lg, lut, kernel="lut")
    assert float((lut.float() - single.float()).abs().max()) <= 2e-2 * float(lut.float().abs().max())


def test_two_call_form_and_native_argument_contract():
    from marlin_style_fluxbin_b200.w3_lut_deployment import finish, inline_main, load_w3_lut_extension, workspace_shape

    layout, x = make_case(288, 384, seed=5, scale_dtype=torch.bfloat16)
    reference, _ = oracle_outputs(layout, x)
    lg, xg = to_cuda(layout), x.cuda()
    workspace = torch.full(workspace_shape(288, 384), float("nan"), device="cuda")
    out = torch.empty(1, 288, device="cuda", dtype=torch.bfloat16)
    inline_main(xg, lg, workspace, row_tile=256)
    assert bool(torch.isfinite(workspace).all())
    finish(workspace, out, row_tile=256)
    assert_parity(out, reference)
    ext = load_w3_lut_extension(256)
    with pytest.raises(RuntimeError):
        ext.m1_out(xg.expand(2, -1).contiguous(), lg["planes"], lg["scales"], lg["perm"], workspace, out, 1, False)
    with pytest.raises(RuntimeError):
        ext.inline_main(xg, lg["planes"], lg["scales"], lg["perm"], workspace[:2])
    with pytest.raises(ValueError):
        inline_main(xg[:, :256], lg, workspace, row_tile=256)


def test_native_rejections_carry_messages():
    from marlin_style_fluxbin_b200 import _native

    layout, x = make_case(64, 256)
    lg, xg = to_cuda(layout), x.cuda()
    out = torch.empty(1, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(_native.NativeError, match="overlaps"):
        _native.w3_gemv(xg, lg["planes"], lg["scales"], None, None, xg[:, :64])
    with pytest.raises(_native.NativeError, match="scratch"):
        _native.w3_gemv(xg, lg["planes"], lg["scales"], None, None, out, scratch=torch.zeros(256, dtype=torch.uint8, device="cuda"))
    with pytest.raises(_native.NativeError, match="multiple of 32"):
        _native.w3_gemv(xg, lg["planes"][:, :, :40].contiguous(), lg["scales"][:, :40].contiguous(), None, None, out[:, :40])
    # the attention-pieces entry points: split count outside 1..8, a pieces buffer that is too small
    matrices = _native.w3_matrix_list([(lg["planes"], lg["scales"], None, out, None)])
    pieces = torch.zeros(_native.attn_scratch_bytes(2), dtype=torch.uint8, device="cuda")
    for splits in (0, 9):
        with pytest.raises(_native.NativeError, match="splits"):
            _native.w3_gemv_attn_merge(pieces, splits, torch.bfloat16, 256, matrices, 1, 64, lg["scales"].dtype)
    head = torch.zeros(1, 256, device="cuda", dtype=torch.bfloat16)
    row, cache = torch.zeros(128, device="cuda", dtype=torch.bfloat16), torch.zeros(1, 16, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(_native.NativeError, match="buffer"):
        _native.attn_decode_partial(head, head[:, :128], head[:, :128], row, row, row, row, cache, cache.clone(), 3, 1e-6, 1.0, pieces[:64])
    assert _native.library().fb_attn_decode_splits(80) == 1 and _native.library().fb_attn_decode_splits(81) == 2
    assert _native.library().fb_attn_decode_splits(100000) == 8 and _native.library().fb_attn_decode_splits(0) == 0


def test_prepared_linear_binding_and_graph():
    from marlin_style_fluxbin_b200.w3_lut_deployment import PackedW3Linear

    layout, x = make_case(256, 512, seed=9, scale_dtype=torch.bfloat16, perm=True)
    reference, _ = oracle_outputs(layout, x)
    with torch.inference_mode():
        module = PackedW3Linear(layout, fallback="dense", row_tile=256).cuda()
        x3 = x.cuda().view(1, 1, 512)
        eager = module(x3).clone()
        assert module.last_route == "packed_m1"
        assert_parity(eager.view(1, 256), reference)
        dense = module(torch.cat((x3, x3), 1))
        assert module.last_route == "dense_fallback" and tuple(dense.shape) == (1, 2, 256)
        assert_parity(dense[:, 0], reference, tol=2e-2)
        module.bind_prepared_decode(torch.bfloat16)
        try:
            module._decode_audit = True
            module.route_counts = {"packed_m1": 0, "dense_fallback": 0}
            bound = module(x3)
            assert torch.equal(bound, eager) and module.route_counts["packed_m1"] == 1
            pointer = bound.data_ptr()
            module._decode_audit = False
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                for _ in range(3):
                    module(x3)
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                output = module(x3)
            x3.mul_(0.5)
            graph.replay()
            torch.cuda.synchronize()
            assert output.data_ptr() == pointer
            assert torch.equal(output.float(), eager.float() * 0.5)
            with pytest.raises(ValueError):
                module(x3.view(1, 512))
        finally:
            module.clear_prepared_decode()
        assert module._decode_output is None


def test_fused_matrices_share_one_launch_and_residual_epilogue():
    """q/k/v-style fusion: three matrices on the same x in one launch give bit-identical rows to
    three single launches; the residual epilogue equals a separate add in the output dtype."""
    from marlin_style_fluxbin_b200 import _native

    k = 1024
    cases = [make_case(o, k, seed=30 + i, zeros=(i == 1)) for i, o in enumerate((256, 64, 96))]
    x = cases[0][1].cuda()
    singles, entries, keep = [], [], []
    residual = torch.randn(1, 256, generator=torch.Generator().manual_seed(2)).bfloat16().cuda()
    for i, (layout, _) in enumerate(cases):
        lg = to_cuda(layout)
        out = torch.empty(1, layout["planes"].shape[2], device="cuda", dtype=torch.bfloat16)
        _native.w3_gemv(x, lg["planes"], lg["scales"], lg.get("zeros"), None, out)
        singles.append(out)
        fused_out = torch.full_like(out, float("nan"))
        entries.append((lg["planes"], lg["scales"], lg.get("zeros"), fused_out, residual if i == 0 else None))
        keep.append(lg)
        reference, _ = oracle_outputs(layout, cases[0][1])
        assert_parity(out, reference)
    array = _native.w3_matrix_list(entries)
    _native.w3_gemv_multi(x, array, 3, 256 + 64 + 96, torch.float16, None)
    torch.cuda.synchronize()
    assert torch.equal(entries[0][3], (singles[0].float() + residual.float()).bfloat16())
    assert torch.equal(entries[1][3], singles[1]) and torch.equal(entries[2][3], singles[2])


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
def test_fused_input_transforms_equal_separate_kernels(dtype):
    """RMSNorm / SwiGLU-gate fused into the table build give the rows of the two-launch form.
    The SwiGLU form is bit-identical (same per-element arithmetic); RMSNorm sums the squares in a
    different order, so its 1/rms may differ in the last bit: 16-bit-level tolerance there."""
    from marlin_style_fluxbin_b200 import _native

    k, o = 2048, 384
    layout, x_host = make_case(o, k, seed=41, zeros=True, act_dtype=dtype)
    lg, x = to_cuda(layout), (x_host * 3).to(dtype).cuda()
    gen = torch.Generator().manual_seed(5)
    weight = (1 + 0.1 * torch.randn(k, generator=gen)).to(dtype).cuda()
    up = torch.randn(1, k, generator=gen).to(dtype).cuda()

    def two_launch(x_eff):
        out = torch.empty(1, o, device="cuda", dtype=dtype)
        _native.w3_gemv(x_eff.contiguous(), lg["planes"], lg["scales"], lg["zeros"], None, out)
        return out

    def fused(kind, operand, eps):
        out = torch.full((1, o), float("nan"), device="cuda", dtype=dtype)
        array = _native.w3_matrix_list([(lg["planes"], lg["scales"], lg["zeros"], out, None)])
        _native.w3_gemv_fused_input(x, kind, operand, eps, array, 1, o, torch.float16)
        torch.cuda.synchronize()
        return out

    act = torch.empty_like(x)
    _native.silu_mul(x, up, act)
    assert torch.equal(fused(_native.W3_INPUT_SILU_MUL, up, 0.0), two_launch(act))
    # and against plain tensor math through the oracle's dequantised product
    silu = (torch.nn.functional.silu(x.float()).to(dtype).float() * up.float()).to(dtype)
    reference, _ = oracle_outputs(layout, silu.cpu())
    assert_parity(fused(_native.W3_INPUT_SILU_MUL, up, 0.0), reference)

    normed = torch.empty_like(x)
    _native.rmsnorm(x, weight, normed, 1e-6)
    got, want = fused(_native.W3_INPUT_RMSNORM, weight, 1e-6), two_launch(normed)
    assert (got.float() - want.float()).abs().max() <= 2e-2 * want.float().abs().max()
    reference, _ = oracle_outputs(layout, normed.cpu())
    assert_parity(got, reference)
    # repeat-exact
    assert torch.equal(got, fused(_native.W3_INPUT_RMSNORM, weight, 1e-6))
    # a permuted column order or M > 1 is refused
    two = torch.cat([x, x])
    out2 = torch.empty(2, o, device="cuda", dtype=dtype)
    lib = _native.library()
    array = _native.w3_matrix_list([(lg["planes"], lg["scales"], lg["zeros"], out2, None)])
    assert lib.fb_w3_gemv_fused_input(two.data_ptr(), _native.dtype_tag(dtype), 3, weight.data_ptr(), 1e-6, array, 1,
                                      _native.dtype_tag(torch.float16), k, None, 0, 0, None) == -1


def test_split_k_combine_flags_non_finite_partials_and_resets():
    """The K split is combined in 64-bit fixed point; a non-finite (or absurdly large) partial sum
    cannot be represented there and is reported as NaN, and the combine words are left clean."""
    from marlin_style_fluxbin_b200 import _native

    o, k = 96, 1024
    layout, x_host = make_case(o, k, seed=77)
    lg = to_cuda(layout)
    scratch = torch.zeros(_native.w3_scratch_bytes(1, o, k), dtype=torch.uint8, device="cuda")
    good = torch.empty(1, o, device="cuda", dtype=torch.bfloat16)
    _native.w3_gemv(x_host.cuda(), lg["planes"], lg["scales"], None, None, good, scratch=scratch)
    for poison in (float("nan"), float("inf"), 3.0e38):
        bad_x = x_host.clone()
        bad_x[0, 300] = poison
        bad = torch.zeros(1, o, device="cuda", dtype=torch.bfloat16)
        _native.w3_gemv(bad_x.cuda(), lg["planes"], lg["scales"], None, None, bad, scratch=scratch)
        torch.cuda.synchronize()
        # a table lookup only meets the poisoned activation where one of the three plane bits of
        # that input position is set (the reference's kernel has the same property)
        touched = ((layout["planes"][300 // 128, :, :, (300 % 128) // 8] >> (300 % 8)) & 1).bool().any(dim=0)
        assert bool(torch.isnan(bad[0].cpu())[touched].all()), poison
        assert torch.equal(bad[0].cpu()[~touched], good[0].cpu()[~touched])
        assert int(scratch.view(torch.int64).abs().sum()) == 0  # status, combine words: all back to zero
        again = torch.empty_like(good)
        _native.w3_gemv(x_host.cuda(), lg["planes"], lg["scales"], None, None, again, scratch=scratch)
        assert torch.equal(again, good)


def test_push_epilogue_and_polling_reduce_on_one_device():
    """The tensor-parallel exchange protocol with both 'ranks' on one device: each rank's GEMV
    over its half of K stores (value, mark) pairs into both exchange buffers; the reduce kernel
    of each rank then finds every mark set (the stores completed earlier on the stream, so nothing
    waits on a later launch), sums in rank order, adds the residual and clears the slots."""
    from marlin_style_fluxbin_b200 import _native

    o, k, world = 512, 2048, 2
    layout, x_host = make_case(o, k, seed=91, zeros=True)
    lg, x = to_cuda(layout), x_host.cuda()
    residual = torch.randn(1, o, generator=torch.Generator().manual_seed(4)).bfloat16().cuda()
    groups = k // 128
    buffers = [torch.zeros(world * o, 2, dtype=torch.int32, device="cuda") for _ in range(world)]  # 8-byte slots
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(_native.w3_scratch_bytes(1, o, k), dtype=torch.uint8, device="cuda")
    dummy = torch.empty(1, o, device="cuda", dtype=torch.bfloat16)
    partial_reference = []
    for rank in range(world):
        lo, hi = rank * groups // world, (rank + 1) * groups // world
        shard = {"planes": lg["planes"][lo:hi].contiguous(), "scales": lg["scales"][lo:hi].contiguous(), "zeros": lg["zeros"][lo:hi].contiguous()}
        x_shard = x[:, lo * 128:hi * 128].contiguous()
        matrix = _native.w3_matrix_list([(shard["planes"], shard["scales"], shard["zeros"], dummy, None)])
        push = _native.w3_push_descriptor([buf.data_ptr() + 8 * rank * o for buf in buffers])
        _native.w3_gemv_push(x_shard, 0, None, 0.0, matrix, (hi - lo) * 128, torch.float16, push, scratch=scratch)
        own = torch.empty(1, o, device="cuda", dtype=torch.bfloat16)
        _native.w3_gemv(x_shard, shard["planes"], shard["scales"], shard["zeros"], None, own, scratch=scratch)
        partial_reference.append(own)
    outs = []
    for rank in range(world):
        out = torch.full((1, o), float("nan"), device="cuda", dtype=torch.bfloat16)
        _native.tp_reduce(buffers[rank].data_ptr(), world, residual, out, status.data_ptr())
        outs.append(out)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert torch.equal(outs[0], outs[1])  # every rank computes the same sum in the same order
    assert all(int(buf.abs().sum()) == 0 for buf in buffers)  # slots cleared for the next use
    reference, _ = oracle_outputs(layout, x_host)
    assert_parity((outs[0].float() - residual.float()).bfloat16(), reference, tol=2e-2)
    # against the two-kernel form with 16-bit partial results: the push keeps fp32 partials
    two_step = ((partial_reference[0].float() + partial_reference[1].float()).bfloat16().float() + residual.float()).bfloat16()
    assert float((outs[0].float() - two_step.float()).abs().max()) <= 2.0 ** -6 * float(two_step.float().abs().max())


@pytest.mark.parametrize("o,k,scale_dtype", ((4096, 4096, torch.float16), (1024, 1024, torch.bfloat16), (4096, 12288, torch.float16)))
def test_decoded_weight_arithmetic_with_zero_points(o, k, scale_dtype):
    """The rounding correction with per-row zero points in {3, 4} (the benchmark's draw): the result
    follows the weight dequantised in the scale's dtype, scale * (code - zero) rounded once, which is
    the oracle's dequantise-then-matmul to fp32 summation order (reference: csrc/w3_lut.cu:105-122,
    gptq_deployment.py:280-315 for the constant zero point)."""
    layout, x = make_case(o, k, seed=13, zeros=True, scale_dtype=scale_dtype)
    reference, structural = oracle_outputs(layout, x)
    lg, xg = to_cuda(layout), x.cuda()
    plain, _ = run(lg, xg, row_tile=1024)
    corrected, _ = run(lg, xg, row_tile=1024, arithmetic="decoded_bf16")
    assert_parity(corrected, reference)
    # bf16 outputs of the corrected kernel equal the rounded oracle up to fp32 summation order:
    # at most one 16-bit ulp, and only in a few rows
    want = torch.from_numpy(reference).bfloat16().float()
    got = corrected.float().cpu()
    assert float((got != want).float().mean()) <= 0.02
    torch.testing.assert_close(got, want, rtol=2.0 ** -7, atol=1e-3)
    # and it is closer to that oracle than the structural arithmetic is
    e_plain = np.abs(plain.float().cpu().numpy() - reference).mean()
    e_corr = np.abs(got.numpy() - reference).mean()
    assert e_corr < e_plain
    # repeat-exact
    assert torch.equal(run(lg, xg, row_tile=1024, arithmetic="decoded_bf16")[0], corrected)


def test_large_finite_activations_stay_inside_the_combine_range():
    """Residual-stream outliers: a few input columns carry activations in the thousands.  The
    fixed-point K-split combine must carry them like the fp32 accumulation of the reference does
    (limit: a partial sum of 2^21 in magnitude, far above what such inputs produce)."""
    layout, x = make_case(4096, 4096, seed=21, zeros=True)
    x = x.float()
    x[0, [5, 777, 2048, 4095]] = torch.tensor([3000.0, -2500.0, 1800.0, 4000.0])
    x = x.bfloat16()
    reference, _ = oracle_outputs(layout, x)
    out, _ = run(to_cuda(layout), x.cuda(), row_tile=1024)
    assert_parity(out, reference)
    layout, x = make_case(4096, 12288, seed=22, zeros=True)
    x = x.float()
    x[0, [1, 6000, 12287]] = torch.tensor([-3500.0, 2200.0, 3900.0])
    x = x.bfloat16()
    reference, _ = oracle_outputs(layout, x)
    out, _ = run(to_cuda(layout), x.cuda(), row_tile=1024)
    assert_parity(out, reference)


def test_polling_reduce_gives_up_after_its_limit():
    """One rank never delivers: the reduce kernel's bounded wait runs out (here after 5 ms), the
    status word becomes 4, the kernel returns, and the slots are left clean."""
    import time

    from marlin_style_fluxbin_b200 import _native

    n, world = 256, 2
    buffer = torch.zeros(world * n, 2, dtype=torch.int32, device="cuda")
    buffer[:n, 0] = torch.full((n,), 1.5).view(torch.int32)  # rank 0 delivered {1.5, mark}
    buffer[:n, 1] = 1
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    out = torch.zeros(1, n, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    began = time.perf_counter()
    _native.tp_reduce(buffer.data_ptr(), world, None, out, status.data_ptr(), wait_ns=5_000_000)
    torch.cuda.synchronize()
    assert time.perf_counter() - began < 2.0
    assert int(status[0]) == 4
    assert int(buffer.abs().sum()) == 0
    # the context is intact: a complete exchange on the same buffers works afterwards
    status.zero_()
    for rank in range(world):
        buffer[rank * n:(rank + 1) * n, 0] = torch.full((n,), float(rank + 1)).view(torch.int32)
        buffer[rank * n:(rank + 1) * n, 1] = 1
    _native.tp_reduce(buffer.data_ptr(), world, None, out, status.data_ptr(), wait_ns=5_000_000)
    torch.cuda.synchronize()
    assert int(status[0]) == 0 and torch.equal(out.float().cpu(), torch.full((1, n), 3.0))


def test_linears_on_the_same_activations_do_not_wait_for_one_another():
    """q/k/v-style launches behind one another on ONE activation buffer: the second and third start without
    waiting for the launch ahead (each with its own scratch), the fourth waits again; results equal the
    launches made one by one with a caller's scratch (which never take that path), eagerly and in a graph
    replayed many times back to back."""
    from marlin_style_fluxbin_b200 import _native

    shapes = ((4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096))
    cases = [to_cuda(make_case(o, k, seed=30 + i, zeros=True)[0]) for i, (o, k) in enumerate(shapes)]
    x = torch.randn(1, 4096, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    other = x.clone()
    own = torch.zeros(_native.w3_scratch_bytes(1, 4096, 4096), dtype=torch.uint8, device="cuda")
    want = []
    for lg in cases:
        out = torch.empty(1, lg["planes"].shape[2], device="cuda", dtype=torch.bfloat16)
        _native.w3_gemv(x, lg["planes"], lg["scales"], lg["zeros"], None, out, scratch=own)
        want.append(out)
    outs = [torch.full_like(w, float("nan")) for w in want]
    def stream_key():
        return (torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream)

    def launch_all():
        seen = []
        for lg, out in zip(cases, outs):
            _native.w3_gemv(x, lg["planes"], lg["scales"], lg["zeros"], None, out)
            seen.append(_native._same_input[stream_key()][1])
        return seen

    _native.w3_gemv(other, cases[0]["planes"], cases[0]["scales"], cases[0]["zeros"], None, torch.empty_like(want[0]))  # another buffer ahead
    assert launch_all() == [1, 2, 3, 1]  # launches in a row on this buffer; the fourth starts a new row
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(outs, want))
    _native.rmsnorm(x, torch.ones(4096, device="cuda", dtype=torch.bfloat16), torch.empty_like(x), 1e-6)
    assert stream_key() not in _native._same_input  # any other launch of the library forgets the buffer
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        launch_all()  # sizes this stream's three scratches
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(8):
                launch_all()
        for out in outs:
            out.fill_(float("nan"))
        for _ in range(50):
            graph.replay()
        stream.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(outs, want))
    _native.check_status(torch.device("cuda"))
