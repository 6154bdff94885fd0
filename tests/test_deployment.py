"""Two-base binary-basis path.  CPU: lossless layout and module contract (cases from the
reference's tests/test_deployment.py, test_planar_layout.py, test_factored_reference.py).
GPU: kernels through the C ABI against the fp64 structural oracle."""
import numpy as np
import pytest
import torch
from torch import nn

from marlin_style_fluxbin_b200 import binary_global
from marlin_style_fluxbin_b200.deployment import (
    FIELDS, KERNELS, PLANAR_FORMAT, PLANAR_KERNELS, PackedHybridLinear, _from_planes, _to_planes, conversion_record,
    convert_artifact, decode_layout, m1_out, replace_block_linears, restore_artifact, workspace_shape,
)
from marlin_style_fluxbin_b200.engine_interface import M1Backend
from marlin_style_fluxbin_b200.evaluation import materialize_hybrid_s8_weight
from marlin_style_fluxbin_b200.factored_reference import structural_gate, structural_reference
from marlin_style_fluxbin_b200.packing import pack_two_bases, unpack_two_bases
from oracle import oracle as orc


def make_payload(o=7, g=3, seed=19):
    """Same recipe as the reference's fixture of that name."""
    rng = torch.Generator().manual_seed(seed)

    def signs(k):
        return pack_two_bases(torch.randint(0, 2, (2, o, k), generator=rng).mul(2).sub(1))

    return dict(zip(FIELDS, (
        signs(g * 128), torch.randn(2, o, g, generator=rng) * .1, torch.randn(2, g, 128, generator=rng),
        torch.stack([torch.randperm(128, generator=rng)[:8].sort().values for _ in range(g)]).short(),
        signs(g * 8), torch.randn(2, o, g, generator=rng) * .07, torch.randn(2, g, 8, generator=rng))))


def oracle(p, dtype):
    return materialize_hybrid_s8_weight(**p, group_size=128, columns_per_group=8, device=p["global_sign_codes"].device, output_dtype=dtype)


def test_matches_reference_fixtures(golden):
    for case in ("hybrid_o17_g3", "hybrid_o65_g10"):
        g = golden(case)
        p = {k.split(".", 1)[1]: torch.from_numpy(v) for k, v in g.items() if k.startswith("payload.")}
        for kind, kernel in (("inter", "v5"), ("planar", "v5_p1024")):
            layout = convert_artifact(p, kernel=kernel)
            for name, value in layout.items():
                assert np.array_equal(value.numpy(), g[f"{kind}.{name}"]), (kind, name)
            x = orc.unbits(g["x_bf16"], torch.bfloat16)
            torch.testing.assert_close(structural_reference(x, layout), torch.from_numpy(g["structural_f64"]), atol=1e-12, rtol=1e-12)
        assert np.array_equal(decode_layout(layout, torch.float32).numpy(), g["dense_f32"])


def test_lossless_conversion_lookup_and_independence():
    for o, g in ((1, 1), (7, 3), (17, 10)):
        p = make_payload(o, g)
        q = convert_artifact(p)
        for key, value in restore_artifact(q).items():
            assert torch.equal(p[key], value), key
        for dtype in (torch.float32, torch.float16, torch.bfloat16):
            assert torch.equal(decode_layout(q, dtype), oracle(p, dtype))
        expected = torch.full((g, 128), -1, dtype=torch.int16)
        expected.scatter_(1, p["refinement_indices"].long(), torch.arange(8, dtype=torch.int16).expand(g, 8))
        assert torch.equal(expected, q["lookup"])
        saved = q["rows"].clone()
        p["global_row_scales"].zero_()
        assert torch.equal(saved, q["rows"])


def test_all_65536_interleaved_patterns_and_planar_roundtrip():
    word = torch.arange(65536, dtype=torch.int32)
    interleaved = torch.stack((word & 255, word >> 8), dim=-1).byte()
    planes = _to_planes(interleaved)
    for basis in range(2):
        expected = torch.zeros_like(word)
        for k in range(8):
            expected |= ((word >> (2 * k + basis)) & 1) << k
        assert torch.equal(planes[:, basis, 0], expected.byte())
    assert torch.equal(interleaved, _from_planes(planes))
    p = make_payload(17, 3)
    legacy = convert_artifact(p)
    x = torch.randn(1, 384, dtype=torch.bfloat16)
    for kernel in PLANAR_KERNELS:
        layout = convert_artifact(p, kernel=kernel)
        assert layout["codes"].shape == (3, 17, 2, 16) and layout["sparse_codes"].shape == (3, 17, 2, 1)
        for field, value in restore_artifact(layout).items():
            assert torch.equal(value, p[field]), field
        assert torch.equal(structural_reference(x, legacy), structural_reference(x, layout))
        assert torch.equal(decode_layout(legacy), decode_layout(layout))
        record = conversion_record(p, layout)
        assert record["format"] == PLANAR_FORMAT and record["layout_bytes"] == conversion_record(p, legacy)["layout_bytes"]
        backend = M1Backend(kernel=kernel)
        assert backend.contract.format == PLANAR_FORMAT and backend.contract.arithmetic == "factored_fp32_v1"
        assert backend.convert(p)["codes"].ndim == 4
    assert M1Backend(kernel="v4_late").workspace_shape(17, 384) == (3 * 272 + 17,)
    assert workspace_shape(17, 384, 4, kernel="v4") == (3 * 272 + 17,) and workspace_shape(17, 384, 4) == (1, 17)


def test_fail_closed_payload_contract():
    for field, mutate in (("refinement_indices", lambda x: x.fill_(128)), ("refinement_indices", lambda x: x.zero_()),
                          ("global_row_scales", lambda x: x.fill_(float("nan"))), ("global_column_scales", lambda x: x.half()),
                          ("refinement_sign_codes", lambda x: x.long())):
        p = make_payload()
        p[field] = mutate(p[field])
        with pytest.raises(ValueError):
            convert_artifact(p)
    with pytest.raises(ValueError):
        convert_artifact({})
    with pytest.raises(ValueError):
        convert_artifact(make_payload(), kernel="unknown")
    assert set(KERNELS) >= {"v1", "v3", "v4_late", "v5", "v5_p1024"}


def test_module_fallback_shape_and_block_adapter():
    from marlin_style_fluxbin_b200.qwen3 import QWEN3_LINEAR_MODULES

    p = make_payload()
    x = torch.randn(1, 2, 384)
    with torch.inference_mode():
        with pytest.raises(ValueError):
            PackedHybridLinear(p)(x)
        layer = PackedHybridLinear(p, fallback="dense")
        torch.testing.assert_close(layer(x), torch.nn.functional.linear(x, oracle(p, x.dtype)))
        assert layer.last_route == "dense_fallback"
    with pytest.raises(RuntimeError):
        layer(x)
    layer.half()
    with torch.inference_mode(), pytest.raises(ValueError):
        layer(x.half())
    with pytest.raises(ValueError, match="CUDA"):
        PackedHybridLinear(make_payload(32, 1)).bind_prepared_decode(torch.bfloat16)
    block = nn.Module()
    block.self_attn, block.mlp, payload = nn.Module(), nn.Module(), {}
    for name in QWEN3_LINEAR_MODULES:
        parent, attr = name.split(".")
        setattr(block.get_submodule(parent), attr, nn.Linear(128, 7, bias=False))
        payload.update({name + "." + k: v for k, v in make_payload(7, 1).items()})
    broken = dict(payload)
    broken.pop(next(iter(broken)))
    with pytest.raises(ValueError):
        replace_block_linears(block, broken)
    assert all(isinstance(block.get_submodule(n), nn.Linear) for n in QWEN3_LINEAR_MODULES)
    assert len(replace_block_linears(block, payload, fallback="dense")) == 7
    with torch.inference_mode():
        assert tuple(block.self_attn.q_proj(torch.zeros(1, 128)).shape) == (1, 7)


def test_two_base_packing_known_answer(golden):
    bases = torch.tensor([[[-1, 1, -1, 1]], [[-1, -1, 1, 1]]], dtype=torch.int8)
    assert int(pack_two_bases(bases).item()) == 0b11100100
    g = golden("two_base_packing")
    assert np.array_equal(pack_two_bases(torch.from_numpy(g["bases"])).numpy(), g["codes"])
    assert np.array_equal(unpack_two_bases(torch.from_numpy(g["codes"])).numpy(), g["bases"])
    with pytest.raises(ValueError):
        pack_two_bases(torch.zeros(2, 3, 8, dtype=torch.int8))


def make_global_case(o, k, seed=0, n_sal=32):
    """Benchmark configuration: Bernoulli(0.5) signs, |N(0,0.02)| fp16 scales, 32 salient bf16 columns ~ N(0,0.05)."""
    gen = torch.Generator().manual_seed(seed)
    bases = torch.randint(0, 2, (2, o, k), generator=gen, dtype=torch.int8) * 2 - 1
    r = (torch.randn(2, o, generator=gen) * 0.02).abs().half()
    c = (torch.randn(2, k, generator=gen) * 0.02).abs().half()
    idx = torch.randperm(k, generator=gen)[:n_sal].sort().values.int()
    sal = (torch.randn(o, n_sal, generator=gen) * 0.05).bfloat16()
    x = torch.randn(1, k, generator=gen).bfloat16()
    return binary_global.make_layout(bases, r, c, idx, sal), bases, x


def test_global_layout_roundtrip_and_oracle_agreement():
    layout, bases, x = make_global_case(40, 256, seed=4, n_sal=8)
    assert torch.equal(binary_global.unpack_sign_planes(layout["codes"]), bases)
    # plane byte order: [base 0: 16 bytes][base 1: 16 bytes], bit j of byte c = input 8c+j
    assert int(layout["codes"][1, 5, 1, 3]) == sum(int(bases[1, 5, 128 + 24 + j] > 0) << j for j in range(8))
    sign_planes = np.ascontiguousarray(np.packbits((bases.numpy() > 0), axis=-1, bitorder="little"))  # [2,O,K/8]
    dense = orc.bb_global_materialize(sign_planes, orc.bits(layout["row_scales"]), orc.bits(layout["column_scales"]),
                                      layout["salient_indices"].numpy(), orc.bits(layout["salient_values"]))
    assert np.array_equal(binary_global.materialize(layout).numpy(), dense)
    y = orc.bb_global_gemv_f64(orc.bits(x), orc.BF16, sign_planes, orc.bits(layout["row_scales"]), orc.bits(layout["column_scales"]),
                               layout["salient_indices"].numpy(), orc.bits(layout["salient_values"]))
    np.testing.assert_allclose(y, (x.double() @ binary_global.materialize(layout).double().T).numpy(), rtol=1e-6, atol=1e-9)


# ------------------------------------------------------------------------------- GPU
def _structural(x, layout):
    """fp64 structural oracle (C) on CPU copies of a kernel layout."""
    cpu = {k: v.cpu().numpy() for k, v in layout.items()}
    return torch.from_numpy(orc.bb_structural_f64(orc.bits(x), orc.tag(x.dtype), cpu))


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ("v5", "v5_p1024", "v1", "v4_late"))
def test_kernel_reference_tail_split_stream_graph(kernel):
    for o, g in ((1, 1), (17, 3), (65, 10), (1025, 2)):
        for dtype in (torch.bfloat16, torch.float16):
            cpu_layout = convert_artifact(make_payload(o, g), kernel=kernel)
            layout = {k: v.cuda() for k, v in cpu_layout.items()}
            for basis in (True, False):
                x = torch.randn(1, g * 128, dtype=dtype, generator=torch.Generator().manual_seed(o + g))
                if basis:  # a basis vector on a refined column catches index-mapping errors
                    x.zero_()
                    x[0, int(cpu_layout["indices"][0, 0])] = 1
                ref = _structural(x, cpu_layout)
                assert torch.equal(ref, structural_reference(x, cpu_layout)) or torch.allclose(ref, structural_reference(x, cpu_layout), atol=1e-12, rtol=1e-12)
                xg = x.cuda()
                for gps in (1, 4, 1024):
                    w = torch.full(workspace_shape(o, g * 128, gps, kernel=kernel), float("nan"), device="cuda")
                    y = torch.empty(1, o, device="cuda", dtype=dtype)

                    def run():
                        m1_out(xg, layout, y, w, groups_per_split=gps, kernel=kernel)

                    run()
                    assert structural_gate(y.cpu(), ref)["passed"], (kernel, o, g, dtype, basis, gps)
                    saved = y.clone()
                    stream = torch.cuda.Stream()
                    stream.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(stream):
                        run()
                        run()
                    torch.cuda.current_stream().wait_stream(stream)
                    assert torch.equal(saved, y)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        run()
                    y.fill_(float("nan"))
                    graph.replay()
                    torch.cuda.synchronize()
                    assert torch.equal(saved, y)
    with pytest.raises(RuntimeError):
        m1_out(xg.expand(2, -1).contiguous(), layout, y, w, groups_per_split=1024, kernel=kernel)


@pytest.mark.gpu
def test_dense_oracle_tolerance_and_interleaved_equals_planar():
    for o, g in ((7, 3), (129, 5), (512, 8)):
        p = make_payload(o, g)
        x = torch.randn(1, g * 128, generator=torch.Generator().manual_seed(5)).bfloat16()
        outs = []
        for kernel in ("v5", "v5_p512"):
            layout = {k: v.cuda() for k, v in convert_artifact(p, kernel=kernel).items()}
            y = torch.empty(1, o, device="cuda", dtype=torch.bfloat16)
            m1_out(x.cuda(), layout, y, torch.empty(workspace_shape(o, g * 128, 8, kernel=kernel), device="cuda"), kernel=kernel)
            outs.append(y)
        ref = torch.nn.functional.linear(x.float(), oracle(p, torch.float32))
        torch.testing.assert_close(outs[0].float().cpu(), ref, atol=.02, rtol=.02)
        assert float((outs[0].float() - outs[1].float()).abs().max()) <= 2 ** -7 * float(ref.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("o,k", ((4096, 4096), (1024, 4096), (12288, 4096), (4096, 12288), (96, 256)))
def test_global_two_base_kernel(o, k):
    layout, bases, x = make_global_case(o, k, seed=o + k)
    sign_planes = np.ascontiguousarray(np.packbits((bases.numpy() > 0), axis=-1, bitorder="little"))
    ref = orc.bb_global_gemv_f64(orc.bits(x), orc.BF16, sign_planes, orc.bits(layout["row_scales"]), orc.bits(layout["column_scales"]),
                                 layout["salient_indices"].numpy(), orc.bits(layout["salient_values"]))
    lg = {name: value.cuda() for name, value in layout.items()}
    out = torch.full((1, o), float("nan"), device="cuda", dtype=torch.bfloat16)
    binary_global.global_two_base_m1_out(x.cuda(), lg, out)
    got = out.float().cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2  # the stated tolerance for 16-bit outputs
    assert structural_gate(out.cpu(), torch.from_numpy(ref))["passed"]
    saved = out.clone()
    binary_global.global_two_base_m1_out(x.cuda(), lg, out)
    assert torch.equal(saved, out)
    # scaling by two is exact in every fp32 step; the combine over groups is in fixed point (steps
    # of 2^-26), which can move a 16-bit rounding boundary in a rare row, by one ulp
    doubled = torch.empty_like(out)
    binary_global.global_two_base_m1_out((x * 2).cuda(), lg, doubled)
    twice = out.float() * 2
    assert float((doubled.float() != twice).float().mean()) <= 5e-3
    assert float((doubled.float() - twice).abs().max()) <= float(twice.abs().max()) * 2.0 ** -7


@pytest.mark.gpu
def test_two_base_kernels_carry_large_finite_activations():
    """Residual-stream outliers (a few activations in the thousands) must go through the fixed-point
    combine over the groups like the reference's fp32 accumulation carries them: both scale
    conventions against their fp64 oracles."""
    o, k = 1024, 2048
    layout, bases, x = make_global_case(o, k, seed=5)
    x = x.float()
    x[0, [3, 700, 2047]] = torch.tensor([3000.0, -2200.0, 3800.0])
    x = x.bfloat16()
    sign_planes = np.ascontiguousarray(np.packbits((bases.numpy() > 0), axis=-1, bitorder="little"))
    ref = orc.bb_global_gemv_f64(orc.bits(x), orc.BF16, sign_planes, orc.bits(layout["row_scales"]), orc.bits(layout["column_scales"]),
                                 layout["salient_indices"].numpy(), orc.bits(layout["salient_values"]))
    out = torch.full((1, o), float("nan"), device="cuda", dtype=torch.bfloat16)
    binary_global.global_two_base_m1_out(x.cuda(), {name: value.cuda() for name, value in layout.items()}, out)
    got = out.float().cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all() and np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2
    # the reference's hybrid payload (per-group fp32 scales of the size its quantiser produces)
    payload = make_payload(256, 4, seed=11)
    kernel_layout = convert_artifact(payload, kernel="v5")
    xh = torch.randn(1, 512, generator=torch.Generator().manual_seed(3))
    xh[0, [0, 130, 511]] = torch.tensor([2500.0, -3100.0, 1900.0])
    xh = xh.bfloat16()
    want = _structural(xh, kernel_layout).numpy().astype(np.float64).reshape(1, -1)
    outh = torch.full((1, 256), float("nan"), device="cuda", dtype=torch.bfloat16)
    workspace = torch.empty(workspace_shape(256, 512, 1, kernel="v5"), device="cuda")
    m1_out(xh.cuda(), {name: value.cuda() for name, value in kernel_layout.items()}, outh, workspace, groups_per_split=1, kernel="v5")
    goth = outh.float().cpu().numpy().astype(np.float64)
    assert np.isfinite(goth).all() and np.abs(goth - want).max() / np.abs(want).max() <= 1e-2


@pytest.mark.gpu
def test_prepared_hybrid_binding_and_graph_replay():
    from marlin_style_fluxbin_b200.static_decode import prepared_linears

    for kernel in ("v3", "v4_late", "v5_p1024"):
        with torch.inference_mode():
            module = PackedHybridLinear(make_payload(128, 2), kernel=kernel, groups_per_split=1).cuda()
            model = torch.nn.Sequential(module)
            x = torch.randn(1, 1, 256, device="cuda", dtype=torch.bfloat16)
            expected = module(x).clone()
            with prepared_linears(model, torch.bfloat16):
                module._decode_audit = True
                module.route_counts = {"packed_m1": 0, "dense_fallback": 0}
                actual = module(x)
                torch.testing.assert_close(actual, expected, atol=0, rtol=0)
                assert module.route_counts["packed_m1"] == 1
                pointer = actual.data_ptr()
                module._decode_audit = False
                stream = torch.cuda.Stream()
                stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(stream):
                    for _ in range(3):
                        module(x)
                torch.cuda.current_stream().wait_stream(stream)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    output = module(x)
                x.mul_(.5)
                graph.replay()
                torch.cuda.synchronize()
                result = output.clone()
                assert output.data_ptr() == pointer
                with pytest.raises(ValueError):
                    module(x.view(1, 256))
            torch.testing.assert_close(result, module(x), atol=0, rtol=0)
            assert module._decode_output is None
