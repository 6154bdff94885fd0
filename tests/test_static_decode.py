"""Static-cache decode runner: CPU contract tests and GPU graph tests (cases from the
reference's tests/test_static_decode.py and tests/test_w3_lut_adapter.py)."""
from unittest.mock import patch

import pytest
import torch
from transformers import Qwen3Config, Qwen3ForCausalLM

from marlin_style_fluxbin_b200.deployment import PackedHybridLinear
from marlin_style_fluxbin_b200.full_model_trial import compare_trace, decode_trace, packed_modules, validate_routes
from marlin_style_fluxbin_b200.static_decode import StaticDecodeSession, prepared_linears
from test_deployment import make_payload


def tiny_model(hidden=32, inter=64, heads=2, kv=1, head_dim=16):
    torch.manual_seed(17)
    cfg = Qwen3Config(vocab_size=64, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=2,
                      num_attention_heads=heads, num_key_value_heads=kv, head_dim=head_dim)
    cfg._attn_implementation = "sdpa"
    return Qwen3ForCausalLM(cfg).eval()


def test_static_matches_dynamic_full_prefix_and_masks_future_slots():
    model = tiny_model()
    ids = torch.tensor([[1, 3, 7]])
    dynamic = decode_trace(model, ids, steps=3)
    session = StaticDecodeSession(model, ids, dynamic["fed_tokens"])
    pointers = [(l.keys.data_ptr(), l.values.data_ptr()) for l in session.cache.layers]
    first = session.audit()
    torch.testing.assert_close(first["logits"], dynamic["logits"], atol=1e-6, rtol=1e-5)
    for _ in range(2):
        timing, trace = session.measure("prepared_eager")
        assert timing["wall_ms"] > 0 and timing["device_ms"] is None
        assert torch.equal(trace["logits"], first["logits"]) and trace["cache_length"] == 6
    assert pointers == [(l.keys.data_ptr(), l.values.data_ptr()) for l in session.cache.layers]
    with torch.inference_mode():
        session.reset()
        for layer in session.cache.layers:  # stale values in future slots must be masked
            layer.keys[:, :, 4:].fill_(100)
            layer.values[:, :, 4:].fill_(100)
        poisoned = session.trace(session.run())
        torch.testing.assert_close(poisoned["logits"], first["logits"], atol=0, rtol=0)
        for i in range(4):
            prefix = torch.cat((ids, dynamic["fed_tokens"][:, :i]), 1)
            expected = model(input_ids=prefix, use_cache=False).logits[:, -1, :]
            torch.testing.assert_close(first["logits"][:, i, :], expected, atol=1e-6, rtol=1e-5)
    with pytest.raises(RuntimeError, match="CUDA"):
        session.capture()
    with pytest.raises(ValueError, match="capture first"):
        session.measure("sequence_graph")
    assert compare_trace(first, dynamic, logprob_tolerance=0.05)["passed"]
    assert validate_routes({"routes": {"a": {"dense_fallback": 1, "packed_m1": 3}}}, expected_linears=1, steps=3)


def test_binding_rejects_cpu_and_cleans_up_on_partial_failure():
    modules = torch.nn.Sequential(PackedHybridLinear(make_payload(32, 1)), PackedHybridLinear(make_payload(32, 1)))
    with pytest.raises(ValueError, match="CUDA"):
        modules[0].bind_prepared_decode(torch.bfloat16)

    def partial(module, dtype):
        module._decode_binding = lambda x: x
        if module is modules[1]:
            raise RuntimeError("partial failure")

    with patch.object(PackedHybridLinear, "bind_prepared_decode", partial):
        with pytest.raises(RuntimeError, match="partial failure"):
            with prepared_linears(modules, torch.bfloat16):
                pass
    assert all(m._decode_binding is None for m in modules)
    assert len(packed_modules(modules)) == 2


@pytest.mark.gpu
def test_cuda_full_sequence_graph_matches_eager():
    model = tiny_model().cuda().to(torch.bfloat16)
    ids = torch.tensor([[1, 3, 7]], device="cuda")
    dynamic = decode_trace(model, ids, steps=3)
    session = StaticDecodeSession(model, ids, dynamic["fed_tokens"])
    expected = session.audit()
    graph = session.capture()
    assert torch.equal(expected["logits"], graph["logits"])
    for mode in ("prepared_eager", "sequence_graph", "sequence_graph"):
        _, trace = session.measure(mode)
        assert torch.equal(expected["logits"], trace["logits"])


@pytest.mark.gpu
@pytest.mark.parametrize("family", ("w3", "hybrid"))
def test_cuda_packed_model_static_graph_routes_and_fused_modules(family):
    from marlin_style_fluxbin_b200.fused_modules import fused_qwen3_modules
    from marlin_style_fluxbin_b200.gptq_deployment import convert_gptq_w3_to_planar
    from marlin_style_fluxbin_b200.qwen3 import QWEN3_LINEAR_MODULES
    from marlin_style_fluxbin_b200.w3_lut_deployment import PackedW3Linear
    from test_gptq_w3_planar import synthetic_raw

    model = tiny_model(hidden=128, inter=256, heads=4, kv=2, head_dim=32).cuda().to(torch.bfloat16)
    for layer in model.model.layers:
        for name in QWEN3_LINEAR_MODULES:
            linear = layer.get_submodule(name)
            parent, child = name.rsplit(".", 1)
            if family == "w3":
                raw, _, _ = synthetic_raw(k=linear.in_features, o=linear.out_features)
                packed = PackedW3Linear(convert_gptq_w3_to_planar(raw, qzero_format=1), fallback="dense", row_tile=256)
            else:
                packed = PackedHybridLinear(make_payload(linear.out_features, linear.in_features // 128),
                                            kernel="v5_p1024", groups_per_split=1, fallback="dense")
            setattr(layer.get_submodule(parent), child, packed.cuda())
    ids = torch.tensor([[1, 3, 7]], device="cuda")
    for fused in (False, True):
        with fused_qwen3_modules(rms_norm=fused, rope=fused):
            dynamic = decode_trace(model, ids, steps=3)
            session = StaticDecodeSession(model, ids, dynamic["fed_tokens"])
            with prepared_linears(model, torch.bfloat16):
                expected = session.audit()
                assert compare_trace(expected, dynamic, logprob_tolerance=.05)["passed"]
                assert len(expected["routes"]) == 14
                assert all(r == {"dense_fallback": 0, "packed_m1": 3} for r in expected["routes"].values())
                graph = session.capture()
                assert torch.equal(expected["logits"], graph["logits"])
                for mode in ("prepared_eager", "sequence_graph", "sequence_graph"):
                    _, trace = session.measure(mode)
                    assert torch.equal(expected["logits"], trace["logits"])
