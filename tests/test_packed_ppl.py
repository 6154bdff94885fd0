"""Teacher-forced single-token perplexity protocol (scoring core of the reference's
scripts/run_qwen3_8b_w3_packed_m1_ppl.py): on CPU the cached one-token scoring must equal the
full-sequence cross entropy of the same model; on a GPU a model whose Linears were swapped for
packed W3 modules is scored through the packed kernels and lands within the quantisation-free
distance of its dense (dequantised) twin."""
import math

import pytest
import torch
from transformers import Qwen3Config, Qwen3ForCausalLM

from marlin_style_fluxbin_b200.packed_ppl import comparison, score_m1_ppl


def tiny_model(hidden=128, inter=256):
    torch.manual_seed(23)
    cfg = Qwen3Config(vocab_size=96, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=2,
                      num_attention_heads=2, num_key_value_heads=1, head_dim=64)
    cfg._attn_implementation = "sdpa"
    return Qwen3ForCausalLM(cfg).eval()


BLOCKS = [[5, 9, 2, 77, 31, 8, 40, 3], [11, 12, 13, 14, 15, 80], [1, 95]]


def test_cached_single_token_scoring_equals_full_sequence_cross_entropy():
    model = tiny_model()
    report = score_m1_ppl(model, BLOCKS, arm="original_bf16", device="cpu", expected_packed_linears=0, progress_every=0)
    total = 0.0
    with torch.inference_mode():
        for block in BLOCKS:
            ids = torch.tensor([block])
            logits = model(input_ids=ids).logits[0, :-1].float()
            total += float(torch.nn.functional.cross_entropy(logits, ids[0, 1:], reduction="sum").double())
    assert report["status"] == "completed" and report["scored_transition_count"] == sum(len(b) - 1 for b in BLOCKS)
    assert math.isclose(report["total_nll"], total, rel_tol=1e-5)
    assert math.isclose(report["perplexity"], math.exp(total / report["scored_transition_count"]), rel_tol=1e-5)
    assert report["packed_route_smoke"] is None and len(report["block_nll_sha256"]) == len(BLOCKS)
    with pytest.raises(RuntimeError, match="count drifted"):
        score_m1_ppl(model, BLOCKS, arm="x", device="cpu", expected_packed_linears=3, progress_every=0)
    with pytest.raises(ValueError, match="two tokens"):
        score_m1_ppl(model, [[1]], arm="x", device="cpu", expected_packed_linears=0, progress_every=0)
    assert comparison(report, report)["ppl_delta"] == 0.0


@pytest.mark.gpu
def test_packed_model_is_scored_through_the_packed_kernels():
    from marlin_style_fluxbin_b200.gptq_deployment import restore_planar_w3
    from marlin_style_fluxbin_b200.qwen3 import QWEN3_LINEAR_MODULES
    from marlin_style_fluxbin_b200.w3_lut_deployment import PackedW3Linear

    dense, packed = tiny_model().bfloat16().cuda(), tiny_model().bfloat16().cuda()
    gen = torch.Generator().manual_seed(5)
    for layer_dense, layer_packed in zip(dense.model.layers, packed.model.layers):
        for name in QWEN3_LINEAR_MODULES:
            linear = layer_dense.get_submodule(name)
            o, k = linear.out_features, linear.in_features
            layout = {"planes": torch.randint(0, 256, (k // 128, 3, o, 16), generator=gen, dtype=torch.uint8),
                      "scales": (torch.rand(k // 128, o, generator=gen) * 0.03 + 0.01).bfloat16(),
                      "perm": torch.arange(k, dtype=torch.int16)}
            linear.weight.data.copy_(restore_planar_w3(layout, dtype=torch.bfloat16))
            parent, leaf = name.rsplit(".", 1)
            setattr(layer_packed.get_submodule(parent), leaf, PackedW3Linear(layout, fallback="error", row_tile=256).cuda())
    with torch.inference_mode():
        base = score_m1_ppl(dense, BLOCKS, arm="decoded_w3_bf16", device="cuda", expected_packed_linears=0, progress_every=0)
        ours = score_m1_ppl(packed, BLOCKS, arm="packed_w3_inline", device="cuda", expected_packed_linears=14, progress_every=0)
    assert ours["packed_route_smoke"] == {"passed": True, "linear_count": 14, "calls_per_linear": 1}
    assert ours["metrics_valid"] and abs(comparison(ours, base)["ppl_relative_percent"]) < 2.0
