"""Fused RMSNorm / RoPE: host contract on CPU, kernels against the oracle on the GPU.
Cases follow the reference's tests/test_fused_modules.py."""
import numpy as np
import pytest
import torch

from marlin_style_fluxbin_b200.fused_modules import (
    fused_apply_rotary_pos_emb, fused_qwen3_modules, fused_rms_norm, rms_norm_reference,
)
from oracle import oracle as orc


def rope_inputs(dtype=torch.bfloat16, device="cpu"):
    torch.manual_seed(20260914)
    shapes = ((1, 32, 1, 128), (1, 8, 1, 128), (1, 1, 128), (1, 1, 128))
    return tuple(torch.randn(s).to(dtype).to(device) for s in shapes)


def test_reference_math_is_bit_exact_with_stock_and_fixture(golden):
    from transformers.models.qwen3 import modeling_qwen3

    for dtype in (torch.float32, torch.bfloat16):
        torch.manual_seed(20260914)
        norm = modeling_qwen3.Qwen3RMSNorm(4096).to(dtype)
        hidden = torch.randn(1, 1, 4096, dtype=dtype)
        assert torch.equal(rms_norm_reference(hidden, norm.weight, norm.variance_epsilon), modeling_qwen3.Qwen3RMSNorm.forward(norm, hidden))
    g = golden("fused_modules")
    x, w = orc.unbits(g["rms.hidden.x"], torch.bfloat16), orc.unbits(g["rms.hidden.w"], torch.bfloat16)
    assert np.array_equal(orc.bits(rms_norm_reference(x, w, 1e-6)), g["rms.hidden.out"])
    assert np.array_equal(orc.bits(fused_rms_norm(x, w, 1e-6)), g["rms.hidden.out"])  # CPU tensors: same math


def test_rope_matches_stock_and_rejects_mismatch(golden):
    from transformers.models.qwen3 import modeling_qwen3

    for dtype, limit in ((torch.float32, 2e-6), (torch.bfloat16, 2 ** -7)):
        q, k, cos, sin = rope_inputs(dtype)
        for got, want in zip(fused_apply_rotary_pos_emb(q, k, cos, sin), modeling_qwen3.apply_rotary_pos_emb(q, k, cos, sin)):
            assert got.shape == want.shape and got.dtype == want.dtype
            assert float((got.float() - want.float()).abs().max()) <= limit * float(want.float().abs().max())
    g = golden("fused_modules")
    args = [orc.unbits(g[f"rope.{n}"], torch.bfloat16) for n in ("q", "k", "cos", "sin")]
    q_out, k_out = fused_apply_rotary_pos_emb(*args)
    assert np.array_equal(orc.bits(q_out), g["rope.q_out"]) and np.array_equal(orc.bits(k_out), g["rope.k_out"])
    q, k, cos, sin = rope_inputs()
    with pytest.raises(ValueError):
        fused_apply_rotary_pos_emb(q, k.to(torch.float32), cos, sin)
    with pytest.raises(ValueError):
        fused_apply_rotary_pos_emb(q, k[..., :64], cos, sin)


def test_patches_are_applied_and_restored():
    from transformers.models.qwen3 import modeling_qwen3

    forward, rope = modeling_qwen3.Qwen3RMSNorm.forward, modeling_qwen3.apply_rotary_pos_emb
    with fused_qwen3_modules() as applied:
        assert applied == {"rms_norm": True, "rope": True}
        assert modeling_qwen3.Qwen3RMSNorm.forward is not forward
        assert modeling_qwen3.apply_rotary_pos_emb is fused_apply_rotary_pos_emb
    assert modeling_qwen3.Qwen3RMSNorm.forward is forward and modeling_qwen3.apply_rotary_pos_emb is rope
    with fused_qwen3_modules(rms_norm=False) as applied:
        assert applied == {"rms_norm": False, "rope": True} and modeling_qwen3.Qwen3RMSNorm.forward is forward
    with pytest.raises(RuntimeError):
        with fused_qwen3_modules():
            raise RuntimeError("boom")
    assert modeling_qwen3.Qwen3RMSNorm.forward is forward and modeling_qwen3.apply_rotary_pos_emb is rope


def test_tiny_model_decode_unchanged_on_cpu():
    from transformers import Qwen3Config
    from transformers.models.qwen3 import modeling_qwen3

    config = Qwen3Config(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=8,
                         num_key_value_heads=2, head_dim=16, vocab_size=256, max_position_embeddings=64,
                         attn_implementation="sdpa")
    torch.manual_seed(20260914)
    model = modeling_qwen3.Qwen3ForCausalLM(config).eval()
    with torch.inference_mode():
        stock = model(input_ids=torch.tensor([[1, 2, 3, 4]])).logits
        with fused_qwen3_modules():
            fused = model(input_ids=torch.tensor([[1, 2, 3, 4]])).logits
    torch.testing.assert_close(fused, stock, atol=2e-5, rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
def test_rmsnorm_kernel_against_oracle(dtype):
    torch.manual_seed(3)
    for rows, dim in ((1, 4096), (40, 128), (3, 5120), (5, 96)):
        x = (torch.randn(rows, dim) * 1.7).to(dtype)
        w = (1 + 0.1 * torch.randn(dim)).to(dtype)
        want = orc.unbits(orc.rmsnorm(orc.bits(x), orc.bits(w), orc.tag(dtype), 1e-6), dtype).float()
        with torch.inference_mode():
            got = fused_rms_norm(x.cuda(), w.cuda(), 1e-6).float().cpu()
        ulp = 2 ** -7 if dtype == torch.bfloat16 else 2 ** -10
        assert float(((got - want).abs() / want.abs().clamp_min(1e-3)).max()) <= ulp  # at most one ulp apart
        assert float((got == want).float().mean()) > 0.98


@pytest.mark.gpu
def test_rope_kernel_bit_exact_with_oracle_and_fixture(golden):
    g = golden("fused_modules")
    args = [orc.unbits(g[f"rope.{n}"], torch.bfloat16).cuda() for n in ("q", "k", "cos", "sin")]
    with torch.inference_mode():
        q_out, k_out = fused_apply_rotary_pos_emb(*args)
    assert np.array_equal(orc.bits(q_out), g["rope.q_out"]) and np.array_equal(orc.bits(k_out), g["rope.k_out"])
    for dtype in (torch.float16, torch.bfloat16):
        q, k, cos, sin = rope_inputs(dtype)
        with torch.inference_mode():
            got_q, got_k = fused_apply_rotary_pos_emb(q.cuda(), k.cuda(), cos.cuda(), sin.cuda())
        assert np.array_equal(orc.bits(got_q), orc.rope(orc.bits(q), orc.bits(cos), orc.bits(sin), orc.tag(dtype)))
        assert np.array_equal(orc.bits(got_k), orc.rope(orc.bits(k), orc.bits(cos), orc.bits(sin), orc.tag(dtype)))


@pytest.mark.gpu
def test_patched_tiny_model_decode_on_gpu_matches_stock():
    from transformers import Qwen3Config
    from transformers.models.qwen3 import modeling_qwen3

    config = Qwen3Config(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=8,
                         num_key_value_heads=2, head_dim=16, vocab_size=256, max_position_embeddings=64,
                         attn_implementation="sdpa")
    torch.manual_seed(20260914)
    model = modeling_qwen3.Qwen3ForCausalLM(config).eval().cuda().to(torch.bfloat16)
    ids = torch.tensor([[1, 2, 3, 4]], device="cuda")
    with torch.inference_mode():
        cache = model(input_ids=ids, use_cache=True).past_key_values
        import copy

        stock = model(input_ids=torch.tensor([[5]], device="cuda"), past_key_values=copy.deepcopy(cache), use_cache=True).logits
        with fused_qwen3_modules():
            fused = model(input_ids=torch.tensor([[5]], device="cuda"), past_key_values=copy.deepcopy(cache), use_cache=True).logits
    assert float((fused.float() - stock.float()).abs().max()) <= 0.02 * float(stock.float().abs().max())
