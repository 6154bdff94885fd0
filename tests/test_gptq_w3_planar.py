"""Host-side W3 layout: bit-exact against reference-generated fixtures and the reference's
own test recipes (its tests/test_gptq_w3_planar.py)."""
import numpy as np
import pytest
import torch

from marlin_style_fluxbin_b200.gptq_deployment import (
    FORMAT, GENERAL_FORMAT, bf16_weight_semantics_w3_matvec, convert_gptq_w3_to_planar,
    decode_planar_w3_codes, inspect_gptq_checkpoint, layout_storage, pack_gptq_w3_codes,
    restore_planar_w3, structural_w3_matvec, unpack_gptq_w3_qweight, unpack_gptq_w3_qzeros,
    validate_planar_w3,
)
from oracle import oracle as orc


def synthetic_raw(*, k=256, o=64, seed=20260916, zero=4):
    """Same recipe as the reference's fixture of that name: uniform codes, fp16 scales in
    [0.001, 0.126), activation-order (desc_act) g_idx."""
    gen = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 8, (k, o), generator=gen, dtype=torch.uint8)
    groups = k // 128
    zeros = torch.full((groups, o), zero, dtype=torch.uint8) if isinstance(zero, int) else zero
    scales = (torch.rand((groups, o), generator=gen) * 0.125 + 0.001).half()
    order = torch.randperm(k, generator=gen)
    g_idx = torch.empty(k, dtype=torch.int32)
    g_idx[order] = torch.arange(groups, dtype=torch.int32).repeat_interleave(128)
    raw = {
        "qweight": pack_gptq_w3_codes(codes),
        "qzeros": pack_gptq_w3_codes(((zeros.to(torch.int16) - 1) & 7).to(torch.uint8), packed_axis=1),
        "scales": scales,
        "g_idx": g_idx,
    }
    return raw, codes, zeros


def raw_from_golden(g):
    return {"qweight": torch.from_numpy(g["qweight"]), "qzeros": torch.from_numpy(g["qzeros"]),
            "scales": orc.unbits(g["scales_f16"], torch.float16), "g_idx": torch.from_numpy(g["g_idx"])}


@pytest.mark.parametrize("case", ("w3_k256_o64", "w3_k512_o256", "w3_k384_o288"))
def test_matches_reference_fixtures_bitwise(golden, case):
    g = golden(case)
    raw = raw_from_golden(g)
    assert np.array_equal(unpack_gptq_w3_qweight(raw["qweight"]).numpy(), g["codes"])
    assert np.array_equal(pack_gptq_w3_codes(torch.from_numpy(g["codes"])).numpy(), g["qweight"])
    assert np.array_equal(unpack_gptq_w3_qzeros(raw["qzeros"], qzero_format=1).numpy(), g["zeros"])
    assert np.array_equal(unpack_gptq_w3_qzeros(torch.from_numpy(g["qzeros_v2"]), qzero_format=2).numpy(), g["zeros"])
    assert np.array_equal(pack_gptq_w3_codes(torch.from_numpy(g["zeros"]), packed_axis=1).numpy(), g["qzeros_v2"])
    layout = convert_gptq_w3_to_planar(raw, qzero_format=1)
    assert np.array_equal(layout["planes"].numpy(), g["planes"])
    assert np.array_equal(orc.bits(layout["scales"]), g["scales_bf16"])
    assert np.array_equal(layout["perm"].numpy(), g["perm"])
    assert np.array_equal(decode_planar_w3_codes(layout).numpy(), g["codes"])
    assert np.array_equal(decode_planar_w3_codes(layout, original_order=False).numpy(), g["sorted_codes"])
    assert np.array_equal(orc.bits(restore_planar_w3(layout)), g["restored_bf16"])
    x = orc.unbits(g["x_bf16"], torch.bfloat16)
    torch.testing.assert_close(structural_w3_matvec(x, layout), torch.from_numpy(g["structural"]), rtol=2e-6, atol=2e-5)
    torch.testing.assert_close(bf16_weight_semantics_w3_matvec(x, layout), torch.from_numpy(g["bf16_weight_semantics"]), rtol=2e-6, atol=2e-5)


def test_boundary_word_layout_built_by_hand():
    codes = (torch.arange(32, dtype=torch.uint8) % 8).reshape(32, 1)
    words = [0, 0, 0]
    for i in range(32):
        for bit in range(3):  # the 96-bit little-endian stream view
            pos = 3 * i + bit
            words[pos // 32] |= ((int(codes[i]) >> bit) & 1) << (pos % 32)
    signed = torch.tensor([w if w < 2**31 else w - 2**32 for w in words], dtype=torch.int32).reshape(3, 1)
    assert torch.equal(unpack_gptq_w3_qweight(signed), codes)
    assert torch.equal(pack_gptq_w3_codes(codes), signed)


def test_canonical_pack_unpack_and_desc_act():
    raw, codes, zeros = synthetic_raw()
    assert torch.equal(unpack_gptq_w3_qweight(raw["qweight"]), codes)
    assert torch.equal(unpack_gptq_w3_qzeros(raw["qzeros"], qzero_format=1), zeros)
    facts = inspect_gptq_checkpoint(raw, qzero_format=1)
    assert facts["decoded_zero_unique"] == [4] and not facts["permutation_identity"]
    layout = convert_gptq_w3_to_planar(raw, qzero_format=1)
    assert set(layout) == {"planes", "scales", "perm"}
    assert layout["perm"].dtype == torch.int16 and layout["scales"].dtype == torch.bfloat16
    assert torch.equal(layout["scales"], raw["scales"].to(torch.bfloat16))
    assert torch.equal(decode_planar_w3_codes(layout), codes)


def test_bf16_restore_matches_gptq_semantics_bitwise():
    raw, codes, zeros = synthetic_raw()
    layout = convert_gptq_w3_to_planar(raw, qzero_format=1)
    gi = raw["g_idx"].long()
    expected = (raw["scales"].to(torch.bfloat16)[gi] * (codes.to(torch.int16) - zeros[gi])).T.contiguous()
    assert torch.equal(restore_planar_w3(layout), expected)


def test_structural_and_corrected_matvecs():
    raw, codes, zeros = synthetic_raw(k=512, o=256, seed=17)
    layout = convert_gptq_w3_to_planar(raw, qzero_format=1)
    x = torch.randn(1, 512, generator=torch.Generator().manual_seed(23), dtype=torch.bfloat16)
    gi = raw["g_idx"].long()
    direct = torch.sum(x.float().T * raw["scales"].to(torch.bfloat16)[gi].float() * (codes.to(torch.int16) - zeros[gi]).float(), dim=0).unsqueeze(0)
    torch.testing.assert_close(structural_w3_matvec(x, layout), direct, rtol=2e-6, atol=2e-5)
    dense = torch.nn.functional.linear(x.float(), restore_planar_w3(layout).float())
    assert torch.equal(bf16_weight_semantics_w3_matvec(x, layout).bfloat16(), dense.bfloat16())
    assert float((structural_w3_matvec(x, layout) - dense).abs().max()) > 0.0


def test_storage_and_validation_contract():
    raw, _, _ = synthetic_raw()
    layout = convert_gptq_w3_to_planar(raw, qzero_format=1)
    record = layout_storage(layout)
    expected = 3 * 256 * 64 // 8 + 2 * 64 * 2 + 2 * 256
    assert record["format"] == FORMAT and record["total_bytes"] == expected
    assert record["bits_per_weight"] == pytest.approx(expected * 8 / (256 * 64))
    broken = dict(layout, perm=torch.zeros_like(layout["perm"]))
    with pytest.raises(ValueError, match="bijection"):
        validate_planar_w3(broken)
    assert validate_planar_w3(broken, check_values=False) == (64, 256)
    with pytest.raises(ValueError):
        validate_planar_w3({"planes": layout["planes"]})


def test_zero_points_default_rejected_general_accepted():
    raw, codes, _ = synthetic_raw(zero=3)
    with pytest.raises(ValueError, match="requires decoded zero=4"):
        convert_gptq_w3_to_planar(raw, qzero_format=1)
    gen = torch.Generator().manual_seed(5)
    zeros = torch.randint(3, 5, (2, 64), generator=gen, dtype=torch.uint8)
    raw, codes, zeros = synthetic_raw(zero=zeros)
    layout = convert_gptq_w3_to_planar(raw, qzero_format=1, general=True)
    assert set(layout) == {"planes", "scales", "perm", "zeros"} and layout["scales"].dtype == torch.float16
    assert torch.equal(layout["zeros"], zeros)
    assert layout_storage(layout)["format"] == GENERAL_FORMAT
    gi = raw["g_idx"].long()
    expected = (raw["scales"][gi] * (codes.to(torch.int16) - zeros[gi])).T.contiguous()
    assert torch.equal(restore_planar_w3(layout, dtype=torch.float16), expected)
    # the oracle agrees bit for bit on the general form
    w = orc.w3_dequant(layout["planes"].numpy(), orc.bits(layout["scales"]), orc.F16, layout["zeros"].numpy(), layout["perm"].numpy(), orc.F16)
    assert np.array_equal(w, orc.bits(expected))
    x = torch.randn(1, 256, generator=gen).bfloat16()
    want = orc.w3_gemv_structural(orc.bits(x), orc.BF16, layout["planes"].numpy(), orc.bits(layout["scales"]), orc.F16, layout["zeros"].numpy(), layout["perm"].numpy())
    np.testing.assert_allclose(structural_w3_matvec(x, layout).numpy(), want, rtol=2e-6, atol=2e-5)
