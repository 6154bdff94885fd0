"""Pins the CPU oracle to the reference: every oracle function is compared with outputs
of the reference's own Python code (fixtures from tests/golden/make_golden.py) and with
the known answers the reference's tests hold."""
import ctypes

import numpy as np
import pytest

from oracle import oracle as orc

W3_CASES = ("w3_k256_o64", "w3_k512_o256", "w3_k384_o288")


def test_boundary_word_layout_known_answer():
    # Hand-built 10-1-10-1-10 words, as in the reference's
    # tests/test_gptq_w3_planar.py:43-60.
    codes = (np.arange(32) % 8).astype(np.uint8).reshape(32, 1)
    words = [0, 0, 0]
    for i in range(10):
        words[0] |= int(codes[i, 0]) << (3 * i)
    words[0] |= (int(codes[10, 0]) & 3) << 30
    words[1] |= int(codes[10, 0]) >> 2
    for i in range(11, 21):
        words[1] |= int(codes[i, 0]) << (1 + 3 * (i - 11))
    words[1] |= (int(codes[21, 0]) & 1) << 31
    words[2] |= int(codes[21, 0]) >> 1
    for i in range(22, 32):
        words[2] |= int(codes[i, 0]) << (2 + 3 * (i - 22))
    signed = np.array([w if w < 2**31 else w - 2**32 for w in words], np.int64).astype(np.int32).reshape(3, 1)
    assert np.array_equal(orc.gptq_unpack_rows(signed), codes)
    assert np.array_equal(orc.gptq_pack_rows(codes), signed)


@pytest.mark.parametrize("case", W3_CASES)
def test_gptq_words_and_planes_bit_exact(golden, case):
    g = golden(case)
    assert np.array_equal(orc.gptq_unpack_rows(g["qweight"]), g["codes"])
    assert np.array_equal(orc.gptq_pack_rows(g["codes"]), g["qweight"])
    assert np.array_equal(orc.gptq_unpack_cols(g["qzeros"], 1), g["zeros"])
    assert np.array_equal(orc.gptq_unpack_cols(g["qzeros_v2"], 2), g["zeros"])
    assert np.array_equal(orc.gptq_pack_cols(g["zeros"]), g["qzeros_v2"])
    # desc_act canonicalisation: stable argsort of g_idx is the layout's perm.
    perm = np.argsort(g["g_idx"], kind="stable").astype(np.int16)
    assert np.array_equal(perm, g["perm"])
    assert np.array_equal(orc.w3_planes_from_codes(g["codes"], perm), g["planes"])
    assert np.array_equal(orc.w3_codes_from_planes(g["planes"], perm, True), g["codes"])
    assert np.array_equal(orc.w3_codes_from_planes(g["planes"], perm, False), g["sorted_codes"])


@pytest.mark.parametrize("case", W3_CASES)
def test_w3_dequant_bitwise_and_matvecs(golden, case):
    g = golden(case)
    restored = orc.w3_dequant(g["planes"], g["scales_bf16"], orc.BF16, None, g["perm"], orc.BF16)
    assert np.array_equal(restored, g["restored_bf16"])
    # The reference's general zero-point expression with explicit zeros gives the same bits.
    k, o = g["codes"].shape
    zeros = np.full((k // 128, o), 4, np.uint8)
    assert np.array_equal(orc.w3_dequant(g["planes"], g["scales_bf16"], orc.BF16, zeros, g["perm"], orc.BF16), restored)
    args = (g["x_bf16"], orc.BF16, g["planes"], g["scales_bf16"], orc.BF16, None, g["perm"])
    np.testing.assert_allclose(orc.w3_gemv_structural(*args), g["structural"], rtol=2e-6, atol=2e-5)
    np.testing.assert_allclose(orc.w3_gemv_dequant(*args), g["dequant_matmul"], rtol=2e-6, atol=2e-5)
    # bf16-weight-semantics oracle equals dequantise-then-matmul (reference test :105-122).
    np.testing.assert_allclose(orc.w3_gemv_dequant(*args), g["bf16_weight_semantics"], rtol=2e-6, atol=2e-5)
    np.testing.assert_allclose(
        orc.w3_gemv_lut_emulation(g["x_bf16"], orc.BF16, g["planes"], g["scales_bf16"], orc.BF16, g["perm"]),
        g["structural"], rtol=2e-6, atol=2e-5)


def test_general_zero_point_matches_direct_formula(golden):
    g = golden("w3_k256_o64")
    rng = np.random.default_rng(3)
    k, o = g["codes"].shape
    zeros = rng.integers(3, 5, size=(k // 128, o)).astype(np.uint8)
    scales = orc.unbits(g["scales_f16"], __import__("torch").float16).float().numpy()
    w = orc.w3_dequant(g["planes"], g["scales_f16"], orc.F16, zeros, g["perm"], orc.F32)
    gi = g["g_idx"].astype(np.int64)
    direct = (scales[gi].astype(np.float32) * (g["codes"].astype(np.float32) - zeros[gi])).astype(np.float16).astype(np.float32).T
    assert np.array_equal(w, direct)


def test_lut_tables_match_reference_helpers():
    ref = orc.reference_lut_lib()
    if ref is None:
        pytest.skip("reference LUT shim not built (reference tree absent at build time)")
    rng = np.random.default_rng(11)
    for _ in range(20):
        values = rng.standard_normal(8).astype(np.float32)
        table = np.empty(256, np.float32)
        ref.ref_build_unsigned_table(table.ctypes.data_as(ctypes.c_void_p), values.ctypes.data_as(ctypes.c_void_p))
        expect = np.empty(256, np.float32)
        for p in range(256):
            s = np.float32(0)
            for b in range(8):
                if (p >> b) & 1:
                    s = np.float32(s + values[b])
            expect[p] = s
        assert np.array_equal(table, expect)  # ascending-bit-order sums, bit for bit
    ref.ref_pattern.restype = ctypes.c_uint
    words = np.arange(65536, dtype=np.uint32)
    inter = np.stack((words & 255, words >> 8), -1).astype(np.uint8)
    planes = orc.bb_to_planes(inter)
    for w in (0, 1, 0x5555, 0xAAAA, 0xFFFF, 0x1234, 40000):
        assert ref.ref_pattern(w) == planes[w, 0, 0]
        assert ref.ref_pattern(w >> 1) == planes[w, 1, 0]


def test_two_base_byte_known_answer_and_roundtrip(golden):
    # K0..K3 give bit pairs 00,01,10,11 from the LSB (reference tests/test_packing.py:21-32).
    bases = np.array([[[-1, 1, -1, 1]], [[-1, -1, 1, 1]]], np.int8)
    assert int(orc.pack_two_bases(bases)[0, 0]) == 0b11100100
    g = golden("two_base_packing")
    assert np.array_equal(orc.pack_two_bases(g["bases"]), g["codes"])
    assert np.array_equal(orc.unpack_two_bases(g["codes"]), g["bases"])
    with pytest.raises(ValueError):
        orc.pack_two_bases(np.zeros((2, 3, 8), np.int8))


def test_all_65536_interleaved_patterns():
    # Reference tests/test_planar_layout.py:14-23.
    word = np.arange(65536, dtype=np.int64)
    inter = np.stack((word & 255, word >> 8), -1).astype(np.uint8)
    planes = orc.bb_to_planes(inter)
    for basis in range(2):
        expected = np.zeros_like(word)
        for k in range(8):
            expected |= ((word >> (2 * k + basis)) & 1) << k
        assert np.array_equal(planes[:, basis, 0], expected.astype(np.uint8))
    assert np.array_equal(orc.bb_from_planes(planes), inter)


@pytest.mark.parametrize("case", ("hybrid_o17_g3", "hybrid_o65_g10"))
def test_hybrid_materialise_and_structural(golden, case):
    g = golden(case)
    payload = {k.split(".", 1)[1]: v for k, v in g.items() if k.startswith("payload.")}
    assert np.array_equal(orc.bb_materialize_hybrid(payload), g["dense_f32"])
    for kind in ("inter", "planar"):
        layout = {k.split(".", 1)[1]: v for k, v in g.items() if k.startswith(kind + ".")}
        y = orc.bb_structural_f64(g["x_bf16"], orc.BF16, layout)
        np.testing.assert_allclose(y, g["structural_f64"], rtol=1e-12, atol=1e-12)
    # planar codes are the bit de-interleave of the interleaved ones
    assert np.array_equal(orc.bb_to_planes(g["inter.codes"]), g["planar.codes"])
    assert np.array_equal(orc.bb_to_planes(g["inter.sparse_codes"]), g["planar.sparse_codes"])


def test_rmsnorm_and_rope_bitwise(golden):
    g = golden("fused_modules")
    for name in ("hidden", "head"):
        out = orc.rmsnorm(g[f"rms.{name}.x"], g[f"rms.{name}.w"], orc.BF16, 1e-6)
        got = orc.unbits(out, __import__("torch").bfloat16).float().numpy()
        want = orc.unbits(g[f"rms.{name}.out"], __import__("torch").bfloat16).float().numpy()
        # one bf16 ulp: the variance is accumulated in a different order than torch's mean
        assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) <= 2**-7
        assert np.mean(out == g[f"rms.{name}.out"]) > 0.99
    assert np.array_equal(orc.rope(g["rope.q"], g["rope.cos"], g["rope.sin"], orc.BF16), g["rope.q_out"])
    assert np.array_equal(orc.rope(g["rope.k"], g["rope.cos"], g["rope.sin"], orc.BF16), g["rope.k_out"])
