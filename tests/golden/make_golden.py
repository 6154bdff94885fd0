"""Regenerates the golden fixtures in this folder by running the REFERENCE project's own
Python code (its packing, layout, dequantisation and reference-math functions) on small
seeded inputs.  Needs the reference tree; run it where that tree is mounted:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

The fixtures are what pins the CPU oracle (and, through it, the CUDA kernels) to the
reference's results.  Inputs follow the reference's own test recipes
(tests/test_gptq_w3_planar.py:21-39 ``synthetic_raw``, tests/test_deployment.py:12-27
``make_payload``, tests/test_fused_modules.py:38-45 ``rope_inputs``).
"""
import sys
from pathlib import Path

import numpy as np
import torch

if len(sys.argv) != 2:
    sys.exit("usage: make_golden.py /path/to/reference")
REFERENCE = Path(sys.argv[1])
sys.path.insert(0, str(REFERENCE / "src"))
sys.path.insert(0, str(REFERENCE / "tests"))

from fluxbin_style import gptq_deployment as gd  # noqa: E402
from fluxbin_style import deployment as dep  # noqa: E402
from fluxbin_style.evaluation import materialize_hybrid_s8_weight  # noqa: E402
from fluxbin_style.factored_reference import structural_reference  # noqa: E402
from fluxbin_style.fused_modules import fused_apply_rotary_pos_emb, rms_norm_reference  # noqa: E402
from fluxbin_style.packing import pack_two_bases, unpack_two_bases  # noqa: E402
from test_deployment import make_payload  # noqa: E402
from test_gptq_w3_planar import synthetic_raw  # noqa: E402

OUT = Path(__file__).resolve().parent


def bits(t):
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16)


def w3_case(name, k, o, seed, x_seed):
    raw, codes, zeros = synthetic_raw(k=k, o=o, seed=seed)
    layout = gd.convert_gptq_w3_to_planar(raw, qzero_format=1)
    x = torch.randn(1, k, generator=torch.Generator().manual_seed(x_seed), dtype=torch.bfloat16)
    restored = gd.restore_planar_w3(layout)
    np.savez_compressed(
        OUT / f"{name}.npz",
        qweight=raw["qweight"].numpy(), qzeros=raw["qzeros"].numpy(),
        scales_f16=bits(raw["scales"]), g_idx=raw["g_idx"].numpy(),
        codes=codes.numpy(), zeros=zeros.numpy(),
        planes=layout["planes"].numpy(), scales_bf16=bits(layout["scales"]),
        perm=layout["perm"].numpy(),
        sorted_codes=gd.decode_planar_w3_codes(layout, original_order=False).numpy(),
        restored_bf16=bits(restored),
        x_bf16=bits(x),
        structural=gd.structural_w3_matvec(x, layout).numpy(),
        bf16_weight_semantics=gd.bf16_weight_semantics_w3_matvec(x, layout).numpy(),
        dequant_matmul=torch.nn.functional.linear(x.float(), restored.float()).numpy(),
        qzeros_v2=gd.pack_gptq_w3_codes(zeros, packed_axis=1).numpy(),
    )


def hybrid_case(name, o, g, seed):
    p = make_payload(o, g, seed)
    inter = dep.convert_artifact(p, kernel="v5")
    planar = dep.convert_artifact(p, kernel="v5_p1024")
    x = torch.randn(1, g * 128, generator=torch.Generator().manual_seed(seed + 1)).bfloat16()
    arrays = {f"payload.{k}": v.numpy() for k, v in p.items()}
    arrays.update({f"inter.{k}": v.numpy() for k, v in inter.items()})
    arrays.update({f"planar.{k}": v.numpy() for k, v in planar.items()})
    arrays["x_bf16"] = bits(x)
    arrays["dense_f32"] = materialize_hybrid_s8_weight(
        **p, group_size=128, columns_per_group=8, device="cpu", output_dtype=torch.float32).numpy()
    arrays["structural_f64"] = structural_reference(x, planar).numpy()
    np.savez_compressed(OUT / f"{name}.npz", **arrays)


def packing_case():
    torch.manual_seed(31)
    bases = torch.where(torch.rand(2, 7, 20) < 0.5, torch.tensor(-1, dtype=torch.int8),
                        torch.tensor(1, dtype=torch.int8))
    codes = pack_two_bases(bases)
    assert torch.equal(unpack_two_bases(codes), bases)
    np.savez_compressed(OUT / "two_base_packing.npz", bases=bases.numpy(), codes=codes.numpy())


def fused_case():
    torch.manual_seed(20260914)
    arrays = {}
    for dim, tagname in ((4096, "hidden"), (128, "head")):
        rows = 1 if dim == 4096 else 40
        x = torch.randn(rows, dim).bfloat16()
        w = (1 + 0.1 * torch.randn(dim)).bfloat16()
        arrays[f"rms.{tagname}.x"] = bits(x)
        arrays[f"rms.{tagname}.w"] = bits(w)
        arrays[f"rms.{tagname}.out"] = bits(rms_norm_reference(x, w, 1e-6))
    q = torch.randn(1, 32, 1, 128).bfloat16()
    k = torch.randn(1, 8, 1, 128).bfloat16()
    cos = torch.randn(1, 1, 128).bfloat16()
    sin = torch.randn(1, 1, 128).bfloat16()
    qo, ko = fused_apply_rotary_pos_emb(q, k, cos, sin)
    arrays.update({"rope.q": bits(q), "rope.k": bits(k), "rope.cos": bits(cos), "rope.sin": bits(sin),
                   "rope.q_out": bits(qo.contiguous()), "rope.k_out": bits(ko.contiguous())})
    np.savez_compressed(OUT / "fused_modules.npz", **arrays)


if __name__ == "__main__":
    w3_case("w3_k256_o64", 256, 64, 20260916, 9)
    w3_case("w3_k512_o256", 512, 256, 17, 23)
    w3_case("w3_k384_o288", 384, 288, 20260916, 5)
    hybrid_case("hybrid_o17_g3", 17, 3, 19)
    hybrid_case("hybrid_o65_g10", 65, 10, 7)
    packing_case()
    fused_case()
    print("wrote", sorted(p.name for p in OUT.glob("*.npz")))
