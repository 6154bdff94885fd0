"""GPTQ W3 checkpoint unpacking and the planar group-128 layout the B200 GEMV kernel reads.

Host-side mirror of the reference's ``gptq_deployment`` module (same function names,
arguments and error behaviour; reference file ``src/fluxbin_style/gptq_deployment.py``).

A GPTQ W3 checkpoint stores 32 three-bit codes in three int32 words.  Read as one
96-bit little-endian stream, code ``i`` simply occupies bits ``3i .. 3i+2`` (which is what
the historical "10-1-10-1-10" description amounts to: codes 10 and 21 straddle a word
boundary).  The deployment layout sorts the input columns by group (``g_idx``), and stores
per group three bit planes of 16 bytes per output row, eight input positions per byte,
least-significant bit first.  The high plane is stored inverted so that, for the usual
zero point 4, ``code - 4 = b0 + 2*b1 - 4*stored_b2``.

Beyond the reference's three-field layout (``planes``, bf16 ``scales``, ``perm``; zero
point fixed at 4) this module accepts an EXTENDED layout with an optional ``zeros`` field
(uint8 ``[G,O]`` zero points) and fp16 or bf16 scales; ``convert_gptq_w3_to_planar(...,
general=True)`` produces it.  All conversions are lossless.
"""
from __future__ import annotations

from typing import Mapping

import torch

FORMAT = "gptq-w3-g128-sym-planar-m1-v1"
GENERAL_FORMAT = "gptq-w3-g128-zp-planar-m1-v1"
GROUP_SIZE = 128
BITS = 3
ZERO = 4
FIELDS = ("planes", "scales", "perm")
OPTIONAL_FIELDS = ("zeros",)
MAX_IN_FEATURES = 32767  # int16 permutation entries


# ----------------------------------------------------------------------------- words
def _stream_windows(words: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``words[..., 3]`` int32 -> two int64 windows holding stream bits 0..63 and 32..95."""
    u = words.to(torch.int64) & 0xFFFFFFFF
    return u[..., 0] | (u[..., 1] << 32), u[..., 1] | (u[..., 2] << 32)


def _codes_from_words(words: torch.Tensor) -> torch.Tensor:
    """``[..., 3]`` words -> ``[..., 32]`` codes (uint8)."""
    low, high = _stream_windows(words)
    index = torch.arange(32, dtype=torch.int64, device=words.device)
    use_low = index <= 10  # codes 0..10 end at bit 32, inside the low window
    shift = torch.where(use_low, 3 * index, 3 * index - 32)
    window = torch.where(use_low, low.unsqueeze(-1), high.unsqueeze(-1))
    return ((window >> shift) & 7).to(torch.uint8)


def _words_from_codes(codes: torch.Tensor) -> torch.Tensor:
    """``[..., 32]`` codes -> ``[..., 3]`` int32 words."""
    c = codes.to(torch.int64)
    # Stream bits 0..63 receive codes 0..21 (code 21's upper bits fall off, as intended);
    # stream bits 32..95 receive codes 10..31 (code 10 contributes only its top bit).
    low = torch.zeros(c.shape[:-1], dtype=torch.int64, device=codes.device)
    for i in range(22):
        low |= c[..., i] << (3 * i)  # int64 wrap-around of bit 63 is harmless: bits are masked below
    high = c[..., 10] >> 2
    for i in range(11, 32):
        high |= c[..., i] << (3 * i - 32)
    w0 = low & 0xFFFFFFFF
    w1 = (low >> 32) & 0xFFFFFFFF
    w2 = (high >> 32) & 0xFFFFFFFF
    words = torch.stack((w0, w1, w2), dim=-1)
    return torch.where(words >= 2**31, words - 2**32, words).to(torch.int32)


def _require_cpu_int32(name: str, value: torch.Tensor, ndim: int) -> None:
    if value.device.type != "cpu" or value.dtype != torch.int32 or value.ndim != ndim:
        raise ValueError(f"{name} must be CPU int32 rank {ndim}")
    if not value.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def unpack_gptq_w3_qweight(qweight: torch.Tensor) -> torch.Tensor:
    """``qweight`` int32 ``[3K/32, O]`` -> unsigned codes uint8 ``[K, O]``."""
    _require_cpu_int32("qweight", qweight, 2)
    rows, cols = qweight.shape
    if rows % 3:
        raise ValueError("packed row count must be divisible by three")
    triples = qweight.reshape(rows // 3, 3, cols).permute(0, 2, 1)  # [blocks, O, 3]
    return _codes_from_words(triples).permute(0, 2, 1).reshape(rows // 3 * 32, cols).contiguous()


def unpack_gptq_w3_qzeros(qzeros: torch.Tensor, *, qzero_format: int) -> torch.Tensor:
    """``qzeros`` int32 ``[G, 3O/32]`` -> zero points uint8 ``[G, O]``.

    Format 1 is the raw checkpoint convention (stored value = zero point - 1); format 2 is
    what a loaded GPTQModel module holds.  The caller states which one it has.
    """
    _require_cpu_int32("qzeros", qzeros, 2)
    if qzero_format not in (1, 2):
        raise ValueError("qzero_format must be 1 (raw GPTQ) or 2 (loaded GPTQ_V2)")
    rows, cols = qzeros.shape
    if cols % 3:
        raise ValueError("packed column count must be divisible by three")
    zeros = _codes_from_words(qzeros.reshape(rows, cols // 3, 3)).reshape(rows, cols // 3 * 32)
    if qzero_format == 1:
        zeros = (zeros + 1) & 7
    return zeros.contiguous()


def pack_gptq_w3_codes(codes: torch.Tensor, *, packed_axis: int = 0) -> torch.Tensor:
    """Inverse of the two unpackers: codes uint8 -> int32 words along rows (0) or columns (1)."""
    if codes.device.type != "cpu" or codes.dtype != torch.uint8 or codes.ndim != 2:
        raise ValueError("codes must be CPU uint8 rank two")
    if packed_axis not in (0, 1):
        raise ValueError("packed_axis must be zero or one")
    logical = codes if packed_axis == 0 else codes.T
    if logical.shape[0] % 32 or bool((logical > 7).any()):
        raise ValueError("packed logical dimension must be divisible by 32 and codes must be W3")
    blocks = logical.reshape(-1, 32, logical.shape[1]).permute(0, 2, 1)  # [blocks, other, 32]
    words = _words_from_codes(blocks).permute(0, 2, 1).reshape(-1, logical.shape[1])
    return words.contiguous() if packed_axis == 0 else words.T.contiguous()


# ---------------------------------------------------------------------------- planes
def _bits_to_bytes(bits: torch.Tensor) -> torch.Tensor:
    """``[..., 128]`` 0/1 values -> ``[..., 16]`` bytes, LSB = lowest position."""
    if bits.dtype != torch.uint8 or bits.shape[-1] != GROUP_SIZE:
        raise ValueError("bit tensor must be uint8 with a 128-element final dimension")
    weights = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.int32, device=bits.device)
    return (bits.reshape(*bits.shape[:-1], 16, 8).to(torch.int32) * weights).sum(-1).to(torch.uint8)


def _bytes_to_bits(values: torch.Tensor) -> torch.Tensor:
    if values.dtype != torch.uint8 or values.shape[-1] != 16:
        raise ValueError("packed planes must be uint8 with a 16-byte final dimension")
    position = torch.arange(8, dtype=torch.int32, device=values.device)
    return ((values.to(torch.int32).unsqueeze(-1) >> position) & 1).to(torch.uint8).flatten(-2)


def inspect_gptq_checkpoint(tensors: Mapping[str, torch.Tensor], *, qzero_format: int = 1) -> dict[str, object]:
    """Validate one Linear's raw GPTQ tensors and report its structure (no conversion)."""
    wanted = {"qweight", "qzeros", "scales", "g_idx"}
    if set(tensors) != wanted:
        raise ValueError(f"expected exactly {sorted(wanted)}")
    qweight, qzeros, scales, g_idx = (tensors[k] for k in ("qweight", "qzeros", "scales", "g_idx"))
    _require_cpu_int32("qweight", qweight, 2)
    _require_cpu_int32("qzeros", qzeros, 2)
    _require_cpu_int32("g_idx", g_idx, 1)
    if scales.device.type != "cpu" or scales.dtype != torch.float16 or scales.ndim != 2:
        raise ValueError("scales must be contiguous CPU float16 [G,O]")
    if not scales.is_contiguous() or not bool(torch.isfinite(scales).all()):
        raise ValueError("scales must be contiguous and finite")
    codes = unpack_gptq_w3_qweight(qweight)
    zeros = unpack_gptq_w3_qzeros(qzeros, qzero_format=qzero_format)
    in_features, out_features = codes.shape
    if in_features % GROUP_SIZE or in_features > MAX_IN_FEATURES:
        raise ValueError("v1 requires K divisible by 128 and representable by int16")
    groups = in_features // GROUP_SIZE
    if tuple(scales.shape) != (groups, out_features) or tuple(zeros.shape) != (groups, out_features):
        raise ValueError("qzero/scale shape does not match qweight")
    if tuple(g_idx.shape) != (in_features,) or int(g_idx.min()) != 0 or int(g_idx.max()) != groups - 1:
        raise ValueError("g_idx shape or range drifted")
    if not bool((torch.bincount(g_idx.long(), minlength=groups) == GROUP_SIZE).all()):
        raise ValueError("each g_idx group must contain exactly 128 input columns")
    order = torch.argsort(g_idx, stable=True)
    if not torch.equal(g_idx[order].long(), torch.arange(in_features) // GROUP_SIZE):
        raise ValueError("sorted g_idx is not canonical group128")
    return {
        "bits": BITS,
        "group_size": GROUP_SIZE,
        "qweight_shape": list(qweight.shape),
        "qzeros_shape": list(qzeros.shape),
        "scales_shape": list(scales.shape),
        "g_idx_shape": list(g_idx.shape),
        "in_features": in_features,
        "out_features": out_features,
        "groups": groups,
        "qzero_format": qzero_format,
        "decoded_zero_unique": sorted(int(v) for v in torch.unique(zeros).tolist()),
        "permutation_identity": bool(torch.equal(order, torch.arange(in_features))),
    }


def validate_planar_w3(layout: Mapping[str, torch.Tensor], *, check_values: bool = True) -> tuple[int, int]:
    """Check the layout contract and return ``(out_features, in_features)``.

    ``check_values=False`` skips everything that would read tensor contents (finite
    scales, permutation bijection, zero-point range), so it launches nothing on a GPU
    and is safe right before or inside graph capture.
    """
    names = set(layout)
    if not set(FIELDS) <= names or not names <= set(FIELDS) | set(OPTIONAL_FIELDS):
        raise ValueError(f"expected exactly {FIELDS}" + f" (optionally {OPTIONAL_FIELDS})")
    planes, scales, perm = (layout[name] for name in FIELDS)
    zeros = layout.get("zeros")
    if planes.dtype != torch.uint8 or planes.ndim != 4 or planes.shape[1] != 3 or planes.shape[3] != 16:
        raise ValueError("planes must be uint8 [G,3,O,16]")
    groups, _, out_features, _ = planes.shape
    if scales.dtype not in (torch.bfloat16, torch.float16) or tuple(scales.shape) != (groups, out_features):
        raise ValueError("deployment scales must be bfloat16 (or float16) [G,O]")
    in_features = groups * GROUP_SIZE
    if in_features > MAX_IN_FEATURES:
        raise ValueError("v1 perm indices must be representable by int16")
    if perm.dtype != torch.int16 or tuple(perm.shape) != (in_features,):
        raise ValueError("perm must be int16 [K]")
    if zeros is not None and (zeros.dtype != torch.uint8 or tuple(zeros.shape) != (groups, out_features)):
        raise ValueError("zeros must be uint8 [G,O]")
    if any(value.device != planes.device or not value.is_contiguous() for value in layout.values()):
        raise ValueError("layout tensors must be contiguous on one device")
    if check_values:
        if not bool(torch.isfinite(scales).all()):
            raise ValueError("scales must be finite")
        wide = perm.long()
        if int(wide.min()) != 0 or int(wide.max()) != in_features - 1 or torch.unique(wide).numel() != in_features:
            raise ValueError("perm must be a bijection over K")
        if zeros is not None and int(zeros.max()) > 7:
            raise ValueError("zero points must be W3 values 0..7")
    return out_features, in_features


def is_identity_perm(perm: torch.Tensor) -> bool:
    return bool(torch.equal(perm.long().cpu(), torch.arange(perm.numel())))


def planes_from_sorted_codes(sorted_codes: torch.Tensor) -> torch.Tensor:
    """Codes uint8 ``[K,O]`` already in group-sorted column order -> planes ``[G,3,O,16]``."""
    in_features, out_features = sorted_codes.shape
    grouped = sorted_codes.reshape(in_features // GROUP_SIZE, GROUP_SIZE, out_features).transpose(1, 2)  # [G,O,128]
    stack = [_bits_to_bytes((grouped >> bit) & 1) for bit in range(2)]
    stack.append(_bits_to_bytes(1 - ((grouped >> 2) & 1)))  # high plane stored inverted
    return torch.stack(stack, dim=1).contiguous()


def convert_gptq_w3_to_planar(
    tensors: Mapping[str, torch.Tensor], *, qzero_format: int = 1, general: bool = False
) -> dict[str, torch.Tensor]:
    """Raw GPTQ tensors of one Linear -> deployment layout.

    Default (``general=False``) is the reference's contract: every zero point must be 4,
    scales are stored as bf16, fields are exactly ``planes``/``scales``/``perm``.  With
    ``general=True`` the fp16 scales are kept as they are and, unless all zero points are
    4, a ``zeros`` field carries them.
    """
    facts = inspect_gptq_checkpoint(tensors, qzero_format=qzero_format)
    if not general and facts["decoded_zero_unique"] != [ZERO]:
        raise ValueError(f"v1 constant-zero fast path requires decoded zero=4, got {facts['decoded_zero_unique']}")
    codes = unpack_gptq_w3_qweight(tensors["qweight"])
    order = torch.argsort(tensors["g_idx"], stable=True)
    layout = {
        "planes": planes_from_sorted_codes(codes[order]),
        # A checkpoint loaded with dtype=bfloat16 casts its fp16 scales before
        # dequantising; the three-field layout stores exactly that value.
        "scales": (tensors["scales"] if general else tensors["scales"].to(torch.bfloat16)).contiguous(),
        "perm": order.to(torch.int16).contiguous(),
    }
    if general and facts["decoded_zero_unique"] != [ZERO]:
        layout["zeros"] = unpack_gptq_w3_qzeros(tensors["qzeros"], qzero_format=qzero_format)
    validate_planar_w3(layout)
    return layout


def decode_planar_w3_codes(layout: Mapping[str, torch.Tensor], *, original_order: bool = True) -> torch.Tensor:
    """Layout -> unsigned codes ``[K,O]`` (in checkpoint column order unless told otherwise)."""
    out_features, in_features = validate_planar_w3(layout)
    planes = layout["planes"]
    low, mid = _bytes_to_bits(planes[:, 0]), _bytes_to_bits(planes[:, 1])
    high = 1 - _bytes_to_bits(planes[:, 2])
    ordered = (low | (mid << 1) | (high << 2)).transpose(1, 2).reshape(in_features, out_features)
    if not original_order:
        return ordered.contiguous()
    result = torch.empty_like(ordered)
    result[layout["perm"].long()] = ordered
    return result


def _signed_codes(layout: Mapping[str, torch.Tensor]) -> torch.Tensor:
    """``code - zero`` as int16 ``[G,128,O]`` in sorted order."""
    out_features, in_features = validate_planar_w3(layout, check_values=False)
    codes = decode_planar_w3_codes(layout, original_order=False).to(torch.int16)
    grouped = codes.reshape(in_features // GROUP_SIZE, GROUP_SIZE, out_features)
    zeros = layout.get("zeros")
    return grouped - (ZERO if zeros is None else zeros.to(torch.int16).unsqueeze(1))


def restore_planar_w3(layout: Mapping[str, torch.Tensor], *, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Dequantise to a dense ``[O,K]`` weight.

    The product ``scale * (code - zero)`` is formed in the scales' own 16-bit dtype (one
    rounding, as a GPTQ module loaded in that dtype computes it) and then cast to ``dtype``.
    """
    out_features, in_features = validate_planar_w3(layout)
    signed = _signed_codes(layout)  # [G,128,O]
    product = layout["scales"].unsqueeze(1) * signed  # 16-bit float * int16 -> 16-bit float
    ordered = product.permute(2, 0, 1).reshape(out_features, in_features)
    weight = torch.empty_like(ordered)
    weight[:, layout["perm"].long()] = ordered
    return weight.to(dtype=dtype).contiguous()


def _sorted_activations(x: torch.Tensor, layout: Mapping[str, torch.Tensor], in_features: int) -> torch.Tensor:
    if x.ndim != 2 or tuple(x.shape) != (1, in_features):
        raise ValueError("x must have shape [1,K]")
    if x.device != layout["planes"].device:
        raise ValueError("x and layout must share a device")
    return x[0, layout["perm"].long()].float().reshape(-1, GROUP_SIZE)


def structural_w3_matvec(x: torch.Tensor, layout: Mapping[str, torch.Tensor]) -> torch.Tensor:
    """FP32 reference without a dense weight: per group, integer dot then one scale multiply."""
    out_features, in_features = validate_planar_w3(layout)
    xs = _sorted_activations(x, layout, in_features)
    signed = _signed_codes(layout).float()  # [G,128,O]
    total = torch.zeros(out_features, dtype=torch.float32, device=x.device)
    for group in range(signed.shape[0]):
        total += (signed[group].T @ xs[group]) * layout["scales"][group].float()
    return total.unsqueeze(0)


def bf16_weight_semantics_w3_matvec(x: torch.Tensor, layout: Mapping[str, torch.Tensor]) -> torch.Tensor:
    """FP32 grouped matvec that reproduces the rounding of the dequantised 16-bit weight.

    With zero point 4 the signed codes are -4..3; ``scale * code`` is exact in the scale's
    dtype except for codes +/-3, so the dense-weight result equals the structural one plus
    ``(round(3*scale) - 3*scale)`` times the signed count-weighted activations at +/-3.
    """
    out_features, in_features = validate_planar_w3(layout)
    if "zeros" in layout:
        raise ValueError("the +/-3 correction form needs the constant zero point 4")
    xs = _sorted_activations(x, layout, in_features)
    signed = _signed_codes(layout)
    scales = layout["scales"]
    delta = (scales * 3).to(scales.dtype).float() - 3.0 * scales.float()
    total = torch.zeros(out_features, dtype=torch.float32, device=x.device)
    for group in range(signed.shape[0]):
        act = xs[group].unsqueeze(-1)
        s = signed[group]
        integer_dot = (s.float() * act).sum(0)
        three_dot = (((s == 3).float() - (s == -3).float()) * act).sum(0)
        total += integer_dot * scales[group].float() + three_dot * delta[group]
    return total.unsqueeze(0)


def layout_storage(layout: Mapping[str, torch.Tensor]) -> dict[str, object]:
    out_features, in_features = validate_planar_w3(layout)
    sizes = {name: value.numel() * value.element_size() for name, value in layout.items()}
    total = sum(sizes.values())
    return {
        "format": GENERAL_FORMAT if "zeros" in layout or layout["scales"].dtype != torch.bfloat16 else FORMAT,
        "shape": [out_features, in_features],
        "tensor_bytes": sizes,
        "total_bytes": total,
        "bits_per_weight": total * 8 / (out_features * in_features),
    }
