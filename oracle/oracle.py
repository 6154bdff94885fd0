"""ctypes front end of the CPU oracle (``fluxbin_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this module;
the product never does.  Arrays are numpy; 16-bit floating values travel as ``uint16``
bit patterns with a dtype tag (``F16``/``BF16``).  ``bits``/``unbits`` convert to and from
torch tensors for callers that hold them.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

F16, BF16, F32 = 0, 1, 2
_HERE = Path(__file__).resolve().parent
_LIB = None


def build(force: bool = False) -> Path:
    """Compile the oracle (and the reference LUT shim when the reference tree exists)."""
    target = _HERE / "libfluxbin_oracle.so"
    source = _HERE / "fluxbin_oracle.c"
    if force or not target.exists() or target.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return target


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(str(build()))
        _LIB.fbo_num_threads.restype = ctypes.c_int
    return _LIB


def reference_lut_lib():
    """The reference's own LUT helpers, or None when they were not built."""
    path = _HERE / "_ref" / "libref_lut.so"
    return ctypes.CDLL(str(path)) if path.exists() else None


def _p(array):
    return None if array is None else array.ctypes.data_as(ctypes.c_void_p)


def _c(array, dtype):
    return None if array is None else np.ascontiguousarray(array, dtype=dtype)


def _check(code, name):
    if code != 0:
        raise ValueError(f"oracle {name} rejected its input (code {code})")


def tag(dtype) -> int:
    """Map a torch or numpy dtype (or its name) to the oracle's tag."""
    name = str(dtype)
    if "bfloat16" in name:
        return BF16
    if "float16" in name or "half" in name:
        return F16
    if "float32" in name:
        return F32
    raise ValueError(f"unsupported dtype {dtype}")


def bits(tensor) -> np.ndarray:
    """torch fp16/bf16 tensor -> uint16 bit patterns (numpy)."""
    import torch

    return tensor.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def unbits(array: np.ndarray, dtype):
    """uint16 bit patterns -> torch tensor of ``dtype`` (torch.float16 / torch.bfloat16)."""
    import torch

    return torch.from_numpy(np.ascontiguousarray(array).view(np.int16)).view(dtype)


def num_threads() -> int:
    return int(lib().fbo_num_threads())


def set_num_threads(count: int) -> None:
    """Threads of the oracle's parallel loops; overrides an OMP_NUM_THREADS a launcher exported."""
    lib().fbo_set_num_threads(ctypes.c_int(int(count)))


# ----------------------------------------------------------------- GPTQ words
def gptq_unpack_rows(qweight: np.ndarray) -> np.ndarray:
    words = _c(qweight, np.int32)
    rows, cols = words.shape
    codes = np.empty((rows // 3 * 32, cols), np.uint8)
    _check(lib().fbo_gptq_w3_unpack_rows(_p(words), ctypes.c_int64(rows), ctypes.c_int64(cols), _p(codes)), "unpack_rows")
    return codes


def gptq_pack_rows(codes: np.ndarray) -> np.ndarray:
    codes = _c(codes, np.uint8)
    k, cols = codes.shape
    words = np.empty((k // 32 * 3, cols), np.int32)
    _check(lib().fbo_gptq_w3_pack_rows(_p(codes), ctypes.c_int64(k), ctypes.c_int64(cols), _p(words)), "pack_rows")
    return words


def gptq_unpack_cols(qzeros: np.ndarray, qzero_format: int) -> np.ndarray:
    words = _c(qzeros, np.int32)
    rows, pc = words.shape
    zeros = np.empty((rows, pc // 3 * 32), np.uint8)
    _check(lib().fbo_gptq_w3_unpack_cols(_p(words), ctypes.c_int64(rows), ctypes.c_int64(pc), qzero_format, _p(zeros)), "unpack_cols")
    return zeros


def gptq_pack_cols(values: np.ndarray) -> np.ndarray:
    values = _c(values, np.uint8)
    rows, cols = values.shape
    words = np.empty((rows, cols // 32 * 3), np.int32)
    _check(lib().fbo_gptq_w3_pack_cols(_p(values), ctypes.c_int64(rows), ctypes.c_int64(cols), _p(words)), "pack_cols")
    return words


# ------------------------------------------------------------------ W3 planes
def w3_planes_from_codes(codes: np.ndarray, perm=None) -> np.ndarray:
    codes = _c(codes, np.uint8)
    k, o = codes.shape
    perm = _c(perm, np.int16)
    planes = np.empty((k // 128, 3, o, 16), np.uint8)
    _check(lib().fbo_w3_planes_from_codes(_p(codes), _p(perm), ctypes.c_int64(k), ctypes.c_int64(o), _p(planes)), "planes_from_codes")
    return planes


def w3_codes_from_planes(planes: np.ndarray, perm=None, original_order=True) -> np.ndarray:
    planes = _c(planes, np.uint8)
    g, _, o, _ = planes.shape
    perm = _c(perm, np.int16)
    codes = np.empty((g * 128, o), np.uint8)
    _check(lib().fbo_w3_codes_from_planes(_p(planes), _p(perm), ctypes.c_int64(g * 128), ctypes.c_int64(o), int(original_order), _p(codes)), "codes_from_planes")
    return codes


def w3_dequant(planes, scales_bits, scale_dtype, zeros=None, perm=None, out_dtype=F32) -> np.ndarray:
    planes = _c(planes, np.uint8)
    g, _, o, _ = planes.shape
    k = g * 128
    scales_bits, zeros, perm = _c(scales_bits, np.uint16), _c(zeros, np.uint8), _c(perm, np.int16)
    out = np.empty((o, k), np.float32 if out_dtype == F32 else np.uint16)
    _check(lib().fbo_w3_dequant(_p(planes), _p(scales_bits), scale_dtype, _p(zeros), _p(perm), ctypes.c_int64(k), ctypes.c_int64(o), out_dtype, _p(out)), "w3_dequant")
    return out


def dense_gemv_f32(w: np.ndarray, x: np.ndarray) -> np.ndarray:
    w, x = _c(w, np.float32), _c(x, np.float32)
    o, k = w.shape
    m = x.shape[0]
    y = np.empty((m, o), np.float32)
    lib().fbo_dense_gemv_f32(_p(w), _p(x), ctypes.c_int64(m), ctypes.c_int64(o), ctypes.c_int64(k), _p(y))
    return y


def dense_gemv_half(w_bits: np.ndarray, w_dtype: int, x: np.ndarray) -> np.ndarray:
    w_bits, x = _c(w_bits, np.uint16), _c(x, np.float32)
    o, k = w_bits.shape
    m = x.shape[0]
    y = np.empty((m, o), np.float32)
    lib().fbo_dense_gemv_half(_p(w_bits), w_dtype, _p(x), ctypes.c_int64(m), ctypes.c_int64(o), ctypes.c_int64(k), _p(y))
    return y


def _w3_gemv(fn, name, x_bits, act_dtype, planes, scales_bits, scale_dtype, zeros, perm):
    planes = _c(planes, np.uint8)
    g, _, o, _ = planes.shape
    k = g * 128
    x_bits = _c(x_bits, np.uint16).reshape(-1, k)
    m = x_bits.shape[0]
    scales_bits, zeros, perm = _c(scales_bits, np.uint16), _c(zeros, np.uint8), _c(perm, np.int16)
    y = np.empty((m, o), np.float32)
    _check(fn(_p(x_bits), act_dtype, ctypes.c_int64(m), _p(planes), _p(scales_bits), scale_dtype, _p(zeros), _p(perm), ctypes.c_int64(k), ctypes.c_int64(o), _p(y)), name)
    return y


def w3_gemv_dequant(x_bits, act_dtype, planes, scales_bits, scale_dtype, zeros=None, perm=None):
    """Dequantise-then-matmul, fp32 accumulate: the oracle of record.  Returns fp32 [M,O]."""
    return _w3_gemv(lib().fbo_w3_gemv_dequant, "w3_gemv_dequant", x_bits, act_dtype, planes, scales_bits, scale_dtype, zeros, perm)


def w3_gemv_structural(x_bits, act_dtype, planes, scales_bits, scale_dtype, zeros=None, perm=None):
    return _w3_gemv(lib().fbo_w3_gemv_structural, "w3_gemv_structural", x_bits, act_dtype, planes, scales_bits, scale_dtype, zeros, perm)


def w3_gemv_lut_emulation(x_bits, act_dtype, planes, scales_bits, scale_dtype, perm=None):
    planes = _c(planes, np.uint8)
    g, _, o, _ = planes.shape
    k = g * 128
    x_bits = _c(x_bits, np.uint16).reshape(k)
    scales_bits, perm = _c(scales_bits, np.uint16), _c(perm, np.int16)
    y = np.empty((1, o), np.float32)
    _check(lib().fbo_w3_gemv_lut_emulation(_p(x_bits), act_dtype, _p(planes), _p(scales_bits), scale_dtype, _p(perm), ctypes.c_int64(k), ctypes.c_int64(o), _p(y)), "w3_gemv_lut_emulation")
    return y


# ------------------------------------------------------------------ two bases
def pack_two_bases(bases: np.ndarray) -> np.ndarray:
    bases = _c(bases, np.int8)
    _, o, k = bases.shape
    codes = np.empty((o, k // 4), np.uint8)
    _check(lib().fbo_pack_two_bases(_p(bases), ctypes.c_int64(o), ctypes.c_int64(k), _p(codes)), "pack_two_bases")
    return codes


def unpack_two_bases(codes: np.ndarray) -> np.ndarray:
    codes = _c(codes, np.uint8)
    o, qk = codes.shape
    bases = np.empty((2, o, qk * 4), np.int8)
    lib().fbo_unpack_two_bases(_p(codes), ctypes.c_int64(o), ctypes.c_int64(qk), _p(bases))
    return bases


def bb_to_planes(interleaved: np.ndarray) -> np.ndarray:
    """[..., 2n] interleaved bytes -> [..., 2, n] planes."""
    inter = _c(interleaved, np.uint8)
    n = inter.shape[-1] // 2
    rows = inter.size // (2 * n)
    out = np.empty(inter.shape[:-1] + (2, n), np.uint8)
    lib().fbo_bb_to_planes(_p(inter), ctypes.c_int64(rows), ctypes.c_int64(n), _p(out))
    return out


def bb_from_planes(planes: np.ndarray) -> np.ndarray:
    planes = _c(planes, np.uint8)
    n = planes.shape[-1]
    rows = planes.size // (2 * n)
    out = np.empty(planes.shape[:-2] + (2 * n,), np.uint8)
    lib().fbo_bb_from_planes(_p(planes), ctypes.c_int64(rows), ctypes.c_int64(n), _p(out))
    return out


def bb_materialize_hybrid(payload: dict) -> np.ndarray:
    """Seven-field payload (numpy arrays, reference field names) -> dense fp32 [O,K]."""
    codes = _c(payload["global_sign_codes"], np.uint8)
    o, width = codes.shape
    g = width // 32
    w = np.empty((o, g * 128), np.float32)
    holders = [
        codes, _c(payload["global_row_scales"], np.float32),
        _c(payload["global_column_scales"], np.float32),
        _c(payload["refinement_indices"], np.int64),
        _c(payload["refinement_sign_codes"], np.uint8),
        _c(payload["refinement_row_scales"], np.float32),
        _c(payload["refinement_column_scales"], np.float32),
    ]
    args = tuple(_p(h) for h in holders)
    _check(lib().fbo_bb_materialize_hybrid(*args, ctypes.c_int64(o), ctypes.c_int64(g), _p(w)), "bb_materialize_hybrid")
    return w


def bb_structural_f64(x_bits, act_dtype, layout: dict) -> np.ndarray:
    """FP64 structural reference on the kernel layout (numpy arrays, layout field names)."""
    codes = _c(layout["codes"], np.uint8)
    planar = int(codes.ndim == 4)
    g, o = codes.shape[:2]
    y = np.empty((1, o), np.float64)
    holders = [
        _c(x_bits, np.uint16), codes, _c(layout["rows"], np.float32), _c(layout["columns"], np.float32),
        _c(layout["indices"], np.int16), _c(layout["sparse_codes"], np.uint8),
        _c(layout["sparse_rows"], np.float32), _c(layout["sparse_columns"], np.float32),
    ]
    _check(lib().fbo_bb_structural_f64(_p(holders[0]), act_dtype, _p(holders[1]), planar, _p(holders[2]), _p(holders[3]), _p(holders[4]), _p(holders[5]), _p(holders[6]), _p(holders[7]), ctypes.c_int64(o), ctypes.c_int64(g), _p(y)), "bb_structural_f64")
    return y


def bb_global_gemv_f64(x_bits, act_dtype, planes, rscale_bits, cscale_bits, sal_idx, sal_bits) -> np.ndarray:
    planes = _c(planes, np.uint8)
    _, o, k8 = planes.shape
    sal_idx = _c(sal_idx, np.int32)
    n_sal = 0 if sal_idx is None else sal_idx.shape[0]
    holders = [_c(x_bits, np.uint16), planes, _c(rscale_bits, np.uint16), _c(cscale_bits, np.uint16), sal_idx, _c(sal_bits, np.uint16)]
    y = np.empty((1, o), np.float64)
    _check(lib().fbo_bb_global_gemv_f64(_p(holders[0]), act_dtype, _p(holders[1]), _p(holders[2]), _p(holders[3]), _p(holders[4]), _p(holders[5]), ctypes.c_int64(n_sal), ctypes.c_int64(o), ctypes.c_int64(k8 * 8), _p(y)), "bb_global_gemv_f64")
    return y


def bb_global_materialize(planes, rscale_bits, cscale_bits, sal_idx, sal_bits) -> np.ndarray:
    planes = _c(planes, np.uint8)
    _, o, k8 = planes.shape
    sal_idx = _c(sal_idx, np.int32)
    n_sal = 0 if sal_idx is None else sal_idx.shape[0]
    holders = [planes, _c(rscale_bits, np.uint16), _c(cscale_bits, np.uint16), sal_idx, _c(sal_bits, np.uint16)]
    w = np.empty((o, k8 * 8), np.float32)
    _check(lib().fbo_bb_global_materialize(_p(holders[0]), _p(holders[1]), _p(holders[2]), _p(holders[3]), _p(holders[4]), ctypes.c_int64(n_sal), ctypes.c_int64(o), ctypes.c_int64(k8 * 8), _p(w)), "bb_global_materialize")
    return w


# ------------------------------------------------------------ RMSNorm / RoPE
def rmsnorm(x_bits, weight_bits, dtype: int, eps: float) -> np.ndarray:
    x_bits = _c(x_bits, np.uint16)
    dim = x_bits.shape[-1]
    rows = x_bits.size // dim
    weight_bits = _c(weight_bits, np.uint16)
    out = np.empty_like(x_bits)
    lib().fbo_rmsnorm(_p(x_bits), _p(weight_bits), dtype, ctypes.c_int64(rows), ctypes.c_int64(dim), ctypes.c_float(eps), _p(out))
    return out


def rope(v_bits, cos_bits, sin_bits, dtype: int) -> np.ndarray:
    v_bits = _c(v_bits, np.uint16)
    dim = v_bits.shape[-1]
    heads = v_bits.size // dim
    cos_bits, sin_bits = _c(cos_bits, np.uint16), _c(sin_bits, np.uint16)
    out = np.empty_like(v_bits)
    lib().fbo_rope(_p(v_bits), _p(cos_bits), _p(sin_bits), dtype, ctypes.c_int64(heads), ctypes.c_int64(dim), _p(out))
    return out
