"""ctypes binding of ``libfluxbin_b200.so`` (the C ABI declared in ``include/fluxbin_b200.h``).

There is no CPU substitute: if the library is missing or cannot be loaded, every call
raises.  Tensors are passed as raw device pointers; the current torch CUDA stream is
used for the launch.
"""
from __future__ import annotations

import ctypes
import os as _os
from pathlib import Path

import torch

LIBRARY = Path(__import__("os").environ.get("FB_LIBRARY", str(Path(__file__).resolve().parent / "libfluxbin_b200.so")))

FB_F16, FB_BF16 = 0, 1
FB_W3_DECODED_BF16 = 1
FB_W3_NO_PDL = 2
FB_W3_GROUP_PARTIALS = 4
FB_W3_SAME_INPUT = 8

_lib = None


class W3Matrix(ctypes.Structure):
    """``fb_w3_matrix_t`` of the C header."""

    _fields_ = [("planes", ctypes.c_void_p), ("scales", ctypes.c_void_p), ("zeros", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("out_features", ctypes.c_int)]


class W3Push(ctypes.Structure):
    """``fb_w3_push_t`` of the C header: per rank, where this rank's rows go and which counter to bump."""

    _fields_ = [("data", ctypes.c_void_p * 8), ("world", ctypes.c_int)]


class NativeError(RuntimeError):
    """A call into the CUDA library was rejected (message from ``fb_last_error``)."""


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIBRARY.exists():
            raise RuntimeError(
                f"{LIBRARY.name} is not built; run `python -m marlin_style_fluxbin_b200.build` "
                "(needs nvcc). There is no CPU or other fallback for the packed kernels."
            )
        lib = ctypes.CDLL(str(LIBRARY))
        lib.fb_last_error.restype = ctypes.c_char_p
        lib.fb_query.restype = ctypes.c_int64
        lib.fb_query.argtypes = [ctypes.c_char_p]
        lib.fb_w3_gemv_scratch_bytes.restype = ctypes.c_size_t
        lib.fb_w3_gemv_scratch_bytes.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
        lib.fb_w3_gemv.restype = ctypes.c_int
        lib.fb_w3_gemv.argtypes = [
            ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
            ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint, ctypes.c_void_p,
        ]
        lib.fb_w3_gemv_multi.restype = ctypes.c_int
        lib.fb_w3_gemv_multi.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(W3Matrix), ctypes.c_int,
                                         ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                                         ctypes.c_uint, ctypes.c_void_p]
        lib.fb_w3_gemv_fused_input.restype = ctypes.c_int
        lib.fb_w3_gemv_fused_input.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_float,
                                               ctypes.POINTER(W3Matrix), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                               ctypes.c_size_t, ctypes.c_uint, ctypes.c_void_p]
        lib.fb_w3_gemm_small_scratch_bytes.restype = ctypes.c_size_t
        lib.fb_w3_gemm_small_scratch_bytes.argtypes = [ctypes.c_int] * 3
        lib.fb_w3_gemm_small.restype = ctypes.c_int
        lib.fb_w3_gemm_small.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                         ctypes.c_size_t, ctypes.c_void_p]
        lib.fb_w3_gemv_push.restype = ctypes.c_int
        lib.fb_w3_gemv_push.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_float,
                                        ctypes.POINTER(W3Matrix), ctypes.c_int, ctypes.c_int, ctypes.POINTER(W3Push), ctypes.c_void_p,
                                        ctypes.c_size_t, ctypes.c_uint, ctypes.c_void_p]
        lib.fb_tp_reduce.restype = ctypes.c_int
        lib.fb_tp_reduce.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p]
        lib.fb_w3_finish.restype = ctypes.c_int
        lib.fb_w3_finish.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        lib.fb_bb_gemv_scratch_bytes.restype = ctypes.c_size_t
        lib.fb_bb_gemv_scratch_bytes.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
        lib.fb_bb_gemv.restype = ctypes.c_int
        lib.fb_bb_gemv.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 7 + [
            ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint, ctypes.c_void_p]
        lib.fb_bb_global_gemv.restype = ctypes.c_int
        lib.fb_bb_global_gemv.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 5 + [ctypes.c_int, ctypes.c_void_p,
            ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint, ctypes.c_void_p]
        lib.fb_rmsnorm.restype = ctypes.c_int
        lib.fb_rmsnorm.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
        lib.fb_rope_qk.restype = ctypes.c_int
        lib.fb_rope_qk.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 4 + [ctypes.c_void_p]
        lib.fb_qknorm_rope_cache.restype = ctypes.c_int
        lib.fb_qknorm_rope_cache.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
        lib.fb_attn_decode.restype = ctypes.c_int
        lib.fb_attn_decode.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        lib.fb_attn_decode_fused.restype = ctypes.c_int
        lib.fb_attn_decode_fused.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_float, ctypes.c_int,
                                                                                         ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        lib.fb_attn_decode_splits.restype = ctypes.c_int
        lib.fb_attn_decode_splits.argtypes = [ctypes.c_int]
        lib.fb_attn_decode_partial.restype = ctypes.c_int
        lib.fb_attn_decode_partial.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_float, ctypes.c_int,
                                                                                          ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        lib.fb_w3_gemv_attn_merge.restype = ctypes.c_int
        lib.fb_w3_gemv_attn_merge.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(W3Matrix), ctypes.c_int, ctypes.c_int,
                                              ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint, ctypes.c_void_p]
        lib.fb_attn_decode_scratch_bytes.restype = ctypes.c_size_t
        lib.fb_attn_decode_scratch_bytes.argtypes = [ctypes.c_int]
        lib.fb_silu_mul.restype = ctypes.c_int
        lib.fb_silu_mul.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.fb_lm_head_shard.restype = ctypes.c_int
        lib.fb_lm_head_shard.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(W3Push), ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                                         ctypes.c_void_p]
        lib.fb_tp_argmax.restype = ctypes.c_int
        lib.fb_tp_argmax.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                     ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p]
        lib.fb_lm_head_scratch_bytes.restype = ctypes.c_size_t
        lib.fb_lm_head_scratch_bytes.argtypes = []
        lib.fb_lm_head_argmax.restype = ctypes.c_int
        lib.fb_lm_head_argmax.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_int] + [ctypes.c_void_p] * 6 + [ctypes.c_size_t, ctypes.c_void_p]
        lib.fb_embed_row.restype = ctypes.c_int
        lib.fb_embed_row.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.fb_w3_gemv_static.restype = ctypes.c_int
        lib.fb_w3_gemv_static.argtypes = lib.fb_w3_gemv.argtypes[:11] + [ctypes.c_uint, ctypes.c_void_p]
        _lib = lib
    return _lib


# The last call into the library per (device, stream), when it was a plain W3 GEMV launch: its activation
# buffer and how many launches in a row have read it.  Any other library call forgets it (see ``w3_gemv``).
_same_input: dict = {}


def check(code: int) -> None:
    _same_input.clear()  # whatever was just launched is now the launch ahead of the next one
    if code != 0:
        raise NativeError(library().fb_last_error().decode() or f"native call failed with code {code}")


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return FB_F16
    if dtype == torch.bfloat16:
        return FB_BF16
    raise ValueError("FP16/BF16 required")


def ptr(tensor):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


def stream_handle(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def query(key: str) -> int:
    return int(library().fb_query(key.encode()))


def w3_scratch_bytes(m: int, out_features: int, in_features: int) -> int:
    return int(library().fb_w3_gemv_scratch_bytes(m, out_features, in_features))


# One zero-initialised scratch per (device, stream, kernel family): calls ordered on one stream may
# share it; the kernels leave it ready for the next call.  It is allocated ONCE at the largest size
# its family can ask for, so that a CUDA graph captured earlier on the stream never holds the
# address of a buffer that a later, larger call replaced; should a call still need more, the old
# buffer is retired, not freed.  The first call allocates, so it must come before graph capture.
_scratch: dict[tuple[int, int, str], torch.Tensor] = {}
_retired: list[torch.Tensor] = []


def _family_bytes(family: str) -> int:
    lib = library()
    if family.startswith("w3#"):  # the second and third scratch of launches that may overlap (one activation row)
        return int(lib.fb_w3_gemv_scratch_bytes(1, 65536, 32640))
    if family == "w3":
        return int(lib.fb_w3_gemv_scratch_bytes(4, 65536, 32640))
    if family == "w3mma":
        return int(lib.fb_w3_gemm_small_scratch_bytes(16, 65536, 32640))
    return int(lib.fb_bb_gemv_scratch_bytes(65536, 32640, 1))


def scratch_for(device: torch.device, nbytes: int, family: str = "w3") -> torch.Tensor:
    """Zero-filled scratch per (device, stream, kernel family).  Families lay their control words
    out differently, and each kernel relies on finding its own words zero, so they never share."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream, family)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("packed GEMV scratch must be sized by a warm-up call before graph capture")
        if buf is not None:
            _retired.append(buf)
        buf = torch.zeros(max(nbytes, _family_bytes(family)), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def status_word(device: torch.device | None = None) -> int:
    """Synchronise and return the largest device-side status word over the scratches handed out by
    ``scratch_for`` (0: no bounded wait expired); nothing is raised or re-zeroed."""
    torch.cuda.synchronize(device)
    return max((int(buf[:4].view(torch.int32)[0]) for buf in _scratch.values()), default=0)


def check_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if a bounded device-side wait expired in any kernel that used a scratch
    handed out by ``scratch_for`` (status word 1: W3 GEMV staging, 3: tensor-core kernel); the scratch
    is re-zeroed, the results of the calls since the last check are invalid."""
    torch.cuda.synchronize(device)
    bad = {}
    for key, buf in _scratch.items():
        code = int(buf[:4].view(torch.int32)[0])
        if code:
            bad[key] = code
            buf.zero_()
    if bad:
        raise NativeError(f"a device-side wait expired: {bad}; scratch re-zeroed")


def w3_gemv(x, planes, scales, zeros, perm, out, *, decoded_bf16=False, group_partials=False,
            pdl=True, scratch=None) -> None:
    """Raw launch: x [M,K], planes [G,3,O,16], scales [G,O], out [M,O]; see the header.

    With ``group_partials`` ``out`` is the fp32 ``[G,O]`` workspace of the two-call form."""
    m, k = x.shape
    o = planes.shape[2]
    need = w3_scratch_bytes(m, o, k)
    if _os.environ.get("FB_NO_PDL"):
        pdl = False
    # Consecutive Linears on the SAME activations (k_proj and v_proj behind q_proj, up_proj behind gate_proj): the
    # launch ahead is a W3 GEMV that read this very buffer, so the buffer was complete before that launch began and
    # this one need not wait for it (FB_W3_SAME_INPUT).  Such launches may overlap, so each takes its own scratch
    # (three rotate; a fourth launch in a row waits again).  Any other call into the library in between, a scratch
    # or a column order chosen by the caller, or several rows switch this off.
    key = (x.device.index if x.device.index is not None else torch.cuda.current_device(), torch.cuda.current_stream(x.device).cuda_stream)
    ahead = _same_input.get(key)
    here = (x.data_ptr(), tuple(x.shape), x.dtype)
    follow = (ahead is not None and ahead[0] == here and ahead[1] < 3 and scratch is None and pdl and m == 1 and perm is None
              and not group_partials and not _os.environ.get("FB_NO_SAME_INPUT"))
    slot = ahead[1] if follow else 0
    own_scratch = scratch is None
    if own_scratch:
        scratch = scratch_for(x.device, need, "w3" if slot == 0 else f"w3#{slot}")
    flags = (FB_W3_DECODED_BF16 if decoded_bf16 else 0) | (0 if pdl else FB_W3_NO_PDL) | (
        FB_W3_GROUP_PARTIALS if group_partials else 0) | (FB_W3_SAME_INPUT if follow else 0)
    with torch.cuda.device(x.device):
        check(library().fb_w3_gemv(
            ptr(x), dtype_tag(x.dtype), m, ptr(planes), ptr(scales), dtype_tag(scales.dtype),
            ptr(zeros), ptr(perm), ptr(out), o, k, ptr(scratch), scratch.numel() * scratch.element_size(),
            flags, stream_handle(x.device)))
    if own_scratch and pdl and m == 1 and perm is None and not group_partials:
        _same_input[key] = (here, slot + 1)


def w3_finish(partials, out) -> None:
    """out[0, o] = sum over rows of partials[:, o] (ascending), cast to out's dtype."""
    splits, o = partials.shape
    with torch.cuda.device(out.device):
        check(library().fb_w3_finish(ptr(partials), splits, o, ptr(out), dtype_tag(out.dtype),
                                     stream_handle(out.device)))


FB_W3_STATIC_SCRATCH_BYTES = 4 << 20


def w3_gemv_static(x, planes, scales, zeros, perm, out, *, decoded_bf16=False, pdl=True) -> None:
    """``w3_gemv`` through the entry point that uses the library's built-in scratch.

    For callers that cannot allocate device memory at the call site; nothing is allocated
    here either.  Rejects problems needing more than ``FB_W3_STATIC_SCRATCH_BYTES`` of
    scratch.  Calls on one device share that scratch, so they must not overlap on the GPU.
    """
    m, k = x.shape
    o = planes.shape[2]
    flags = (FB_W3_DECODED_BF16 if decoded_bf16 else 0) | (0 if pdl else FB_W3_NO_PDL)
    with torch.cuda.device(x.device):
        check(library().fb_w3_gemv_static(
            ptr(x), dtype_tag(x.dtype), m, ptr(planes), ptr(scales), dtype_tag(scales.dtype),
            ptr(zeros), ptr(perm), ptr(out), o, k, flags, stream_handle(x.device)))


def rmsnorm(x, weight, out, eps: float) -> None:
    """``out = weight * dtype(x * rsqrt(mean(x^2) + eps))`` over the last dimension of ``x``."""
    dim = x.shape[-1]
    with torch.cuda.device(x.device):
        check(library().fb_rmsnorm(ptr(x), ptr(weight), ptr(out), x.numel() // dim, dim, float(eps),
                                   dtype_tag(x.dtype), stream_handle(x.device)))


def rope_qk(q, k, cos, sin, q_out, k_out) -> None:
    """Rotary embedding of one position: ``q [Hq,D]``, ``k [Hk,D]`` (any leading unit dims), ``cos/sin [D]``."""
    dim = q.shape[-1]
    with torch.cuda.device(q.device):
        check(library().fb_rope_qk(ptr(q), ptr(k), ptr(cos), ptr(sin), ptr(q_out), ptr(k_out),
                                   q.numel() // dim, k.numel() // dim, dim, dtype_tag(q.dtype), stream_handle(q.device)))


def bb_scratch_bytes(out_features: int, in_features: int, global_scales: bool) -> int:
    return int(library().fb_bb_gemv_scratch_bytes(out_features, in_features, int(global_scales)))


def bb_gemv(x, layout, out, *, pdl=True, scratch=None) -> None:
    """Two-base GEMV on the reference's kernel layout (dict with the eight layout fields)."""
    codes = layout["codes"]
    groups, o = codes.shape[0], codes.shape[1]
    k = groups * 128
    if scratch is None:
        scratch = scratch_for(x.device, bb_scratch_bytes(o, k, False), "bb")
    with torch.cuda.device(x.device):
        check(library().fb_bb_gemv(
            ptr(x), dtype_tag(x.dtype), ptr(codes), int(codes.ndim == 4), ptr(layout["rows"]), ptr(layout["columns"]),
            ptr(layout["sparse_codes"]), ptr(layout["sparse_rows"]), ptr(layout["sparse_columns"]), ptr(layout["indices"]),
            ptr(out), o, k, ptr(scratch), scratch.numel() * scratch.element_size(), 0 if pdl else FB_W3_NO_PDL,
            stream_handle(x.device)))


def bb_global_gemv(x, codes, row_scales, col_scales, salient_idx, salient, out, *, pdl=True, scratch=None) -> None:
    """Two-base GEMV with matrix-wide fp16 scales and dense bf16 residual columns."""
    groups, o = codes.shape[0], codes.shape[1]
    k = groups * 128
    if scratch is None:
        scratch = scratch_for(x.device, bb_scratch_bytes(o, k, True), "bb")
    n_sal = 0 if salient_idx is None else salient_idx.numel()
    with torch.cuda.device(x.device):
        check(library().fb_bb_global_gemv(
            ptr(x), dtype_tag(x.dtype), ptr(codes), ptr(row_scales), ptr(col_scales), ptr(salient_idx), ptr(salient),
            n_sal, ptr(out), o, k, ptr(scratch), scratch.numel() * scratch.element_size(), 0 if pdl else FB_W3_NO_PDL,
            stream_handle(x.device)))


def _addr(tensor):
    return None if tensor is None else tensor.data_ptr()


def w3_matrix_list(entries):
    """Build the C array for ``w3_gemv_multi`` from ``(planes, scales, zeros, out, residual)`` tuples.

    Keep the returned array (and the tensors) alive for as long as launches use it."""
    array = (W3Matrix * len(entries))()
    for slot, (planes, scales, zeros, out, residual) in zip(array, entries):
        slot.planes, slot.scales, slot.zeros = _addr(planes), _addr(scales), _addr(zeros)
        slot.out, slot.residual, slot.out_features = _addr(out), _addr(residual), planes.shape[2]
    return array


def w3_gemv_multi(x, matrices, n_matrices, total_out, scale_dtype, perm, *, decoded_bf16=False, pdl=True, scratch=None) -> None:
    """One launch for several matrices sharing ``x`` ``[M,K]``; ``matrices`` from ``w3_matrix_list``."""
    m, k = x.shape
    if scratch is None:
        scratch = scratch_for(x.device, w3_scratch_bytes(m, total_out, k))
    flags = (FB_W3_DECODED_BF16 if decoded_bf16 else 0) | (0 if pdl else FB_W3_NO_PDL)
    with torch.cuda.device(x.device):
        check(library().fb_w3_gemv_multi(ptr(x), dtype_tag(x.dtype), m, matrices, n_matrices, dtype_tag(scale_dtype),
                                         ptr(perm), k, ptr(scratch), scratch.numel() * scratch.element_size(), flags,
                                         stream_handle(x.device)))


def qknorm_rope_cache(q, k, v, q_weight, k_weight, cos, sin, q_out, k_cache, v_cache, position: int, eps: float) -> None:
    """Per-head RMSNorm of q/k, rotary embedding, and the KV-cache write of one token (see the header)."""
    dim = q_weight.numel()
    with torch.cuda.device(q.device):
        check(library().fb_qknorm_rope_cache(ptr(q), ptr(k), ptr(v), ptr(q_weight), ptr(k_weight), ptr(cos), ptr(sin), ptr(q_out),
                                             ptr(k_cache), ptr(v_cache), q.numel() // dim, k.numel() // dim, dim, int(position),
                                             k_cache.shape[-2], float(eps), dtype_tag(q.dtype), stream_handle(q.device)))


def attn_scratch_bytes(q_heads: int) -> int:
    return int(library().fb_attn_decode_scratch_bytes(q_heads))


def attn_decode(q, k_cache, v_cache, out, length: int, scale: float, scratch) -> None:
    """Single-query attention over cache positions ``0..length-1``; ``scratch``: zeroed uint8 buffer of ``attn_scratch_bytes``."""
    dim = k_cache.shape[-1]
    with torch.cuda.device(q.device):
        check(library().fb_attn_decode(ptr(q), ptr(k_cache), ptr(v_cache), ptr(out), q.numel() // dim, k_cache.shape[-3], dim,
                                       int(length), k_cache.shape[-2], float(scale), dtype_tag(q.dtype), ptr(scratch),
                                       scratch.numel(), stream_handle(q.device)))


def attn_decode_fused(q, k, v, q_weight, k_weight, cos, sin, k_cache, v_cache, out, position: int, eps: float, scale: float,
                      scratch) -> None:
    """``qknorm_rope_cache`` + ``attn_decode`` in one launch: raw q/k/v rows of the token at ``position``;
    writes cache row ``position`` and attends over positions ``0..position``."""
    dim = k_cache.shape[-1]
    with torch.cuda.device(q.device):
        check(library().fb_attn_decode_fused(ptr(q), ptr(k), ptr(v), ptr(q_weight), ptr(k_weight), ptr(cos), ptr(sin), ptr(k_cache),
                                             ptr(v_cache), ptr(out), q.numel() // dim, k_cache.shape[-3], dim, int(position),
                                             k_cache.shape[-2], float(eps), float(scale), dtype_tag(q.dtype), ptr(scratch),
                                             scratch.numel(), stream_handle(q.device)))


def attn_decode_partial(q, k, v, q_weight, k_weight, cos, sin, k_cache, v_cache, position: int, eps: float, scale: float,
                        partials) -> int:
    """``attn_decode_fused`` without its last step: every CTA leaves its share (output, max, sum) in ``partials``
    (uint8, ``attn_scratch_bytes`` long) for ``w3_gemv_attn_merge``.  Returns the number of splits per head."""
    dim = k_cache.shape[-1]
    with torch.cuda.device(q.device):
        check(library().fb_attn_decode_partial(ptr(q), ptr(k), ptr(v), ptr(q_weight), ptr(k_weight), ptr(cos), ptr(sin), ptr(k_cache),
                                               ptr(v_cache), q.numel() // dim, k_cache.shape[-3], dim, int(position), k_cache.shape[-2],
                                               float(eps), float(scale), dtype_tag(q.dtype), ptr(partials), partials.numel(),
                                               stream_handle(q.device)))
    return int(library().fb_attn_decode_splits(int(position) + 1))


def w3_gemv_attn_merge(partials, splits: int, act_dtype, in_features: int, matrices, n_matrices, total_out, scale_dtype, *,
                       scratch=None, decoded_bf16=False) -> None:
    """``w3_gemv_multi`` for one activation row that is the attention output still in ``splits`` pieces per head
    (``attn_decode_partial``); the pieces are merged while the tables are built."""
    if scratch is None:
        scratch = scratch_for(partials.device, w3_scratch_bytes(1, total_out, in_features))
    with torch.cuda.device(partials.device):
        check(library().fb_w3_gemv_attn_merge(ptr(partials), int(splits), dtype_tag(act_dtype), matrices, n_matrices, dtype_tag(scale_dtype),
                                              int(in_features), ptr(scratch), scratch.numel() * scratch.element_size(),
                                              FB_W3_DECODED_BF16 if decoded_bf16 else 0, stream_handle(partials.device)))


def silu_mul(gate, up, out) -> None:
    with torch.cuda.device(gate.device):
        check(library().fb_silu_mul(ptr(gate), ptr(up), ptr(out), gate.numel(), dtype_tag(gate.dtype), stream_handle(gate.device)))


W3_INPUT_RMSNORM, W3_INPUT_SILU_MUL, W3_INPUT_ATTN_PIECES = 1, 2, 3


def w3_gemv_fused_input(x, transform: int, operand, eps: float, matrices, n_matrices, total_out, scale_dtype, *,
                        pdl=True, scratch=None, decoded_bf16=False) -> None:
    """``w3_gemv_multi`` for one activation row whose producer (RMSNorm or the SwiGLU gate) runs inside the launch."""
    k = x.shape[-1]
    if scratch is None:
        scratch = scratch_for(x.device, w3_scratch_bytes(1, total_out, k))
    with torch.cuda.device(x.device):
        check(library().fb_w3_gemv_fused_input(ptr(x), dtype_tag(x.dtype), transform, ptr(operand), float(eps), matrices, n_matrices,
                                               dtype_tag(scale_dtype), k, ptr(scratch), scratch.numel() * scratch.element_size(),
                                               (0 if pdl else FB_W3_NO_PDL) | (FB_W3_DECODED_BF16 if decoded_bf16 else 0),
                                               stream_handle(x.device)))


def w3_gemm_small(x, planes, scales, zeros, perm, out, *, scratch=None) -> None:
    """Tensor-core form for ``x`` of 1..16 rows: x [M,K], planes [G,3,O,16], scales [G,O], out [M,O]."""
    m, k = x.shape
    o = planes.shape[2]
    if scratch is None:
        scratch = scratch_for(x.device, library().fb_w3_gemm_small_scratch_bytes(m, o, k), "w3mma")
    with torch.cuda.device(x.device):
        check(library().fb_w3_gemm_small(ptr(x), dtype_tag(x.dtype), m, ptr(planes), ptr(scales), dtype_tag(scales.dtype),
                                         ptr(zeros) if zeros is not None else None, ptr(perm) if perm is not None else None,
                                         ptr(out), o, k, ptr(scratch), scratch.numel() * scratch.element_size(),
                                         stream_handle(x.device)))


def w3_push_descriptor(data_ptrs) -> W3Push:
    """``fb_w3_push_t`` from one slot-array pointer per rank (plain integers)."""
    push = W3Push()
    push.world = len(data_ptrs)
    for r, data in enumerate(data_ptrs):
        push.data[r] = data
    return push


def w3_gemv_push(x, transform: int, operand, eps: float, matrix, k: int, scale_dtype, push: W3Push, *, scratch, pdl=True,
                 decoded_bf16=False, act_dtype=None) -> None:
    """Row-split Linear of a tensor-parallel rank: results go to every rank's exchange buffer (see the header).
    With ``W3_INPUT_ATTN_PIECES`` ``x`` is the pieces buffer of ``attn_decode_partial``, ``eps`` the splits per head and
    ``act_dtype`` the activation dtype."""
    with torch.cuda.device(x.device):
        check(library().fb_w3_gemv_push(ptr(x), dtype_tag(x.dtype if act_dtype is None else act_dtype), transform, ptr(operand), float(eps), matrix, dtype_tag(scale_dtype), k,
                                        ctypes.byref(push), ptr(scratch), scratch.numel() * scratch.element_size(),
                                        (0 if pdl else FB_W3_NO_PDL) | (FB_W3_DECODED_BF16 if decoded_bf16 else 0),
                                        stream_handle(x.device)))


def tp_reduce(parts_ptr: int, world: int, residual, out, status_ptr: int, wait_ns: int = 0) -> None:
    """Receiving half of the push: polls every rank's slots, sums their rows, adds the residual.

    ``wait_ns`` bounds the poll (0 = the library default of ten seconds); on expiry the status word
    becomes 4 and the kernel returns."""
    with torch.cuda.device(out.device):
        check(library().fb_tp_reduce(ctypes.c_void_p(parts_ptr), world, ptr(residual), ptr(out), out.numel(), dtype_tag(out.dtype),
                                     ctypes.c_void_p(status_ptr), int(wait_ns), stream_handle(out.device)))


def lm_head_scratch_bytes() -> int:
    return int(library().fb_lm_head_scratch_bytes())


def lm_head_argmax(x, norm_weight, eps: float, weight, best, *, logits=None, forced_next=None, embedding=None, next_hidden=None,
                   scratch) -> None:
    """Greedy LM head in one launch: optional final RMSNorm of ``x [1,K]``, ``weight [V,K]`` GEMV, argmax into
    ``best`` (int64 ``[1]``); optionally the 16-bit logits, and the embedding row of the next token
    (``forced_next`` int64 ``[1]`` on the device, else the choice) copied into ``next_hidden``."""
    vocab, k = weight.shape
    with torch.cuda.device(x.device):
        check(library().fb_lm_head_argmax(ptr(x), ptr(norm_weight), float(eps), ptr(weight), vocab, k, dtype_tag(x.dtype), ptr(logits),
                                          ptr(best), ptr(forced_next), ptr(embedding), ptr(next_hidden), ptr(scratch),
                                          scratch.numel() * scratch.element_size(), stream_handle(x.device)))


def lm_head_shard(x, norm_weight, eps: float, weight_shard, row_base: int, keys: W3Push, rank: int, *, logits_shard=None, scratch) -> None:
    """The LM head over one rank's rows of the vocabulary (``weight_shard [V/p, K]``, a contiguous row range starting at
    ``row_base``): the shard's best key goes to slot ``rank`` of every rank's key array; follow with ``tp_argmax``."""
    rows, k = weight_shard.shape
    with torch.cuda.device(x.device):
        check(library().fb_lm_head_shard(ptr(x), ptr(norm_weight), float(eps), ptr(weight_shard), rows, int(row_base), k, dtype_tag(x.dtype),
                                         ptr(logits_shard), ctypes.byref(keys), int(rank), ptr(scratch), scratch.numel() * scratch.element_size(),
                                         stream_handle(x.device)))


def tp_argmax(keys_ptr: int, world: int, best, status_ptr: int, *, forced_next=None, embedding=None, next_hidden=None, wait_ns: int = 0) -> None:
    """Receiving half of ``lm_head_shard``: the largest of the ``world`` delivered keys becomes ``best`` (int64 ``[1]``); optionally
    the embedding row of ``forced_next`` (or of the choice) is copied into ``next_hidden``.  Bounded poll, status 6 on expiry."""
    vocab, k = embedding.shape if embedding is not None else (0, 0)
    with torch.cuda.device(best.device):
        check(library().fb_tp_argmax(ctypes.c_void_p(keys_ptr), world, ptr(best), ptr(forced_next), ptr(embedding), ptr(next_hidden), vocab, k,
                                     ctypes.c_void_p(status_ptr), int(wait_ns), stream_handle(best.device)))


def embed_row(embedding, token, out) -> None:
    """``out[0, :] = embedding[token[0], :]`` for a token id held on the device (int64 ``[1]``)."""
    vocab, k = embedding.shape
    with torch.cuda.device(out.device):
        check(library().fb_embed_row(ptr(embedding), ptr(token), ptr(out), vocab, k, stream_handle(out.device)))
