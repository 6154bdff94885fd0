"""The scratch-free entry point ``fb_w3_gemv_static``: for hosts that cannot allocate device
memory where they call the library (memory fully pooled elsewhere, a framework allocator they
must not bypass, a graph capture in progress).  Its results must equal those of ``fb_w3_gemv``
with a caller-owned scratch, call after call, because both run the same kernel; only the home
of the split-K scratch differs.  Collected last on purpose: a failure here stops nothing else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(o, k, seed, m=1):
    gen = torch.Generator().manual_seed(seed)
    groups = k // 128
    planes = torch.randint(0, 256, (groups, 3, o, 16), generator=gen, dtype=torch.uint8).cuda()
    scales = (torch.rand(groups, o, generator=gen) * 0.015 + 0.005).half().cuda()
    zeros = torch.randint(3, 5, (groups, o), generator=gen, dtype=torch.uint8).cuda()
    x = torch.randn(m, k, generator=gen).bfloat16().cuda()
    return x, planes, scales, zeros


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    from marlin_style_fluxbin_b200 import _native

    for call, (o, k) in enumerate(((1024, 2048), (4096, 4096))):  # 8 and 16 K blocks: split-K in use
        x, planes, scales, zeros = _problem(o, k, seed=40 + call)
        expected = torch.full((1, o), float("nan"), device="cuda", dtype=torch.bfloat16)
        scratch = torch.zeros(_native.w3_scratch_bytes(1, o, k), dtype=torch.uint8, device="cuda")
        _native.w3_gemv(x, planes, scales, zeros, None, expected, scratch=scratch)
        for repeat in range(2):  # the second call meets whatever the first left in the array
            got = torch.full((1, o), float("nan"), device="cuda", dtype=torch.bfloat16)
            _native.w3_gemv_static(x, planes, scales, zeros, None, got)
            torch.cuda.synchronize()
            assert bool(torch.isfinite(got).all()), (o, k, repeat)
            torch.testing.assert_close(got.float(), expected.float(), rtol=0, atol=0)


def test_static_scratch_with_several_rows_and_with_a_long_k():
    """Four activation rows use four times the combine words; K = 12288 makes a CTA walk three K
    blocks (running sums in registers, or in the partials area of the array behind the combine words)."""
    from marlin_style_fluxbin_b200 import _native

    for o, k, m in ((2048, 1024, 4), (4096, 12288, 1), (1024, 12288, 2)):
        x, planes, scales, zeros = _problem(o, k, seed=o + k + m, m=m)
        assert _native.w3_scratch_bytes(m, o, k) <= _native.FB_W3_STATIC_SCRATCH_BYTES
        expected = torch.full((m, o), float("nan"), device="cuda", dtype=torch.bfloat16)
        scratch = torch.zeros(_native.w3_scratch_bytes(m, o, k), dtype=torch.uint8, device="cuda")
        _native.w3_gemv(x, planes, scales, zeros, None, expected, scratch=scratch)
        for _ in range(2):
            got = torch.full((m, o), float("nan"), device="cuda", dtype=torch.bfloat16)
            _native.w3_gemv_static(x, planes, scales, zeros, None, got)
            torch.cuda.synchronize()
            assert torch.equal(got, expected), (o, k, m)
    if torch.cuda.device_count() > 1:  # the array exists once per GPU: its address is looked up per device
        with torch.cuda.device(1):
            x, planes, scales, zeros = (t.to("cuda:1") for t in _problem(1024, 2048, seed=3))
            want = torch.empty(1, 1024, device="cuda:1", dtype=torch.bfloat16)
            _native.w3_gemv(x, planes, scales, zeros, None, want, scratch=torch.zeros(_native.w3_scratch_bytes(1, 1024, 2048), dtype=torch.uint8, device="cuda:1"))
            got = torch.empty_like(want)
            _native.w3_gemv_static(x, planes, scales, zeros, None, got)
            torch.cuda.synchronize("cuda:1")
            assert torch.equal(got, want)


def test_static_scratch_rejects_oversized_problem_without_launching():
    from marlin_style_fluxbin_b200 import _native

    o, k = 65536, 32640  # 255 groups are walked as 16 super-blocks: 16 x 65536 fp32 partials = 4 MiB, plus the combine words
    assert _native.w3_scratch_bytes(1, o, k) > _native.FB_W3_STATIC_SCRATCH_BYTES
    x, planes, scales, zeros = _problem(64, 256, seed=1)
    out = torch.zeros(1, 64, device="cuda", dtype=torch.bfloat16)
    # pointers are never dereferenced: the size check comes first
    import ctypes

    code = _native.library().fb_w3_gemv_static(
        _native.ptr(x), 1, 1, _native.ptr(planes), _native.ptr(scales), 0, None, None, _native.ptr(out), o, k, 0,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert code == -2
    assert b"built-in scratch holds" in _native.library().fb_last_error()
    assert float(out.abs().max()) == 0.0
