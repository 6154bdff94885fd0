"""Single-kernel RMSNorm and rotary embedding for the stock HF Qwen3 decode path.

Mirror of the reference's ``fused_modules`` (``src/fluxbin_style/fused_modules.py:30-112``):
same function names and the same context manager that patches
``Qwen3RMSNorm.forward`` and ``modeling_qwen3.apply_rotary_pos_emb`` and restores them on exit.
The reference gets its RMSNorm fusion from ``torch.compile`` and its RoPE from tensor algebra;
here both are hand-written sm_100a kernels behind the C ABI (``fb_rmsnorm``, ``fb_rope_qk``).
The kernels serve CUDA fp16/bf16 tensors; the one-position RoPE kernel serves decode steps.
Anything else (CPU tensors, fp32, prefill with many positions) runs the same mathematics as
plain tensor operations, which is also what the patched functions compute in the reference.
"""
from __future__ import annotations

from contextlib import contextmanager

import torch

from . import _native


def rms_norm_reference(hidden_states, weight, eps):
    """The stock Qwen3RMSNorm arithmetic as a free function (fp32 statistics, cast, then weight)."""
    dtype = hidden_states.dtype
    wide = hidden_states.to(torch.float32)
    wide = wide * torch.rsqrt(wide.pow(2).mean(-1, keepdim=True) + eps)
    return weight * wide.to(dtype)


def _kernel_eligible(*tensors) -> bool:
    first = tensors[0]
    return (first.is_cuda and first.dtype in (torch.float16, torch.bfloat16) and not torch.is_grad_enabled()
            and all(t.is_cuda and t.dtype == first.dtype and t.is_contiguous() for t in tensors))


def fused_rms_norm(hidden_states, weight, eps):
    """RMSNorm in one kernel launch when the tensors are CUDA 16-bit, else the reference math."""
    if not _kernel_eligible(hidden_states, weight) or weight.numel() != hidden_states.shape[-1]:
        return rms_norm_reference(hidden_states, weight, eps)
    out = torch.empty_like(hidden_states)
    _native.rmsnorm(hidden_states, weight, out, eps)
    return out


def fused_rms_norm_forward(self, hidden_states):
    return fused_rms_norm(hidden_states, self.weight, self.variance_epsilon)


def _rope_algebra(q, k, cos, sin, unsqueeze_dim):
    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    q_heads = q.shape[unsqueeze_dim]
    both = torch.cat((q, k), dim=unsqueeze_dim)
    half = both.shape[-1] // 2
    turned = torch.cat((-both[..., half:], both[..., :half]), dim=-1)
    result = torch.addcmul(both * cos, turned, sin)
    return result.narrow(unsqueeze_dim, 0, q_heads), result.narrow(unsqueeze_dim, q_heads, k.shape[unsqueeze_dim])


def fused_apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1):
    """Rotate q and k together.  One kernel for a single position on CUDA, tensor algebra otherwise."""
    if q.ndim != k.ndim or q.dtype != k.dtype or q.shape[-1] != k.shape[-1]:
        raise ValueError("fused RoPE requires q/k with matching rank, dtype and head_dim")
    dim = q.shape[-1]
    single_position = cos.numel() == dim and sin.numel() == dim and q.numel() == q.shape[unsqueeze_dim] * dim \
        and k.numel() == k.shape[unsqueeze_dim] * dim
    if single_position and dim % 2 == 0 and _kernel_eligible(q, k, cos, sin):
        q_out, k_out = torch.empty_like(q), torch.empty_like(k)
        _native.rope_qk(q, k, cos, sin, q_out, k_out)
        return q_out, k_out
    return _rope_algebra(q, k, cos, sin, unsqueeze_dim)


@contextmanager
def fused_qwen3_modules(*, rms_norm=True, rope=True):
    """Patch the HF Qwen3 RMSNorm class and rotary function in place; restore on exit or error.

    The patch is at class / module scope on purpose, so every arm of a comparison built
    from ``transformers`` shares the same non-Linear path.
    """
    from transformers.models.qwen3 import modeling_qwen3

    applied = {"rms_norm": bool(rms_norm), "rope": bool(rope)}
    saved = {}
    try:
        if rms_norm:
            saved["rms_norm"] = modeling_qwen3.Qwen3RMSNorm.forward
            modeling_qwen3.Qwen3RMSNorm.forward = fused_rms_norm_forward
        if rope:
            saved["rope"] = modeling_qwen3.apply_rotary_pos_emb
            modeling_qwen3.apply_rotary_pos_emb = fused_apply_rotary_pos_emb
        yield applied
    finally:
        if "rms_norm" in saved:
            modeling_qwen3.Qwen3RMSNorm.forward = saved["rms_norm"]
        if "rope" in saved:
            modeling_qwen3.apply_rotary_pos_emb = saved["rope"]
