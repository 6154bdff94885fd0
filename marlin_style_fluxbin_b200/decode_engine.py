"""Batch-1 Qwen3 decode engine on the packed W3 kernels: five launches per layer, one CUDA graph.

The reference drives an unmodified HF ``Qwen3ForCausalLM`` whose Linears were swapped
(``static_decode.py:15-138``); that drop-in route is kept in ``static_decode.py`` here.  This
engine is the B200-first route for the same decode step: fused q/k/v and gate/up GEMV launches,
residual adds folded into the o/down GEMV epilogues, one kernel each for RMSNorm, q/k-norm +
RoPE + KV-cache write, single-query attention and the SwiGLU gate, all chained with programmatic
dependent launch and captured, for a whole continuation, in one CUDA graph.

The same engine runs a BF16 arm (dense dequantised weights through cuBLAS, identical glue
kernels), which is the same-box baseline the packed path is compared with, and shards itself
tensor-parallel: q/k/v/gate/up by output rows, o/down by input groups; after each of the two
row-split GEMVs of a layer the packed arm pushes its rows into every rank's exchange buffer from
the GEMV epilogue (``tp_push``), the BF16 arm runs an NCCL sum-allreduce.

Both arms end a step with the same LM-head launch (final RMSNorm, dense 16-bit GEMV, argmax and
the next token's embedding row in one kernel).  ``truth_logits`` runs the same model in fp32
(activations and dequantised weights) as the yardstick either arm is measured against.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch.nn import functional as F

from . import _native
from .gptq_deployment import restore_planar_w3


@dataclass(frozen=True)
class ModelShape:
    layers: int
    hidden: int
    q_heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rope_theta: float = 1e6
    eps: float = 1e-6

    @property
    def q_width(self):
        return self.q_heads * self.head_dim

    @property
    def kv_width(self):
        return self.kv_heads * self.head_dim


QWEN3_8B = ModelShape(36, 4096, 32, 8, 128, 12288, 151936)
QWEN3_32B = ModelShape(64, 5120, 64, 8, 128, 25600, 151936)


def synthetic_w3(out_features, in_features, device, generator):
    """A W3 g128 Linear drawn as the benchmark configs state: uniform codes (uniform random
    plane bytes), fp16 scales U(0.005, 0.02), zero points in {3, 4}, contiguous groups."""
    groups = in_features // 128
    return {
        "planes": torch.randint(0, 256, (groups, 3, out_features, 16), dtype=torch.uint8, device=device, generator=generator),
        "scales": (torch.rand(groups, out_features, device=device, generator=generator) * 0.015 + 0.005).half(),
        "zeros": torch.randint(3, 5, (groups, out_features), dtype=torch.uint8, device=device, generator=generator),
        "perm": torch.arange(in_features, dtype=torch.int16, device=device),
    }


def shard_rows(layout, rank, size):
    """Column-parallel shard: a contiguous slice of the output rows (all groups)."""
    o = layout["planes"].shape[2]
    lo, hi = rank * o // size, (rank + 1) * o // size
    return {"planes": layout["planes"][:, :, lo:hi].contiguous(), "scales": layout["scales"][:, lo:hi].contiguous(),
            "zeros": layout["zeros"][:, lo:hi].contiguous(), "perm": layout["perm"]}


def shard_groups(layout, rank, size):
    """Row-parallel shard: a contiguous slice of the input groups (all output rows)."""
    g = layout["planes"].shape[0]
    lo, hi = rank * g // size, (rank + 1) * g // size
    return {"planes": layout["planes"][lo:hi].contiguous(), "scales": layout["scales"][lo:hi].contiguous(),
            "zeros": layout["zeros"][lo:hi].contiguous(), "perm": torch.arange((hi - lo) * 128, dtype=torch.int16, device=layout["perm"].device)}


def head_key(logit: float, row: int) -> int:
    """The 64-bit key under which the LM-head kernels compare candidates (host mirror of the device code):
    the fp32 bits of the (16-bit rounded) logit mapped to an unsigned order in the high word, ``2^32 - 1 - row``
    in the low word, so that the largest key is the largest logit and, among equals, the lowest row, which is
    ``torch.argmax``'s rule.  Keys of vocabulary shards compare across ranks because ``row`` is the global row."""
    import struct

    bits = struct.unpack("<I", struct.pack("<f", float(logit)))[0]
    ordered = (~bits & 0xFFFFFFFF) if bits & 0x80000000 else (bits | 0x80000000)
    return (ordered << 32) | (0xFFFFFFFF - int(row))


def head_key_row(key: int) -> int:
    return 0xFFFFFFFF - (int(key) & 0xFFFFFFFF)


class _Layer:
    __slots__ = ("q", "k", "v", "o", "gate", "up", "down", "ln1", "ln2", "q_norm", "k_norm", "dense", "qkv_list", "gu_list", "o_list", "down_list",
                 "o_push", "down_push")


class DecodeEngine:
    """``arm`` is ``"w3"`` (packed kernels) or ``"bf16"`` (dense dequantised weights, cuBLAS)."""

    def __init__(self, shape: ModelShape, *, device, max_positions: int, arm: str = "w3", seed: int = 20260916,
                 tp_rank: int = 0, tp_size: int = 1, group=None, dtype=torch.bfloat16, fuse_inputs: bool = True,
                 fuse_attention: bool = True, tp_push: bool | None = None, arithmetic: str = "structural"):
        if arm not in ("w3", "bf16"):
            raise ValueError("arm must be w3 or bf16")
        if arithmetic not in ("structural", "decoded_bf16"):
            raise ValueError("arithmetic must be structural or decoded_bf16")
        # packed arm: "decoded_bf16" follows the weight dequantised in the scale's dtype
        # (the reference's fast_corrected route), "structural" is scale * integer dot
        self.decoded = arithmetic == "decoded_bf16"
        if shape.q_heads % tp_size or shape.kv_heads % tp_size or (shape.hidden // 128) % tp_size or (shape.intermediate // 128) % tp_size:
            raise ValueError("heads and group counts must divide by the tensor-parallel size")
        self.shape, self.device, self.arm, self.dtype = shape, torch.device(device), arm, dtype
        self.tp_rank, self.tp_size, self.group = tp_rank, tp_size, group
        self.max_positions = max_positions
        # RMSNorm and the SwiGLU gate run inside the GEMV that consumes them (w3 arm only)
        self.fuse_inputs = fuse_inputs
        # q/k-norm, RoPE and the cache write run inside the attention launch (both arms)
        self.fuse_attention = fuse_attention
        # tensor parallel, packed arm: the row-split GEMVs push their rows straight into every
        # rank's exchange buffer (peer stores over NVLink) and a small kernel sums them, instead
        # of an NCCL allreduce between the two Linears.  Off: NCCL allreduce.
        self.tp_push = (tp_size > 1 and arm == "w3") if tp_push is None else (tp_push and tp_size > 1 and arm == "w3")
        s, p = shape, tp_size
        self.q_heads, self.kv_heads = s.q_heads // p, s.kv_heads // p
        self.inter = s.intermediate // p
        gen = torch.Generator(device=self.device).manual_seed(seed)  # same stream of draws on every rank
        normal = lambda *size: (torch.randn(*size, device=self.device, generator=gen) * 0.02).to(dtype)  # noqa: E731
        self.embedding = normal(s.vocab, s.hidden)
        self.lm_head = normal(s.vocab, s.hidden)
        self.final_norm = torch.ones(s.hidden, device=self.device, dtype=dtype)
        self.layers = []
        for _ in range(s.layers):
            layer = _Layer()
            full = {name: synthetic_w3(o, k, self.device, gen) for name, o, k in (
                ("q", s.q_width, s.hidden), ("k", s.kv_width, s.hidden), ("v", s.kv_width, s.hidden), ("o", s.hidden, s.q_width),
                ("gate", s.intermediate, s.hidden), ("up", s.intermediate, s.hidden), ("down", s.hidden, s.intermediate))}
            for name in ("q", "k", "v", "gate", "up"):
                setattr(layer, name, shard_rows(full[name], tp_rank, p))
            for name in ("o", "down"):
                setattr(layer, name, shard_groups(full[name], tp_rank, p))
            del full
            layer.ln1 = torch.ones(s.hidden, device=self.device, dtype=dtype)
            layer.ln2 = torch.ones(s.hidden, device=self.device, dtype=dtype)
            layer.q_norm = torch.ones(s.head_dim, device=self.device, dtype=dtype)
            layer.k_norm = torch.ones(s.head_dim, device=self.device, dtype=dtype)
            layer.dense = self._dense(layer) if arm == "bf16" else None
            self.layers.append(layer)
        # rotary table, fp32 angles cast to the activation dtype (as the HF rotary module does)
        inv_freq = 1.0 / (s.rope_theta ** (torch.arange(0, s.head_dim, 2, device=self.device, dtype=torch.float32) / s.head_dim))
        angles = torch.arange(max_positions, device=self.device, dtype=torch.float32)[:, None] * inv_freq[None, :]
        angles = torch.cat((angles, angles), dim=-1)
        self.cos, self.sin = angles.cos().to(dtype).contiguous(), angles.sin().to(dtype).contiguous()
        self.k_cache = torch.zeros(s.layers, self.kv_heads, max_positions, s.head_dim, device=self.device, dtype=dtype)
        self.v_cache = torch.zeros_like(self.k_cache)
        # activation buffers of one token
        buf = lambda n: torch.zeros(1, n, device=self.device, dtype=dtype)  # noqa: E731
        self.h, self.h_next, self.xn = buf(s.hidden), buf(s.hidden), buf(s.hidden)
        # q/k/v and gate/up live side by side, so that the dense arm's fused GEMMs write them in place
        qw, kw = self.q_heads * s.head_dim, self.kv_heads * s.head_dim
        self.qkv, self.gate_up = buf(qw + 2 * kw), buf(2 * self.inter)
        self.q, self.k, self.v = self.qkv[:, :qw], self.qkv[:, qw:qw + kw], self.qkv[:, qw + kw:]
        self.gate, self.up = self.gate_up[:, :self.inter], self.gate_up[:, self.inter:]
        self.q_rot, self.attn, self.act = buf(qw), buf(qw), buf(self.inter)
        self.logits = torch.zeros(1, s.vocab, device=self.device, dtype=dtype)
        self.next_token = torch.zeros(1, dtype=torch.long, device=self.device)
        self.head_scratch = torch.zeros(_native.lm_head_scratch_bytes(), dtype=torch.uint8, device=self.device)
        self.keep_logits = True      # False: the 16-bit logits never leave the chip (greedy decode only)
        self._h_is_embedded = False  # the LM head of the previous step already wrote the next embedding row into h
        self.launches_per_step = 0
        self.attn_scratch = torch.zeros(_native.attn_scratch_bytes(self.q_heads), dtype=torch.uint8, device=self.device)
        if arm == "w3":
            self._build_matrix_lists()
        if self.tp_push:
            self._build_exchange()

    # ------------------------------------------------------------------ weights
    def _dense(self, layer):
        """Dequantised 16-bit weights of this rank's shards (fused q/k/v and gate/up)."""
        d = lambda lay: restore_planar_w3(lay, dtype=self.dtype)  # noqa: E731
        return {"qkv": torch.cat((d(layer.q), d(layer.k), d(layer.v)), 0), "o": d(layer.o),
                "gate_up": torch.cat((d(layer.gate), d(layer.up)), 0), "down": d(layer.down)}

    def _build_matrix_lists(self):
        first = self.tp_rank == 0  # the residual is added by exactly one rank before the allreduce
        for layer in self.layers:
            entry = lambda lay, out, residual=None: (lay["planes"], lay["scales"], lay["zeros"], out, residual)  # noqa: E731
            layer.qkv_list = _native.w3_matrix_list([entry(layer.q, self.q), entry(layer.k, self.k), entry(layer.v, self.v)])
            layer.gu_list = _native.w3_matrix_list([entry(layer.gate, self.gate), entry(layer.up, self.up)])
            layer.o_list = _native.w3_matrix_list([entry(layer.o, self.h_next, self.h if first else None)])
            layer.down_list = _native.w3_matrix_list([entry(layer.down, self.h, self.h_next if first else None)])
        need = max(_native.w3_scratch_bytes(1, 2 * self.inter, self.shape.hidden),
                   _native.w3_scratch_bytes(1, self.shape.hidden, self.inter))
        self.scratch = torch.zeros(need, dtype=torch.uint8, device=self.device)

    def _build_exchange(self):
        """Symmetric exchange buffer (one per rank, peer-mapped): for each of the two reduction
        sites of a layer, 8-byte (value, mark) slots [world, hidden]."""
        import torch.distributed._symmetric_memory as symm

        hidden, world = self.shape.hidden, self.tp_size
        header = 64  # 8-byte slots: a status word first, [8..16) the LM-head keys of the ranks, then [site][rank][hidden] (value, mark) pairs
        self._xchg = symm.empty(2 * (header + 2 * world * hidden), dtype=torch.float32, device=self.device)
        self._xchg.zero_()
        group = self.group if self.group is not None else torch.distributed.group.WORLD
        handle = symm.rendezvous(self._xchg, group.group_name)
        bases = [int(ptr) for ptr in handle.buffer_ptrs]
        torch.cuda.synchronize(self.device)
        torch.distributed.barrier(group=self.group)
        mine = bases[self.tp_rank]
        self._sites = []
        for site in range(2):
            data = 8 * (header + site * world * hidden)
            push = _native.w3_push_descriptor([base + data + 8 * self.tp_rank * hidden for base in bases])
            self._sites.append({"push": push, "parts": mine + data, "status": mine})
        # vocabulary-split LM head: every rank scans V / world rows and delivers its best key to every rank
        self.split_head = self.shape.vocab % world == 0
        if self.split_head:
            rows = self.shape.vocab // world
            self._head_rows = (self.tp_rank * rows, rows)
            self._head_keys = _native.w3_push_descriptor([base + 8 * 8 for base in bases])
            self._head_keys_mine = mine + 8 * 8
        for layer in self.layers:  # no residual in the GEMV: the reduce kernel adds it on every rank
            entry = lambda lay, out: (lay["planes"], lay["scales"], lay["zeros"], out, None)  # noqa: E731
            layer.o_push = _native.w3_matrix_list([entry(layer.o, self.h_next)])
            layer.down_push = _native.w3_matrix_list([entry(layer.down, self.h)])

    # ------------------------------------------------------------------ collectives
    def _allreduce(self, tensor):
        if self.tp_size > 1:
            torch.distributed.all_reduce(tensor, group=self.group)

    # ------------------------------------------------------------------ prefill (dense, not timed)
    @torch.inference_mode()
    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt through dense (dequantised) weights with plain tensor operations, fill
        the KV cache for positions ``0..T-1`` and return the logits of the last position."""
        s = self.shape
        tokens = input_ids.reshape(-1).to(self.device)
        t = tokens.numel()
        if not 1 <= t < self.max_positions:
            raise ValueError("prompt does not fit the KV cache")
        h = self.embedding[tokens]
        cos, sin = self.cos[:t].unsqueeze(0), self.sin[:t].unsqueeze(0)
        rotate = lambda x: torch.cat((-x[..., s.head_dim // 2:], x[..., :s.head_dim // 2]), dim=-1)  # noqa: E731
        norm = lambda x, w: (w * (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + s.eps)).to(self.dtype))  # noqa: E731
        for index, layer in enumerate(self.layers):
            dense = layer.dense if layer.dense is not None else self._dense(layer)
            x = norm(h, layer.ln1)
            qkv = F.linear(x, dense["qkv"])
            q, k, v = qkv.split((self.q_heads * s.head_dim, self.kv_heads * s.head_dim, self.kv_heads * s.head_dim), dim=-1)
            q = norm(q.reshape(t, self.q_heads, s.head_dim), layer.q_norm).transpose(0, 1)
            k = norm(k.reshape(t, self.kv_heads, s.head_dim), layer.k_norm).transpose(0, 1)
            v = v.reshape(t, self.kv_heads, s.head_dim).transpose(0, 1)
            q = q * cos + rotate(q) * sin
            k = k * cos + rotate(k) * sin
            self.k_cache[index, :, :t] = k
            self.v_cache[index, :, :t] = v
            attn = F.scaled_dot_product_attention(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), is_causal=True, enable_gqa=True)
            y = F.linear(attn[0].transpose(0, 1).reshape(t, -1), dense["o"])
            self._allreduce(y)
            h = h + y
            x = norm(h, layer.ln2)
            gate, up = F.linear(x, dense["gate_up"]).split(self.inter, dim=-1)
            y = F.linear(F.silu(gate) * up, dense["down"])
            self._allreduce(y)
            h = h + y
            del dense
        last = norm(h[-1:], self.final_norm)
        return F.linear(last, self.lm_head)

    # ------------------------------------------------------------------ one decode step
    @torch.inference_mode()
    def step(self, token: torch.Tensor, position: int, next_forced: torch.Tensor | None = None, embed_next: bool = False,
             choice_out: torch.Tensor | None = None) -> None:
        """Decode one token (``token``: device int64 ``[1]``) at ``position``; leaves the greedy choice in
        ``self.next_token`` (and the logits in ``self.logits`` while ``keep_logits``).  No allocation, no host sync.

        ``embed_next``: the LM-head launch also writes the embedding row of the next token (``next_forced``,
        a device int64 ``[1]``, or the greedy choice) into the hidden-state buffer, and the next ``step`` then
        skips its gather launch.  ``choice_out`` (device int64 ``[1]``) receives the greedy choice instead of
        ``self.next_token``."""
        s, nat = self.shape, _native
        w3 = self.arm == "w3"
        f16 = torch.float16
        launches = 0
        if not self._h_is_embedded:
            nat.embed_row(self.embedding, token, self.h)
            launches += 1
        cos, sin = self.cos[position], self.sin[position]
        scale = 1.0 / math.sqrt(s.head_dim)
        dec = self.decoded
        for index, layer in enumerate(self.layers):
            fuse = w3 and self.fuse_inputs
            if not fuse:
                nat.rmsnorm(self.h, layer.ln1, self.xn, s.eps)
            if fuse:
                nat.w3_gemv_fused_input(self.h, nat.W3_INPUT_RMSNORM, layer.ln1, s.eps, layer.qkv_list, 3,
                                        self.qkv.numel(), f16, scratch=self.scratch, decoded_bf16=dec)
            elif w3:
                nat.w3_gemv_multi(self.xn, layer.qkv_list, 3, self.qkv.numel(), f16, None, scratch=self.scratch, decoded_bf16=dec)
            else:
                torch.mm(self.xn, layer.dense["qkv"].t(), out=self.qkv)  # q, k, v are views of this buffer
            # packed arm, unsharded: the attention launch stops at per-split pieces and the o GEMV merges them in its table build
            merge_in_o = w3 and self.fuse_attention and (self.tp_push or self.tp_size == 1)
            if merge_in_o:
                splits = nat.attn_decode_partial(self.q, self.k, self.v, layer.q_norm, layer.k_norm, cos, sin, self.k_cache[index],
                                                 self.v_cache[index], position, s.eps, scale, self.attn_scratch)
            elif self.fuse_attention:
                nat.attn_decode_fused(self.q, self.k, self.v, layer.q_norm, layer.k_norm, cos, sin, self.k_cache[index],
                                      self.v_cache[index], self.attn, position, s.eps, scale, self.attn_scratch)
            else:
                nat.qknorm_rope_cache(self.q, self.k, self.v, layer.q_norm, layer.k_norm, cos, sin, self.q_rot,
                                      self.k_cache[index], self.v_cache[index], position, s.eps)
                nat.attn_decode(self.q_rot, self.k_cache[index], self.v_cache[index], self.attn, position + 1, scale, self.attn_scratch)
            if self.tp_push:
                site = self._sites[0]
                if merge_in_o:
                    nat.w3_gemv_push(self.attn_scratch, nat.W3_INPUT_ATTN_PIECES, None, float(splits), layer.o_push, self.attn.shape[-1], f16,
                                     site["push"], scratch=self.scratch, decoded_bf16=dec, act_dtype=self.dtype)
                else:
                    nat.w3_gemv_push(self.attn, 0, None, 0.0, layer.o_push, self.attn.shape[-1], f16, site["push"], scratch=self.scratch,
                                     decoded_bf16=dec)
                nat.tp_reduce(site["parts"], self.tp_size, self.h, self.h_next, site["status"])
            elif merge_in_o:
                nat.w3_gemv_attn_merge(self.attn_scratch, splits, self.dtype, self.attn.shape[-1], layer.o_list, 1, s.hidden, f16,
                                       scratch=self.scratch, decoded_bf16=dec)
            elif w3:
                nat.w3_gemv_multi(self.attn, layer.o_list, 1, s.hidden, f16, None, scratch=self.scratch, decoded_bf16=dec)
            elif self.tp_rank == 0:
                torch.addmm(self.h, self.attn, layer.dense["o"].t(), out=self.h_next)  # the residual rides in the GEMM epilogue
            else:
                torch.mm(self.attn, layer.dense["o"].t(), out=self.h_next)
            if not self.tp_push:
                self._allreduce(self.h_next)
            if not fuse:
                nat.rmsnorm(self.h_next, layer.ln2, self.xn, s.eps)
            if fuse:
                nat.w3_gemv_fused_input(self.h_next, nat.W3_INPUT_RMSNORM, layer.ln2, s.eps, layer.gu_list, 2, 2 * self.inter, f16,
                                        scratch=self.scratch, decoded_bf16=dec)
            elif w3:
                nat.w3_gemv_multi(self.xn, layer.gu_list, 2, 2 * self.inter, f16, None, scratch=self.scratch, decoded_bf16=dec)
            else:
                torch.mm(self.xn, layer.dense["gate_up"].t(), out=self.gate_up)  # gate, up are views of this buffer
            if not fuse:
                nat.silu_mul(self.gate, self.up, self.act)
            if self.tp_push:
                site = self._sites[1]
                if fuse:
                    nat.w3_gemv_push(self.gate, nat.W3_INPUT_SILU_MUL, self.up, 0.0, layer.down_push, self.inter, f16, site["push"],
                                     scratch=self.scratch, decoded_bf16=dec)
                else:
                    nat.w3_gemv_push(self.act, 0, None, 0.0, layer.down_push, self.inter, f16, site["push"], scratch=self.scratch,
                                     decoded_bf16=dec)
                nat.tp_reduce(site["parts"], self.tp_size, self.h_next, self.h, site["status"])
            elif fuse:
                nat.w3_gemv_fused_input(self.gate, nat.W3_INPUT_SILU_MUL, self.up, 0.0, layer.down_list, 1, s.hidden, f16,
                                        scratch=self.scratch, decoded_bf16=dec)
            elif w3:
                nat.w3_gemv_multi(self.act, layer.down_list, 1, s.hidden, f16, None, scratch=self.scratch, decoded_bf16=dec)
            elif self.tp_rank == 0:
                torch.addmm(self.h_next, self.act, layer.dense["down"].t(), out=self.h)
            else:
                torch.mm(self.act, layer.dense["down"].t(), out=self.h)
            if not self.tp_push:
                self._allreduce(self.h)
            launches += (5 if fuse else 8) + (0 if self.fuse_attention else 1) + (2 if self.tp_size > 1 else 0)
        # final RMSNorm + LM head + argmax (+ the next token's embedding row, written over the hidden
        # state once every CTA has staged it) in one launch
        if self.tp_push and self.split_head:
            base, rows = self._head_rows
            nat.lm_head_shard(self.h, self.final_norm, s.eps, self.lm_head[base:base + rows], base, self._head_keys, self.tp_rank,
                              logits_shard=self.logits[:, base:base + rows] if self.keep_logits else None, scratch=self.head_scratch)
            nat.tp_argmax(self._head_keys_mine, self.tp_size, self.next_token if choice_out is None else choice_out, self._sites[0]["status"],
                          forced_next=next_forced if embed_next else None, embedding=self.embedding if embed_next else None,
                          next_hidden=self.h if embed_next else None)
            self._h_is_embedded = embed_next
            self.launches_per_step = launches + 2
            return
        nat.lm_head_argmax(self.h, self.final_norm, s.eps, self.lm_head, self.next_token if choice_out is None else choice_out, logits=self.logits if self.keep_logits else None,
                           forced_next=next_forced if embed_next else None, embedding=self.embedding if embed_next else None,
                           next_hidden=self.h if embed_next else None, scratch=self.head_scratch)
        self._h_is_embedded = embed_next
        self.launches_per_step = launches + 1

    def check_status(self) -> None:
        """After a synchronise: raise if a bounded device-side wait gave up (W3 GEMV staging: 1, tensor-core
        kernel: 3, tensor-parallel reduce: 4, tensor-parallel argmax: 6).  The scratch and exchange words are re-zeroed so that the
        engine is usable again; the outputs of the failed run are invalid."""
        codes = {}
        if self.arm == "w3":
            codes["w3 scratch"] = int(self.scratch[:4].view(torch.int32)[0])
        if self.tp_push:
            codes["tp exchange"] = int(self._xchg[:1].view(torch.int32)[0])
        bad = {k: v for k, v in codes.items() if v}
        if bad:
            if self.arm == "w3":
                self.scratch.zero_()
            if self.tp_push:
                self._xchg.zero_()
            self.head_scratch.zero_()
            raise RuntimeError(f"a device-side wait expired: {bad}; scratch re-zeroed, results of that run are invalid")

    def full_logits(self) -> torch.Tensor:
        """A copy of the last step's logits ``[1, vocab]``; with the vocabulary-split LM head every rank holds a
        shard, which an (eager, untimed) all-gather completes."""
        if not (self.tp_push and getattr(self, "split_head", False)):
            return self.logits.clone()
        base, rows = self._head_rows
        shards = [torch.empty(1, rows, device=self.device, dtype=self.dtype) for _ in range(self.tp_size)]
        torch.distributed.all_gather(shards, self.logits[:, base:base + rows].contiguous(), group=self.group)
        return torch.cat(shards, dim=-1)

    # ------------------------------------------------------------------ whole continuation
    @torch.inference_mode()
    def decode(self, first_token: torch.Tensor, start: int, steps: int, forced: torch.Tensor | None = None):
        """Eagerly decode ``steps`` tokens from ``start``; returns (tokens fed, greedy predictions, logits)."""
        fed, predicted, logits = [], [], []
        token = first_token.reshape(1).to(self.device)
        self._h_is_embedded = False
        for i in range(steps):
            if forced is not None:
                token = forced[i:i + 1].to(self.device)
            fed.append(token.clone())
            self.step(token, start + i)
            predicted.append(self.next_token.clone())
            logits.append(self.full_logits())
            token = self.next_token
        torch.cuda.synchronize(self.device)
        self.check_status()
        return torch.cat(fed), torch.cat(predicted), torch.cat(logits)

    @torch.inference_mode()
    def capture(self, first_token: torch.Tensor, start: int, steps: int, forced: torch.Tensor | None = None):
        """Capture the whole continuation in one CUDA graph (greedy feedback through a device
        buffer, or teacher-forced tokens).  Returns ``(graph, predictions [steps], last logits)``;
        replaying needs the KV cache prefix in place (later positions are simply overwritten).
        After a replay, synchronise and call ``check_status``."""
        self.token_in = first_token.reshape(1).to(self.device).clone()
        forced_dev = None if forced is None else forced.to(self.device).clone()
        predictions = torch.zeros(steps, dtype=torch.long, device=self.device)
        # the graph holds raw addresses of these tensors: keep them alive as long as the engine
        self._graph_inputs = getattr(self, "_graph_inputs", []) + [self.token_in, forced_dev, predictions]
        # the side stream must see the tensors above initialised: order it after the current stream now
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))

        def body():
            # one gather for the first token; every later step finds its embedding row written by the
            # LM-head launch of the step before (the forced token, or the greedy choice)
            self._h_is_embedded = False
            for i in range(steps):
                last = i + 1 == steps
                following = None if forced_dev is None or last else forced_dev[i + 1:i + 2]
                # the LM-head launch writes its choice straight into the prediction list: no copy node in the graph
                self.step(self.token_in if forced_dev is None else forced_dev[0:1], start + i, next_forced=following, embed_next=not last,
                          choice_out=predictions[i:i + 1])
            self._h_is_embedded = False

        with torch.cuda.stream(stream):
            self.step(self.token_in, start)  # warm-up: kernel attributes, scratch, cuBLAS handles
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                body()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        return graph, predictions, self.logits

    # ------------------------------------------------------------------ fp32 yardstick
    @torch.inference_mode()
    def truth_logits(self, input_ids: torch.Tensor, fed: torch.Tensor) -> torch.Tensor:
        """Logits of the decode steps with fp32 activations and fp32 dequantised weights: the prompt
        followed by the tokens fed at each step runs through ONE causal forward pass (cached decode equals
        the full-prefix forward, reference tests/test_full_model_trial.py:34-55).  Weights are dequantised
        layer by layer, scale * (code - zero) rounded once in the scale's dtype and widened; rotary
        angles stay fp32.  Returns ``[steps, vocab]`` fp32.  Unsharded engines only."""
        if self.tp_size != 1:
            raise ValueError("the fp32 yardstick runs on an unsharded engine")
        s = self.shape
        tokens = torch.cat((input_ids.reshape(-1).to(self.device), fed.reshape(-1).to(self.device)))
        t, steps = tokens.numel(), fed.numel()
        h = self.embedding[tokens].float()
        inv_freq = 1.0 / (s.rope_theta ** (torch.arange(0, s.head_dim, 2, device=self.device, dtype=torch.float32) / s.head_dim))
        angles = torch.arange(t, device=self.device, dtype=torch.float32)[:, None] * inv_freq[None, :]
        angles = torch.cat((angles, angles), dim=-1)
        cos, sin = angles.cos().unsqueeze(0), angles.sin().unsqueeze(0)
        rotate = lambda x: torch.cat((-x[..., s.head_dim // 2:], x[..., :s.head_dim // 2]), dim=-1)  # noqa: E731
        norm = lambda x, w: w.float() * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + s.eps))  # noqa: E731
        dq = lambda lay: restore_planar_w3(lay, dtype=torch.float32)  # noqa: E731
        previous = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            for layer in self.layers:
                x = norm(h, layer.ln1)
                q = F.linear(x, dq(layer.q)).reshape(t, s.q_heads, s.head_dim)
                k = F.linear(x, dq(layer.k)).reshape(t, s.kv_heads, s.head_dim)
                v = F.linear(x, dq(layer.v)).reshape(t, s.kv_heads, s.head_dim).transpose(0, 1)
                q = norm(q, layer.q_norm).transpose(0, 1)
                k = norm(k, layer.k_norm).transpose(0, 1)
                q = q * cos + rotate(q) * sin
                k = k * cos + rotate(k) * sin
                attn = F.scaled_dot_product_attention(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), is_causal=True, enable_gqa=True)
                h = h + F.linear(attn[0].transpose(0, 1).reshape(t, -1), dq(layer.o))
                x = norm(h, layer.ln2)
                act = F.silu(F.linear(x, dq(layer.gate))) * F.linear(x, dq(layer.up))
                h = h + F.linear(act, dq(layer.down))
            last = norm(h[t - steps:], self.final_norm)
            return F.linear(last, self.lm_head.float())
        finally:
            torch.backends.cuda.matmul.allow_tf32 = previous
