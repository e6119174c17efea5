"""Grouped-query attention with a rotary encoding on the leading part of q and k, optional biases, an optional
cap on the scores, an optional window, and keys and values of different sizes:

    q, k, v = W h (+ b);   q, k <- rotated (the encoding says which elements pair up and by what angles)
    score(i, j) = cap((q_i . k_j) * scale),  cap(s) = softcap * tanh(s / softcap),   0 <= i - j < window
    out = W_o softmax(score) v

One stacked projection gives q | k | v in float32, so biases, rotation and scores see unrounded values; keys
and values go to the pages in the cache's dtype.  A mixer without keys and values of its own (``own_kv``
False) projects q alone and attends over the pages of the run step whose cache entry it reads: that step's
keys as cached (rotated) and its values.
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import PAGED_ALL, PAGED_WINDOW
from ..config.spec import RotatedAttentionSpec, RunStep
from ..errors import ConfigError, Unsupported
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import POSITION_ENCODINGS, ROTATION, CacheNeed, Part, lookup, register_mixer
from .linear import Linear


@register_mixer("rotated_attention")
class RotatedAttention(Part):
    def __init__(self, spec: RotatedAttentionSpec, prefix: str, tensors: dict, mctx):
        self.spec = s = spec
        p, nm = prefix, spec.names
        parts = (nm.q, nm.k, nm.v) if s.own_kv else (nm.q,)
        self.proj = Linear(torch.cat([tensors[p + n] for n in parts], dim=0).contiguous(), p + "q_k_v")
        self.bias = torch.cat([tensors[p + n + nm.bias_suffix] for n in parts]).contiguous() if s.bias else None
        self.out = Linear(tensors[p + nm.o], p + nm.o)
        self.position = None
        if s.position is not None:
            self.position = lookup(POSITION_ENCODINGS, s.position.kind, "position encoding")(s.position, mctx)
            if getattr(self.position, "applies", ROTATION) != ROTATION:
                raise Unsupported(f"position encoding {s.position.kind!r} acts on {self.position.applies!r}; "
                                  f"this attention applies rotations of q and k only")

    @classmethod
    def tensor_decls(cls, s: RotatedAttentionSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.names
        sizes = {nm.q: s.heads * s.head_dim}
        if s.own_kv:
            sizes.update({nm.k: s.kv_heads * s.head_dim, nm.v: s.kv_heads * s.v_head_dim})
        decls = [TensorDecl(p + n, (rows, s.hidden_size), MATRIX) for n, rows in sizes.items()]
        if s.bias:
            decls += [TensorDecl(p + n + nm.bias_suffix, (rows,), VECTOR) for n, rows in sizes.items()]
        decls.append(TensorDecl(p + nm.o, (s.hidden_size, s.heads * s.v_head_dim), MATRIX))
        return decls

    @classmethod
    def cache_need_of(cls, s: RotatedAttentionSpec) -> CacheNeed:
        if s.window and s.cache_window and s.cache_window < s.window:
            raise ConfigError("a rotated attention's cache keeps fewer keys than its window sees")
        keeps = s.cache_window if s.window else None
        return CacheNeed(PAGED_WINDOW if keeps else PAGED_ALL, s.kv_heads, s.head_dim, keeps,
                         v_head_dim=None if s.v_head_dim == s.head_dim else s.v_head_dim)

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep, out_dtype=None) -> torch.Tensor:
        """-> [T, hidden] in ``out_dtype`` (default: the activation dtype)."""
        s = self.spec
        if run_step.writes_cache != s.own_kv:
            raise ConfigError("a rotated attention writes its cache entry exactly when it has keys and values of its own")
        T = x.shape[0]
        proj = self.proj(ctx, x, "rot_attn.proj", out_dtype=torch.float32)
        k_pool, v_pool, group = ctx.cache.kv_of_entry(run_step.cache)
        page_size = k_pool.shape[2]
        rot = self.position.rotation(ctx) if self.position is not None else None
        same = s.head_dim == s.v_head_dim
        # bfloat16 with keys and values of one size: the framework's attention of equal head sizes (decode steps on
        # its TMA kernels, prompts on tensor memory or mma.sync); with a cap only where the tensor-memory kernel serves
        plain = (ctx.dtype == torch.bfloat16 and same and not s.softcap and s.head_dim % 16 == 0 and s.head_dim <= 256)
        capped_rows = (same and bool(s.softcap) and ctx.max_q_len > 4
                       and ops.sinks_on_tcgen05(ctx, ctx.dtype, s.heads, s.kv_heads, s.head_dim, s.v_head_dim, page_size))
        low_q = plain or capped_rows
        q = ctx.workspace.get("rot_attn.q", T, s.heads * s.head_dim, ctx.dtype if low_q else torch.float32)
        ops.attention_bias_append(proj, self.bias, q, k_pool, v_pool, ctx.kv_slot[group], s.heads, s.kv_heads,
                                  s.head_dim, s.v_head_dim, write_kv=s.own_kv, rotation=rot)
        attended = ctx.workspace.get("rot_attn.out", T, s.heads * s.v_head_dim, ctx.dtype)
        if low_q:
            ops.paged_attention(ctx, q, k_pool, v_pool, attended, ctx.block_tables[group], s.heads, s.kv_heads,
                                s.head_dim, page_size, s.softmax_scale, s.window or 0,
                                mods=(None, None, None, s.softcap) if capped_rows else None)
        else:
            ops.paged_attention_general(ctx, q, k_pool, v_pool, attended, ctx.block_tables[group], None, s.heads,
                                        s.kv_heads, s.head_dim, s.v_head_dim, s.softmax_scale, s.window or 0,
                                        softcap=s.softcap)
        return self.out(ctx, attended, "rot_attn.o", out_dtype=out_dtype)
