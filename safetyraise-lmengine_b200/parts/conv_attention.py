"""Grouped-query attention whose q, k and v each pass a short causal convolution over time:

    q, k, v = conv(W h)                     per channel, no bias, zeros before a request's first token
    q, k <- N(w_q, q), N(w_k, k)            RMS norm per head, one weight of head_dim for all heads
    q, k <- rotated                         the encoding says which elements pair up and by what angles
    p_ij = exp(s_ij) / (sink + sum_j' exp(s_ij')),  s_ij = (q_i . k_j) * scale,  0 <= i - j < window
    out = W_o sum_j p_ij v_j

with sink = 1 when ``unit_sink`` is set: one more key whose score is 0 and which has no value.  In the kernels that is
the initial state of a row's running softmax (maximum 0, sum 1, output 0), so it costs nothing.

One stacked projection gives q | k | v in float32; one kernel convolves, norms, rotates, writes q and appends k and v
to the pages.  The mixer keeps two things per request: pages of keys and values, and the last taps - 1 projected rows
(a fixed-size float32 state in the request's slot), so its run step names two cache entries.
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import FIXED_STATE, PAGED_ALL, PAGED_WINDOW
from ..config.spec import ConvAttentionSpec, RunStep
from ..errors import ConfigError, Unsupported
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import POSITION_ENCODINGS, ROTATION, CacheNeed, Part, lookup, register_mixer
from .linear import Linear


@register_mixer("conv_attention")
class ConvAttention(Part):
    def __init__(self, spec: ConvAttentionSpec, prefix: str, tensors: dict, mctx):
        self.spec = s = spec
        p, nm = prefix, spec.names
        parts = (nm.q, nm.k, nm.v)
        self.proj = Linear(torch.cat([tensors[p + n] for n in parts], dim=0).contiguous(), p + "q_k_v")
        self.channels = s.heads * s.head_dim + s.kv_heads * (s.head_dim + s.v_head_dim)
        self.conv_w = torch.cat([tensors[p + n + nm.conv_suffix] for n in parts], dim=0).float().contiguous()
        self.q_norm_w = self.k_norm_w = None
        if s.qk_norm_eps is not None:
            self.q_norm_w, self.k_norm_w = tensors[p + nm.q + nm.norm_suffix], tensors[p + nm.k + nm.norm_suffix]
        self.sink = torch.zeros(s.heads, dtype=torch.float32, device=mctx.device) if s.unit_sink else None
        self.out = Linear(tensors[p + nm.o], p + nm.o)
        self.position = None
        if s.position is not None:
            self.position = lookup(POSITION_ENCODINGS, s.position.kind, "position encoding")(s.position, mctx)
            if getattr(self.position, "applies", ROTATION) != ROTATION:
                raise Unsupported(f"position encoding {s.position.kind!r} is not a rotation")
        self._no_state = None

    @classmethod
    def tensor_decls(cls, s: ConvAttentionSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.names
        sizes = {nm.q: s.heads * s.head_dim, nm.k: s.kv_heads * s.head_dim, nm.v: s.kv_heads * s.v_head_dim}
        decls = [TensorDecl(p + n, (rows, s.hidden_size), MATRIX) for n, rows in sizes.items()]
        if s.qk_norm_eps is not None:
            decls += [TensorDecl(p + n + nm.norm_suffix, (s.head_dim,), VECTOR) for n in (nm.q, nm.k)]
        decls += [TensorDecl(p + n + nm.conv_suffix, (rows, s.conv_taps), VECTOR) for n, rows in sizes.items()]
        decls.append(TensorDecl(p + nm.o, (s.hidden_size, s.heads * s.v_head_dim), MATRIX))
        return decls

    @classmethod
    def cache_need_of(cls, s: ConvAttentionSpec):
        """The pages and, with a convolution of more than one tap, the carried rows: a tuple of two needs."""
        pages = CacheNeed(PAGED_WINDOW if s.window else PAGED_ALL, s.kv_heads, s.head_dim, s.window,
                          v_head_dim=None if s.v_head_dim == s.head_dim else s.v_head_dim)
        if s.conv_taps <= 1:
            return pages
        channels = s.heads * s.head_dim + s.kv_heads * (s.head_dim + s.v_head_dim)
        return (pages, CacheNeed(FIXED_STATE, state_shape=((s.conv_taps - 1) * channels,), state_dtype=torch.float32))

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep, out_dtype=None) -> torch.Tensor:
        """-> [T, hidden] in ``out_dtype`` (default: the activation dtype)."""
        s = self.spec
        T = x.shape[0]
        if len(run_step.more_caches) != (1 if s.conv_taps > 1 else 0):
            raise ConfigError("a run step of an attention behind convolutions names its pages' entry and its carried rows'")
        proj = self.proj(ctx, x, "conv_attn.proj", out_dtype=torch.float32)
        k_pool, v_pool, group = ctx.cache.kv_of_entry(run_step.cache)
        if s.conv_taps > 1:
            state = ctx.cache.state_of_entry(run_step.more_caches[0])
        else:
            if self._no_state is None:
                self._no_state = torch.zeros((1, 1), dtype=torch.float32, device=proj.device)
            state = self._no_state
        page_size = k_pool.shape[2]
        rot = self.position.rotation(ctx) if self.position is not None else None
        # prompts with heads of 128 for keys and values: the tensor-memory kernel, which takes its queries in bfloat16
        # and starts every row's softmax from the head's sink
        on_tcgen05 = (v_pool is not None and not s.window and ctx.max_q_len > 4 and s.unit_sink
                      and ops.sinks_on_tcgen05(ctx, ctx.dtype, s.heads, s.kv_heads, s.head_dim, s.v_head_dim, page_size))
        q = ctx.workspace.get("conv_attn.q", T, s.heads * s.head_dim, ctx.dtype if on_tcgen05 else torch.float32)
        ops.conv_norm_rope_append(ctx, proj, self.conv_w, state, 0, self.q_norm_w, self.k_norm_w, s.qk_norm_eps, rot, q,
                                  k_pool, v_pool, ctx.kv_slot[group], s.heads, s.kv_heads, s.head_dim, s.v_head_dim)
        ops.conv_carry(ctx, proj, 0, self.channels, s.conv_taps, state, 0)
        attended = ctx.workspace.get("conv_attn.out", T, s.heads * s.v_head_dim, ctx.dtype)
        if on_tcgen05:
            ops.paged_attention(ctx, q, k_pool, v_pool, attended, ctx.block_tables[group], s.heads, s.kv_heads,
                                s.head_dim, page_size, s.softmax_scale, 0, sinks=self.sink)
        else:
            ops.paged_attention_general(ctx, q, k_pool, v_pool, attended, ctx.block_tables[group], self.sink, s.heads,
                                        s.kv_heads, s.head_dim, s.v_head_dim, s.softmax_scale, s.window or 0)
        return self.out(ctx, attended, "conv_attn.o", out_dtype=out_dtype)
