"""A gated linear recurrence per channel, beside a gate branch:

    y = gelu_tanh(W_y h + b_y)
    u = conv(W_x h + b_x) + b_conv                   a short causal convolution per channel, zeros before the start
    r = logistic(R_a u + b_a);  i = logistic(R_i u + b_i)            R block-diagonal: ``blocks`` square blocks
    a = exp(-decay_scale r softplus(lam));   S <- a S + sqrt(1 - a^2) i u        from S = 0, the first token included
    out = W_o (S * y)

One stacked projection gives the two branches in float32; convolution, gates, decay and state are float32.  What a
request carries is a fixed-size float32 row of its slot: S [width], then the convolution's last taps - 1 inputs.
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import FIXED_STATE
from ..config.spec import GatedRecurrenceSpec, RunStep
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import CacheNeed, Part, register_mixer
from .linear import Linear


@register_mixer("gated_linear_recurrence")
class GatedLinearRecurrence(Part):
    def __init__(self, spec: GatedRecurrenceSpec, prefix: str, tensors: dict, mctx):
        self.spec = s = spec
        p, nm = prefix, spec.names
        self.proj = Linear(torch.cat([tensors[p + nm.gate_branch], tensors[p + nm.recurrent_branch]], dim=0).contiguous(),
                           p + "y_x")
        self.y_bias, self.x_bias = tensors[p + nm.gate_branch + ".b"], tensors[p + nm.recurrent_branch + ".b"]
        self.conv_w, self.conv_b = tensors[p + nm.conv], tensors[p + nm.conv + ".b"]
        self.Ra, self.Ri = tensors[p + nm.decay_gate], tensors[p + nm.input_gate]
        self.ba = tensors[p + nm.decay_gate + ".b"].reshape(-1).contiguous()
        self.bi = tensors[p + nm.input_gate + ".b"].reshape(-1).contiguous()
        # the decay's rate per channel, once: decay_scale * softplus(lam), float32
        self.rate = (s.decay_scale * torch.nn.functional.softplus(tensors[p + nm.decay].double())).float().contiguous()
        self.out = Linear(tensors[p + nm.o], p + nm.o)

    @classmethod
    def tensor_decls(cls, s: GatedRecurrenceSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.names
        C, B = s.width, s.blocks
        return [TensorDecl(p + nm.gate_branch, (C, s.hidden_size), MATRIX), TensorDecl(p + nm.gate_branch + ".b", (C,), VECTOR),
                TensorDecl(p + nm.recurrent_branch, (C, s.hidden_size), MATRIX),
                TensorDecl(p + nm.recurrent_branch + ".b", (C,), VECTOR),
                TensorDecl(p + nm.conv, (C, s.conv_taps), VECTOR), TensorDecl(p + nm.conv + ".b", (C,), VECTOR),
                TensorDecl(p + nm.decay_gate, (B, C // B, C // B), MATRIX), TensorDecl(p + nm.decay_gate + ".b", (B, C // B), VECTOR),
                TensorDecl(p + nm.input_gate, (B, C // B, C // B), MATRIX), TensorDecl(p + nm.input_gate + ".b", (B, C // B), VECTOR),
                TensorDecl(p + nm.decay, (C,), VECTOR), TensorDecl(p + nm.o, (s.hidden_size, C), MATRIX)]

    @staticmethod
    def state_size(s: GatedRecurrenceSpec) -> int:
        return s.width * s.conv_taps            # S, then taps - 1 carried inputs per channel

    @classmethod
    def cache_need_of(cls, s: GatedRecurrenceSpec) -> CacheNeed:
        return CacheNeed(FIXED_STATE, state_shape=(cls.state_size(s),), state_dtype=torch.float32)

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep, out_dtype=None) -> torch.Tensor:
        """-> [T, hidden] in ``out_dtype`` (default: the activation dtype)."""
        s = self.spec
        T, C = x.shape[0], s.width
        ws = ctx.workspace
        proj = self.proj(ctx, x, "recurrence.proj", out_dtype=torch.float32)       # y columns, then x columns
        state = ctx.cache.state_of_entry(run_step.cache)                            # [slots, state_size]
        u = ws.get("recurrence.u", T, C, torch.float32)
        ops.short_conv(ctx, proj, C, C, self.conv_w, state, C, u, in_bias=self.x_bias, out_bias=self.conv_b)
        ops.conv_carry(ctx, proj, C, C, s.conv_taps, state, C, in_bias=self.x_bias)
        a = ws.get("recurrence.a", T, C, torch.float32)
        b = ws.get("recurrence.b", T, C, torch.float32)
        ops.recurrence_gates(u, self.Ra, self.Ri, self.ba, self.bi, self.rate, a, b, s.blocks)
        gated = ws.get("recurrence.out", T, C, ctx.dtype)
        # long portions in segments side by side; the float32 path walks token by token (its sums keep one order)
        ops.linear_recurrence(ctx, a, b, proj, 0, self.y_bias, state, gated,
                              in_segments=ctx.dtype != torch.float32 and ctx.max_q_len >= 256)
        return self.out(ctx, gated, "recurrence.proj_out", out_dtype=out_dtype)
