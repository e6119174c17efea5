"""A matrix memory with exponential gates: a recurrent mixer with a state S [head_dim, v_head_dim] and a vector n
[head_dim] per head, and a running maximum m of the gates' logarithms (all three start at zero).

    q = W_q h / sqrt(head_dim);  k = W_k h;  v = W_v h
    i = cap tanh((W_i h + b_i) / cap);   f = log logistic(cap tanh((W_f h + b_f) / cap))         per head
    m' = max(f + m, i);   S <- exp(f + m - m') S + exp(i - m') k v^T;   n <- exp(f + m - m') n + exp(i - m') k
    o = S^T q / (max(|n . q|, exp(-m')) + floor)
    out = W_o (U(o) * w * logistic(W_g h))        U: each head over its root mean square

One stacked projection gives q | k | v | output gate | i | f in float32; gates, decays, state and the read-out are
float32.  The state (S, n, m of every head) is a fixed-size float32 row of the request's slot: zero for a new request,
carried from token to token, put back when a step fails.
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import FIXED_STATE
from ..config.spec import MatrixMemorySpec, RunStep
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import CacheNeed, Part, register_mixer
from .linear import Linear


@register_mixer("matrix_memory")
class MatrixMemory(Part):
    def __init__(self, spec: MatrixMemorySpec, prefix: str, tensors: dict, mctx):
        self.spec = s = spec
        p, nm = prefix, spec.names
        stacked = [tensors[p + n] for n in (nm.q, nm.k, nm.v, nm.gate, nm.write, nm.forget)]
        self.proj = Linear(torch.cat(stacked, dim=0).contiguous(), p + "q_k_v_g_i_f")
        self.bias_i, self.bias_f = tensors[p + nm.write + ".b"], tensors[p + nm.forget + ".b"]
        self.out_norm_w = tensors[p + nm.out_norm]
        self.gate_off = 2 * s.heads * s.head_dim + s.heads * s.v_head_dim
        self.out = Linear(tensors[p + nm.o], p + nm.o)

    @classmethod
    def tensor_decls(cls, s: MatrixMemorySpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.names
        qk, v = s.heads * s.head_dim, s.heads * s.v_head_dim
        return [TensorDecl(p + nm.q, (qk, s.hidden_size), MATRIX), TensorDecl(p + nm.k, (qk, s.hidden_size), MATRIX),
                TensorDecl(p + nm.v, (v, s.hidden_size), MATRIX), TensorDecl(p + nm.gate, (v, s.hidden_size), MATRIX),
                TensorDecl(p + nm.write, (s.heads, s.hidden_size), MATRIX), TensorDecl(p + nm.write + ".b", (s.heads,), VECTOR),
                TensorDecl(p + nm.forget, (s.heads, s.hidden_size), MATRIX), TensorDecl(p + nm.forget + ".b", (s.heads,), VECTOR),
                TensorDecl(p + nm.out_norm, (v,), VECTOR), TensorDecl(p + nm.o, (s.hidden_size, v), MATRIX)]

    @staticmethod
    def state_size(s: MatrixMemorySpec) -> int:
        return s.heads * s.head_dim * s.v_head_dim + s.heads * s.head_dim + s.heads

    @classmethod
    def cache_need_of(cls, s: MatrixMemorySpec) -> CacheNeed:
        return CacheNeed(FIXED_STATE, state_shape=(cls.state_size(s),), state_dtype=torch.float32)

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep, out_dtype=None) -> torch.Tensor:
        """-> [T, hidden] in ``out_dtype`` (default: the activation dtype)."""
        s = self.spec
        T, H, d, dv = x.shape[0], s.heads, s.head_dim, s.v_head_dim
        proj = self.proj(ctx, x, "memory.proj", out_dtype=torch.float32)
        state = ctx.cache.state_of_entry(run_step.cache)                    # [slots, state_size]
        o = ctx.workspace.get("memory.o", T, H * dv, torch.float32)
        ops.matrix_memory_recurrence(ctx, proj, self.bias_i, self.bias_f, s.gate_cap, s.denominator_floor, state, o, H, d, dv)
        gated = ctx.workspace.get("memory.out", T, H * dv, ctx.dtype)
        ops.matrix_memory_output(o, self.out_norm_w, s.norm_eps, proj, self.gate_off, gated, H, dv)
        return self.out(ctx, gated, "memory.proj_out", out_dtype=out_dtype)
