"""The selective scan: a recurrent mixer with a state S [inner, state] per request.

    [x | z] = W_in h;   x <- silu(conv(x) + b_conv)          a short causal convolution per channel over time
    [dt | B | C] = W_x x;   dt <- softplus(W_dt dt + b_dt)    one step size per channel
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c,   A = -exp(A_log)
    out = W_o (y * silu(z))

The three projections ahead of the recurrence write float32, so step sizes, decays, B, C and x enter it
unrounded; the recurrence itself is float32.  What a request carries from token to token is a fixed-size
float32 state in the request's slot: S of every channel and the last taps - 1 inputs of every channel's
convolution.  It starts at zero (the engine zeroes a slot for its new occupant) and is put back when a step
fails (the engine's snapshot).
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import FIXED_STATE
from ..config.spec import RunStep, SelectiveScanSpec
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import CacheNeed, Part, register_mixer
from .linear import Linear


@register_mixer("selective_scan")
class SelectiveScan(Part):
    def __init__(self, spec: SelectiveScanSpec, prefix: str, tensors: dict, mctx):
        self.spec = spec
        p, nm = prefix, spec.names
        self.inp = Linear(tensors[p + nm.inp], p + nm.inp)
        self.conv_w, self.conv_b = tensors[p + nm.conv], tensors[p + nm.conv + ".b"]
        self.x_proj = Linear(tensors[p + nm.x], p + nm.x)
        self.dt_proj = Linear(tensors[p + nm.dt], p + nm.dt)
        self.dt_bias = tensors[p + nm.dt + ".b"]
        self.A = (-torch.exp(tensors[p + nm.a_log].float())).contiguous()
        self.D = tensors[p + nm.d]
        self.out = Linear(tensors[p + nm.o], p + nm.o)

    @classmethod
    def tensor_decls(cls, s: SelectiveScanSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.names
        return [TensorDecl(p + nm.inp, (2 * s.inner, s.hidden_size), MATRIX),
                TensorDecl(p + nm.conv, (s.inner, s.conv_taps), VECTOR),
                TensorDecl(p + nm.conv + ".b", (s.inner,), VECTOR),
                TensorDecl(p + nm.x, (s.dt_rank + 2 * s.state, s.inner), MATRIX),
                TensorDecl(p + nm.dt, (s.inner, s.dt_rank), MATRIX),
                TensorDecl(p + nm.dt + ".b", (s.inner,), VECTOR),
                TensorDecl(p + nm.a_log, (s.inner, s.state), VECTOR),
                TensorDecl(p + nm.d, (s.inner,), VECTOR),
                TensorDecl(p + nm.o, (s.hidden_size, s.inner), MATRIX)]

    @staticmethod
    def state_size(s: SelectiveScanSpec) -> int:
        return s.inner * (s.state + s.conv_taps - 1)

    @classmethod
    def cache_need_of(cls, s: SelectiveScanSpec) -> CacheNeed:
        return CacheNeed(FIXED_STATE, state_shape=(cls.state_size(s),), state_dtype=torch.float32)

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep, out_dtype=None) -> torch.Tensor:
        """-> [T, hidden] in ``out_dtype`` (default: the activation dtype)."""
        s = self.spec
        T, C, N, R = x.shape[0], s.inner, s.state, s.dt_rank
        ws = ctx.workspace
        state = ctx.cache.state_of_entry(run_step.cache)                    # [slots, state_size]
        xz = self.inp(ctx, x, "scan.xz", out_dtype=torch.float32)
        xc = ws.get("scan.x", T, C, torch.float32)
        low = ctx.dtype != torch.float32          # the B / C / dt product takes its input in the activation dtype
        xl = ws.get("scan.x_low", T, C, ctx.dtype) if low else None
        ops.scan_conv(ctx, xz, self.conv_w, self.conv_b, state, xc, xl, C, N, s.conv_taps)
        dbc = self.x_proj(ctx, xl if low else xc, "scan.dbc", out_dtype=torch.float32)
        dl = ws.get("scan.dt_in", T, R, ctx.dtype)          # the step sizes' low-rank part, contiguous, for its product
        ops.cast_columns(dbc, 0, dl)
        dt_raw = self.dt_proj(ctx, dl, "scan.dt_raw", out_dtype=torch.float32)
        y = ws.get("scan.y", T, C, ctx.dtype)
        ops.selective_scan(ctx, xc, xz, dbc, R, dt_raw, self.dt_bias, self.A, self.D, state, y, C, N, s.conv_taps)
        return self.out(ctx, y, "scan.o", out_dtype=out_dtype)
