"""Several mixers side by side on the same input:

    out = mean_k  w_k * y_k / sqrt(mean(y_k^2) + eps),   y_k = mixer_k(h)

Each output is RMS-normed over the model width with a plain weight of its own before the mean.  Every mixer
keeps what it keeps (pages, a state in the slot) under a cache entry of its own: the run step names the
first one's entry in ``cache`` and the others' in ``more_caches``.
"""
from __future__ import annotations

import dataclasses
from typing import List

import torch

from ..config.spec import RunStep, SideBySideSpec
from ..errors import ConfigError, Unsupported
from ..kernels import ops
from ..weights.loader import VECTOR, TensorDecl
from .base import MIXERS, Part, lookup, register_mixer


@register_mixer("side_by_side")
class SideBySide(Part):
    def __init__(self, spec: SideBySideSpec, prefix: str, tensors: dict, mctx):
        if len(spec.mixers) != 2 or len(spec.out_norm_names) != 2 or spec.mixers[0].kind == spec.mixers[1].kind:
            raise Unsupported("mixers side by side come in pairs of two kinds (each kind has one set of buffers)")
        self.spec = spec
        self.mixers = [lookup(MIXERS, m.kind, "mixer")(m, prefix, tensors, mctx) for m in spec.mixers]
        self.out_weights = [tensors[prefix + n] for n in spec.out_norm_names]
        self.replayable = all(getattr(m, "replayable", True) for m in self.mixers)
        self._steps = {}

    @classmethod
    def tensor_decls(cls, s: SideBySideSpec, prefix: str) -> List[TensorDecl]:
        decls = []
        for m in s.mixers:
            decls += lookup(MIXERS, m.kind, "mixer").tensor_decls(m, prefix)
        return decls + [TensorDecl(prefix + n, (s.hidden_size,), VECTOR) for n in s.out_norm_names]

    @classmethod
    def cache_need_of(cls, s: SideBySideSpec):
        """One need per mixer, in their order (a tuple: the run step carries one cache entry for each)."""
        return tuple(lookup(MIXERS, m.kind, "mixer").cache_need_of(m) for m in s.mixers)

    def _step_of(self, run_step: RunStep, k: int) -> RunStep:
        got = self._steps.get((run_step, k))
        if got is None:
            entries = (run_step.cache,) + tuple(run_step.more_caches)
            if len(entries) != len(self.mixers):
                raise ConfigError(f"a run step of {len(self.mixers)} mixers side by side names {len(entries)} cache entries")
            got = self._steps[(run_step, k)] = dataclasses.replace(run_step, cache=entries[k], more_caches=())
        return got

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep) -> torch.Tensor:
        # the mixers' results in float32: they are normed before anything rounds them
        ys = [m.forward(ctx, x, self._step_of(run_step, k), out_dtype=torch.float32) for k, m in enumerate(self.mixers)]
        out = ctx.workspace.get("side.out", x.shape[0], self.spec.hidden_size, ctx.dtype)
        ops.paired_rmsnorm_mean(ys[0], self.out_weights[0], ys[1], self.out_weights[1], self.spec.out_norm_eps, out)
        return out
