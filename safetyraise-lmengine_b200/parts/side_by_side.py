"""Several mixers side by side on the same input:

    out = mean_k  w_k * y_k / sqrt(mean(y_k^2) + eps),   y_k = mixer_k(h)

Each output is RMS-normed over the model width with a plain weight of its own before the mean.  With ``combine``
"weighted_sum" nothing is normed: out = sum_k weights[k] * y_k.  Every mixer keeps what it keeps (pages, a state in
the slot) under cache entries of its own: the run step names them one after the other, the first in ``cache`` and
the rest in ``more_caches`` (a mixer that keeps two things takes two).
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
        if len(spec.mixers) != 2 or spec.mixers[0].kind == spec.mixers[1].kind:
            raise Unsupported("mixers side by side come in pairs of two kinds (each kind has one set of buffers)")
        if spec.combine not in ("normed_mean", "weighted_sum"):
            raise Unsupported(f"mixers side by side combined by {spec.combine!r} are not implemented")
        if len(spec.out_norm_names if spec.combine == "normed_mean" else spec.weights) != 2:
            raise ConfigError("mixers side by side: one output norm, or one weight, for each")
        self.spec = spec
        self.mixers = [lookup(MIXERS, m.kind, "mixer")(m, prefix, tensors, mctx) for m in spec.mixers]
        self.out_weights = [tensors[prefix + n] for n in spec.out_norm_names] if spec.combine == "normed_mean" else None
        # how many cache entries each mixer's run step names
        self.entries_of = [len(n) if isinstance(n, tuple) else 1
                           for n in (lookup(MIXERS, m.kind, "mixer").cache_need_of(m) for m in spec.mixers)]
        self.replayable = all(getattr(m, "replayable", True) for m in self.mixers)
        self._steps = {}

    @classmethod
    def tensor_decls(cls, s: SideBySideSpec, prefix: str) -> List[TensorDecl]:
        decls = []
        for m in s.mixers:
            decls += lookup(MIXERS, m.kind, "mixer").tensor_decls(m, prefix)
        if s.combine != "normed_mean":
            return decls
        return decls + [TensorDecl(prefix + n, (s.hidden_size,), VECTOR) for n in s.out_norm_names]

    @classmethod
    def cache_need_of(cls, s: SideBySideSpec):
        """The mixers' needs, in their order (a tuple: the run step carries one cache entry for each need)."""
        needs = []
        for m in s.mixers:
            need = lookup(MIXERS, m.kind, "mixer").cache_need_of(m)
            needs += list(need) if isinstance(need, tuple) else [need]
        return tuple(needs)

    def _step_of(self, run_step: RunStep, k: int) -> RunStep:
        got = self._steps.get((run_step, k))
        if got is None:
            entries = (run_step.cache,) + tuple(run_step.more_caches)
            if len(entries) != sum(self.entries_of):
                raise ConfigError(f"a run step of mixers side by side with {sum(self.entries_of)} needs names "
                                  f"{len(entries)} cache entries")
            at = sum(self.entries_of[:k])
            got = self._steps[(run_step, k)] = dataclasses.replace(run_step, cache=entries[at],
                                                                   more_caches=entries[at + 1:at + self.entries_of[k]])
        return got

    @property
    def offers_terms(self) -> bool:
        """Whether forward(..., as_terms=True) hands back the mixers' results with their weights instead of their sum
        (for a block whose own kernel adds them to the stream)."""
        return self.spec.combine == "weighted_sum"

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep, as_terms: bool = False):
        # the mixers' results in float32: they are normed, or summed, before anything rounds them
        ys = [m.forward(ctx, x, self._step_of(run_step, k), out_dtype=torch.float32) for k, m in enumerate(self.mixers)]
        out = ctx.workspace.get("side.out", x.shape[0], self.spec.hidden_size, ctx.dtype)
        if self.spec.combine == "weighted_sum" and as_terms:
            return tuple(zip(ys, self.spec.weights))
        if self.spec.combine == "weighted_sum":
            ops.weighted_sum(ys[0], self.spec.weights[0], ys[1], self.spec.weights[1], out)
            return out
        ops.paired_rmsnorm_mean(ys[0], self.out_weights[0], ys[1], self.out_weights[1], self.spec.out_norm_eps, out)
        return out
