"""The arrangements of norms, mixer and feed-forward around the residual stream.

``pre_norm``: r = x + mixer(norm(x)); x' = r + ff(norm(r))  (src/model/native.rs:526-562).
``sandwich_gated``: a norm before and after each sublayer and a learned gate on its result (see the class).
``parallel``: h = norm(x); x' = x + mixer(h) + ff(h): one norm, both sublayers read it.
``post_norm``: x' = norm(a x + mixer(x)), then x'' = norm(a x' + ff(x')): the norm comes after the sum.

The residual stream is a float32 tensor updated in place.  A block does not add
its feed-forward output itself: it returns it as *pending*, and the next norm
(the next block's, or the final one) adds it in the same kernel that norms.
"""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import LayerSpec, RunStep
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import FEED_FORWARDS, MIXERS, NORMS, Block, NormedInput, lookup, register_block
from .linear import Linear


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, spec: LayerSpec, tensors: dict, mctx):
        p = spec.weight_prefix
        self.spec = spec
        self.mixer_norm = lookup(NORMS, spec.mixer_norm.kind, "norm")(spec.mixer_norm, p + spec.mixer_norm_name,
                                                                      tensors, mctx)
        self.mixer = lookup(MIXERS, spec.mixer.kind, "mixer")(spec.mixer, p, tensors, mctx)
        self.ff_norm = self.feed_forward = None          # a layer of a mixer alone: x + mixer(norm(x))
        if spec.feed_forward is not None:
            self.ff_norm = lookup(NORMS, spec.feed_forward_norm.kind, "norm")(
                spec.feed_forward_norm, p + spec.feed_forward_norm_name, tensors, mctx)
            self.feed_forward = lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward")(
                spec.feed_forward, p, tensors, mctx)
        self.hidden = spec.mixer_norm.size
        self.replayable = all(getattr(part, "replayable", True)
                              for part in (self.mixer_norm, self.ff_norm, self.mixer, self.feed_forward))

    @classmethod
    def tensor_decls(cls, spec: LayerSpec, prefix: str = "") -> List[TensorDecl]:
        p = spec.weight_prefix
        decls = (lookup(NORMS, spec.mixer_norm.kind, "norm").tensor_decls(spec.mixer_norm, p + spec.mixer_norm_name)
                 + lookup(MIXERS, spec.mixer.kind, "mixer").tensor_decls(spec.mixer, p))
        if spec.feed_forward is not None:
            decls += (lookup(NORMS, spec.feed_forward_norm.kind, "norm").tensor_decls(spec.feed_forward_norm,
                                                                                      p + spec.feed_forward_norm_name)
                      + lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward").tensor_decls(
                          spec.feed_forward, p))
        return decls

    def fuses(self, ctx) -> bool:
        """Whether this block runs its norms inside the products around them for this step: both parts
        offer forward_fused and the step is small enough for the kernels that carry the fusions."""
        return (self.feed_forward is not None
                and getattr(self.mixer_norm, "fusable", False) and getattr(self.ff_norm, "fusable", False)
                and hasattr(self.mixer, "forward_fused") and hasattr(self.feed_forward, "forward_fused")
                and self.mixer.can_fuse(ctx) and self.feed_forward.can_fuse(ctx)
                and not ctx.options.get("unfused_norms", False))

    def prepared_input_norm(self, ctx):
        """This block takes its input already multiplied by its first norm's weight when it fuses."""
        return self.mixer_norm if self.fuses(ctx) else None

    def forward(self, ctx, residual, pending, run_step: RunStep, next_block=None):
        """See parts.base.Block.  When this block runs its norms inside the products around them and the
        block behind it takes a prepared input, the down projection's epilogue prepares it."""
        T = residual.shape[0]
        if self.fuses(ctx):
            asks = getattr(next_block, "prepared_input_norm", None)      # None behind the last block
            next_norm = asks(ctx) if asks is not None else None
            if isinstance(pending, NormedInput):
                nx = pending
            else:
                n = ctx.workspace.get("block.normed", T, self.hidden, ctx.dtype)
                self.mixer_norm.apply(residual, pending, n)
                nx = NormedInput(n, None, self.hidden, self.mixer_norm.spec.eps)
            nx = self.mixer.forward_fused(ctx, nx, run_step, residual, self.ff_norm)
            return self.feed_forward.forward_fused(ctx, nx, residual, next_norm)
        assert not isinstance(pending, NormedInput), "a prepared input was handed to a block that did not ask for one"
        n = ctx.workspace.get("block.normed", T, self.hidden, ctx.dtype)
        self.mixer_norm.apply(residual, pending, n)
        mixed = self.mixer.forward(ctx, n, run_step)
        if self.feed_forward is None:
            return mixed                      # the next norm adds it
        self.ff_norm.apply(residual, mixed, n)
        return self.feed_forward.forward(ctx, n)


@register_block("parallel")
class ParallelBlock(Block):
    """One norm whose output both sublayers read; the sum of their results joins the stream:

        h = norm(x);   x <- x + (mixer(h) + ff(h))

    A feed-forward that takes an addend (``takes_addend``) adds the mixer's result where it forms its own;
    otherwise the mixer's result is added to the stream here and the feed-forward's is left pending."""

    def __init__(self, spec: LayerSpec, tensors: dict, mctx):
        p = spec.weight_prefix
        self.spec = spec
        self.norm = lookup(NORMS, spec.mixer_norm.kind, "norm")(spec.mixer_norm, p + spec.mixer_norm_name, tensors, mctx)
        self.mixer = lookup(MIXERS, spec.mixer.kind, "mixer")(spec.mixer, p, tensors, mctx)
        self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward = lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward")(
                spec.feed_forward, p, tensors, mctx)
        self.hidden = spec.mixer_norm.size
        self.replayable = all(getattr(part, "replayable", True) for part in (self.norm, self.mixer, self.feed_forward))

    @classmethod
    def tensor_decls(cls, spec: LayerSpec, prefix: str = "") -> List[TensorDecl]:
        p = spec.weight_prefix
        decls = (lookup(NORMS, spec.mixer_norm.kind, "norm").tensor_decls(spec.mixer_norm, p + spec.mixer_norm_name)
                 + lookup(MIXERS, spec.mixer.kind, "mixer").tensor_decls(spec.mixer, p))
        if spec.feed_forward is not None:
            decls += lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward").tensor_decls(spec.feed_forward, p)
        return decls

    def forward(self, ctx, residual, pending, run_step: RunStep, next_block=None):
        assert not isinstance(pending, NormedInput), "a prepared input was handed to a block that did not ask for one"
        n = ctx.workspace.get("block.normed", residual.shape[0], self.hidden, ctx.dtype)
        self.norm.apply(residual, pending, n)
        mixed = self.mixer.forward(ctx, n, run_step)
        if self.feed_forward is None:
            return mixed                      # the next norm adds it
        if getattr(self.feed_forward, "takes_addend", False):
            return self.feed_forward.forward(ctx, n, add=mixed)
        ops.residual_add(residual, mixed)
        return self.feed_forward.forward(ctx, n)


@register_block("sandwich_gated")
class SandwichGatedBlock(Block):
    """Norms on both sides of each sublayer, and a learned gate on the sublayer's result:

        n = norm_a(x);   x <- x + norm_b(sigmoid(R n + r) * sublayer(n))

    once for the mixer and, if the layer has one, once for the feed-forward.  R [hidden, hidden] and r
    read the same normed input as the sublayer.  The gate, the second norm, the addition into the float32
    residual stream and the norm ahead of the next sublayer are one kernel (ops.gated_postnorm_add)."""

    def __init__(self, spec: LayerSpec, tensors: dict, mctx):
        p = spec.weight_prefix
        self.spec = spec
        norm = lambda ns, name: lookup(NORMS, ns.kind, "norm")(ns, p + name, tensors, mctx)
        self.mixer_norm = norm(spec.mixer_norm, spec.mixer_norm_name)
        self.mixer_post_norm = norm(spec.mixer_post_norm, spec.mixer_post_norm_name)
        self.mixer = lookup(MIXERS, spec.mixer.kind, "mixer")(spec.mixer, p, tensors, mctx)
        self.mixer_gate = Linear(tensors[p + spec.mixer_gate_name], p + spec.mixer_gate_name)
        self.mixer_gate_bias = tensors[p + spec.mixer_gate_name + ".b"]
        self.feed_forward = None
        if spec.feed_forward is not None:
            self.ff_norm = norm(spec.feed_forward_norm, spec.feed_forward_norm_name)
            self.ff_post_norm = norm(spec.feed_forward_post_norm, spec.feed_forward_post_norm_name)
            self.feed_forward = lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward")(
                spec.feed_forward, p, tensors, mctx)
            self.ff_gate = Linear(tensors[p + spec.feed_forward_gate_name], p + spec.feed_forward_gate_name)
            self.ff_gate_bias = tensors[p + spec.feed_forward_gate_name + ".b"]
        self.hidden = spec.mixer_norm.size
        self.replayable = all(getattr(part, "replayable", True) for part in (self.mixer, self.feed_forward))

    @classmethod
    def tensor_decls(cls, spec: LayerSpec, prefix: str = "") -> List[TensorDecl]:
        p, H = spec.weight_prefix, spec.mixer_norm.size
        norm = lambda ns, name: lookup(NORMS, ns.kind, "norm").tensor_decls(ns, p + name)
        gate = lambda name: [TensorDecl(p + name, (H, H), MATRIX), TensorDecl(p + name + ".b", (H,), VECTOR)]
        decls = (norm(spec.mixer_norm, spec.mixer_norm_name) + norm(spec.mixer_post_norm, spec.mixer_post_norm_name)
                 + lookup(MIXERS, spec.mixer.kind, "mixer").tensor_decls(spec.mixer, p) + gate(spec.mixer_gate_name))
        if spec.feed_forward is not None:
            decls += (norm(spec.feed_forward_norm, spec.feed_forward_norm_name)
                      + norm(spec.feed_forward_post_norm, spec.feed_forward_post_norm_name)
                      + lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward").tensor_decls(spec.feed_forward, p)
                      + gate(spec.feed_forward_gate_name))
        return decls

    def _join(self, ctx, residual, sub, gate_logits, gate_bias, post_norm, next_norm, n):
        """residual += post_norm(sigmoid(gate) * sub); n = next_norm(residual) when something follows."""
        ops.gated_postnorm_add(residual, sub, gate_logits, gate_bias, post_norm.weight, post_norm.spec.eps,
                               next_norm.weight if next_norm is not None else None,
                               next_norm.spec.eps if next_norm is not None else 0.0,
                               n if next_norm is not None else None)

    def forward(self, ctx, residual, pending, run_step: RunStep, next_block=None):
        """See parts.base.Block.  A block of this kind behind this one gets its input already normed: the
        kernel that adds the last sublayer's result to the residual stream applies that block's first
        norm as well, and the NormedInput it is handed (without partial sums) says so."""
        T = residual.shape[0]
        n = ctx.workspace.get("block.normed", T, self.hidden, ctx.dtype)
        if isinstance(pending, NormedInput):
            assert pending.ss_parts is None and pending.xw.data_ptr() == n.data_ptr(), \
                "only a block of this kind hands this block a prepared input"
        else:
            self.mixer_norm.apply(residual, pending, n)
        after = next_block.mixer_norm if isinstance(next_block, SandwichGatedBlock) else None
        handed = NormedInput(n, None, self.hidden, after.spec.eps) if after is not None else None

        mixed = self.mixer.forward(ctx, n, run_step)
        gate = self.mixer_gate(ctx, n, "block.gate")
        self._join(ctx, residual, mixed, gate, self.mixer_gate_bias, self.mixer_post_norm,
                   self.ff_norm if self.feed_forward is not None else after, n)
        if self.feed_forward is None:
            return handed
        h = self.feed_forward.forward(ctx, n)
        gate = self.ff_gate(ctx, n, "block.gate")
        self._join(ctx, residual, h, gate, self.ff_gate_bias, self.ff_post_norm, after, n)
        return handed


@register_block("post_norm")
class PostNormBlock(Block):
    """The norm comes after the sum, and the stream itself is what gets normed:

        x <- norm_1(a x + mixer(x));   x <- norm_2(a x + ff(x))        a = ``residual_scale``

    The sublayers read the stream as it is (in the activation dtype).  One kernel per sublayer scales, adds, norms,
    rewrites the float32 stream and leaves the activation-dtype copy that the next sublayer's products read
    (ops.postnorm_scale_add), so nothing is left pending behind a block of this kind: a block of this kind behind it is
    handed that copy as its input (a NormedInput without partial sums); any other block norms the stream itself."""

    def __init__(self, spec: LayerSpec, tensors: dict, mctx):
        p = spec.weight_prefix
        self.spec = spec
        norm = lambda ns, name: lookup(NORMS, ns.kind, "norm")(ns, p + name, tensors, mctx)
        self.mixer_norm = norm(spec.mixer_norm, spec.mixer_norm_name)
        self.mixer = lookup(MIXERS, spec.mixer.kind, "mixer")(spec.mixer, p, tensors, mctx)
        self.ff_norm = self.feed_forward = None
        if spec.feed_forward is not None:
            self.ff_norm = norm(spec.feed_forward_norm, spec.feed_forward_norm_name)
            self.feed_forward = lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward")(
                spec.feed_forward, p, tensors, mctx)
        self.hidden = spec.mixer_norm.size
        self.alpha = float(spec.residual_scale)
        self.replayable = all(getattr(part, "replayable", True) for part in (self.mixer, self.feed_forward))

    @classmethod
    def tensor_decls(cls, spec: LayerSpec, prefix: str = "") -> List[TensorDecl]:
        return PreNormBlock.tensor_decls(spec, prefix)       # the same parts under the same names

    def _join(self, residual, sub, norm, copy):
        """sub: a sublayer's result, or two results with their weights ((y1, w1), (y2, w2)) that this kernel sums."""
        terms = sub if isinstance(sub, tuple) else None
        ops.postnorm_scale_add(residual, None if terms else sub, norm.weight, self.alpha, norm.spec.eps,
                               norm.spec.unit_offset, copy, terms=terms)

    def forward(self, ctx, residual, pending, run_step: RunStep, next_block=None):
        T = residual.shape[0]
        low = ctx.dtype != torch.float32
        # the sublayers' input: the stream itself in float32, its copy in the activation dtype otherwise
        x = ctx.workspace.get("block.normed", T, self.hidden, ctx.dtype) if low else residual
        if isinstance(pending, NormedInput):
            assert pending.ss_parts is None and pending.xw.data_ptr() == x.data_ptr(), \
                "only a block of this kind hands this block a prepared input"
        else:
            if pending is not None:
                ops.residual_add(residual, pending)
            if low:
                ops.cast(residual, x)
        if getattr(self.mixer, "offers_terms", False):      # a weighted pair: its sum rides in the kernel below
            mixed = self.mixer.forward(ctx, x, run_step, as_terms=True)
        else:
            mixed = self.mixer.forward(ctx, x, run_step)
        self._join(residual, mixed, self.mixer_norm, x if low else None)
        if self.feed_forward is not None:
            self._join(residual, self.feed_forward.forward(ctx, x), self.ff_norm, x if low else None)
        if isinstance(next_block, PostNormBlock):
            return NormedInput(x, None, self.hidden, 0.0)
        return None
