"""A feed-forward of routed experts, plus one expert that every token runs.

    z = W_r h + b                      float32
    E(h) = the ``top`` experts with the largest z;  w = softmax(z restricted to E(h))
    out = sum_{e in E(h)} w_e * expert_e(h)  +  shared(h)
    expert(h) = W_down (g * logistic(alpha g) * (u + 1)),  g = min(W_gate h, limit),  u = clamp(W_up h, -limit, limit)

Variants by the specification: ``scoring`` "logistic" takes w_e = logistic(z_e), not renormalised; ``activation``
"silu" is the plain gate * logistic(gate) * up; ``weight_on_input`` computes sum_e expert_e(w_e h) instead: the
experts have no biases, so W (w h) = w (W h), and the first grouped product multiplies its gate and up sums by
the pair's weight ahead of the activation (steps of many tokens, whose rows are gathered into tiles, scale the
gathered rows).

``gated`` False: an expert (and the shared one) is W_down act(W_up h) with ``activation`` "gelu" (the exact one).
``scoring`` "softmax_over_all": the scores are the softmax over all experts' logits, the choice may be limited to the
best ``groups_kept`` of ``groups`` equal groups of neighbouring experts (a group counts as its largest score), and the
weights are the chosen scores over their sum.

The pairs (token, chosen expert) are ordered by expert on the device and every expert's rows run through
one grouped product per projection; a token's result does not depend on what else is in the step, and
nothing is planned on the host, so decode steps replay from CUDA graphs.
"""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import RoutedExpertsSpec
from ..errors import Unsupported
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import Part, register_feed_forward
from .linear import Linear


@register_feed_forward("routed_experts")
class RoutedExperts(Part):
    def __init__(self, spec: RoutedExpertsSpec, prefix: str, tensors: dict, mctx):
        if spec.activation not in (("clamped_glu", "silu") if spec.gated else ("gelu",)):
            raise Unsupported(f"routed experts with activation {spec.activation!r} are not implemented")
        if not spec.gated and spec.weight_on_input:
            raise Unsupported("a weight on an expert's input comes with gated experts only")
        if spec.scoring not in ops.ROUTER_SCORING:
            raise Unsupported(f"routed experts with router scoring {spec.scoring!r} are not implemented")
        if spec.activation == "silu" and spec.shared_size:
            raise Unsupported("an expert that every token runs comes with the clamped activation only")
        self.spec = spec
        self.groups = (spec.groups, spec.groups_kept)
        if not spec.gated:
            self._init_plain(spec, prefix, tensors, mctx)
            return
        self.limit = spec.limit if spec.activation == "clamped_glu" else 0.0      # 0: the plain gated activation
        p, nm = prefix, spec.expert_names
        self.router_bias = tensors[p + nm.router_bias] if spec.router_bias else None
        each = lambda part: [tensors[p + nm.expert.format(e) + part] for e in range(spec.experts)]
        # [experts, 2 ff, hidden] and [experts, hidden, ff].  For the tensor-core product the gate and up rows are
        # interleaved in blocks of 16 (8 gate rows, then the 8 up rows of the same features), so that its epilogue
        # holds both halves of a feature; otherwise per expert the gate rows, then the up rows.
        I, H = spec.intermediate_size, spec.hidden_size
        self.interleaved = (mctx.dtype == torch.bfloat16 and I % 8 == 0 and H % 8 == 0
                            and tensors[p + nm.expert.format(0) + nm.gate].dtype == torch.bfloat16)
        if self.interleaved:
            pair = lambda g, u: torch.stack([g.view(I // 8, 8, H), u.view(I // 8, 8, H)], dim=1).reshape(2 * I, H)
        else:
            pair = lambda g, u: torch.cat([g, u], dim=0)
        self.in_tiles = self.interleaved         # steps of many tokens may run the experts' products in whole tiles
        self.gate_up = torch.stack([pair(g, u) for g, u in zip(each(nm.gate), each(nm.up))]).contiguous()
        self.down = torch.stack(each(nm.down)).contiguous()
        # one product for everything that reads the layer's input whole: the shared expert's gate rows, its up
        # rows, then the router's rows; its result is float32 (the router's logits are)
        first, self.shared_down = [tensors[p + nm.router]], None
        if spec.shared_size:
            sp = p + nm.shared
            first = [tensors[sp + nm.gate], tensors[sp + nm.up]] + first
            self.shared_down = Linear(tensors[sp + nm.down], sp + nm.down)
        self.first = Linear(torch.cat(first, dim=0).contiguous(), p + "shared_gate_up_router")
        self.router_column = 2 * spec.shared_size

    def _init_plain(self, spec, prefix, tensors, mctx):
        """Experts without a gate: [experts, ff, hidden] and [experts, hidden, ff]; the first product of the layer's input
        stacks the shared expert's up rows and the router's rows (float32 result)."""
        p, nm = prefix, spec.expert_names
        each = lambda part: [tensors[p + nm.expert.format(e) + part] for e in range(spec.experts)]
        self.router_bias = tensors[p + nm.router_bias] if spec.router_bias else None
        self.interleaved = False
        self.limit = 0.0
        I, H = spec.intermediate_size, spec.hidden_size
        self.in_tiles = (mctx.dtype == torch.bfloat16 and I % 8 == 0 and H % 8 == 0
                         and tensors[p + nm.expert.format(0) + nm.up].dtype == torch.bfloat16)
        self.gate_up = torch.stack(each(nm.up)).contiguous()
        self.down = torch.stack(each(nm.down)).contiguous()
        first, self.shared_down = [tensors[p + nm.router]], None
        if spec.shared_size:
            sp = p + nm.shared
            first = [tensors[sp + nm.up]] + first
            self.shared_down = Linear(tensors[sp + nm.down], sp + nm.down)
        self.first = Linear(torch.cat(first, dim=0).contiguous(), p + "shared_up_router")
        self.router_column = spec.shared_size

    @classmethod
    def tensor_decls(cls, s: RoutedExpertsSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.expert_names
        H = s.hidden_size
        decls = []
        for e in range(s.experts):
            ep = p + nm.expert.format(e)
            if s.gated:
                decls.append(TensorDecl(ep + nm.gate, (s.intermediate_size, H), MATRIX))
            decls += [TensorDecl(ep + nm.up, (s.intermediate_size, H), MATRIX),
                      TensorDecl(ep + nm.down, (H, s.intermediate_size), MATRIX)]
        decls.append(TensorDecl(p + nm.router, (s.experts, H), MATRIX))
        if s.router_bias:
            decls.append(TensorDecl(p + nm.router_bias, (s.experts,), VECTOR))
        if s.shared_size:
            sp = p + nm.shared
            if s.gated:
                decls.append(TensorDecl(sp + nm.gate, (s.shared_size, H), MATRIX))
            decls += [TensorDecl(sp + nm.up, (s.shared_size, H), MATRIX), TensorDecl(sp + nm.down, (H, s.shared_size), MATRIX)]
        return decls

    takes_addend = True       # forward(..., add=...) adds a tensor of the output's shape and dtype in the combination

    def forward(self, ctx, x: torch.Tensor, add=None) -> torch.Tensor:
        s = self.spec
        T, H = x.shape
        ws = ctx.workspace
        pairs = T * s.top
        if add is not None and self.shared_down is not None:
            raise Unsupported("routed experts add either their shared expert's output or a given tensor")
        # the router in float32: its input may be the activation dtype's rounding of the normed stream
        first = self.first(ctx, x, "moe.first", out_dtype=torch.float32)
        choice = ws.get("moe.choice", T, s.top, torch.int32)
        weight = ws.get("moe.weight", T, s.top, torch.float32)
        # steps of many tokens (64 rows an expert on average): the experts' products on the persistent tensor-memory
        # kernel, every expert's rows in whole tiles of 128 of a gathered copy of the input
        if (self.in_tiles and ops.grouped_products_in_tensor_memory and pairs >= 64 * s.experts
                and s.intermediate_size % 8 == 0):
            ops.moe_route(first, self.router_bias, s.top, choice, weight, column=self.router_column, experts=s.experts,
                          scoring=s.scoring, groups=self.groups)
            return self._forward_tiles(ctx, x, first, choice, weight, add)
        heads = ws.get("moe.heads", 2, s.experts + 1, torch.int32, reserve=2)
        order = ws.get("moe.order", 2 * T, s.top, torch.int32, reserve=2 * ws.max_tokens)
        offsets, tiles = heads[0], heads[1]
        pair_of_row, row_of_pair = order[:T].view(-1), order[T:].view(-1)
        if ops.moe_sort_routes(T, s.experts):          # a small step: the block that orders the pairs routes them too
            ops.moe_sort(choice, s.experts, offsets, tiles, pair_of_row, row_of_pair,
                         route=(first, self.router_column, self.router_bias, weight), scoring=s.scoring,
                         groups=self.groups)
        else:
            ops.moe_route(first, self.router_bias, s.top, choice, weight, column=self.router_column, experts=s.experts,
                          scoring=s.scoring, groups=self.groups)
            ops.moe_sort(choice, s.experts, offsets, tiles, pair_of_row, row_of_pair)
        y = ws.get("moe.y", pairs, s.intermediate_size, ctx.dtype, reserve=ws.max_tokens * s.top)
        if s.gated:
            ops.moe_grouped(x, pair_of_row, s.top, self.gate_up, y, offsets, tiles, glu=True, interleaved=self.interleaved,
                            limit=self.limit, alpha=s.glu_alpha, pair_scale=weight if s.weight_on_input else None)
        else:
            ops.moe_grouped(x, pair_of_row, s.top, self.gate_up, y, offsets, tiles, act=s.activation)
        rows = ws.get("moe.rows", pairs, H, torch.float32, reserve=ws.max_tokens * s.top)
        ops.moe_grouped(y, None, 1, self.down, rows, offsets, tiles)
        out = ws.get("moe.out", T, H, ctx.dtype)
        ops.moe_combine(rows, row_of_pair.view(T, s.top), None if s.weight_on_input else weight,
                        add if add is not None else self._shared(ctx, first), out)
        return out

    def _shared(self, ctx, first):
        """The output of the expert that every token runs (its gate and up columns lead the first product), or None."""
        if self.shared_down is None:
            return None
        s = self.spec
        ys = ctx.workspace.get("moe.shared_y", first.shape[0], s.shared_size, ctx.dtype)
        if s.gated:
            ops.clamped_glu(first, ys, s.shared_limit, s.glu_alpha)
        else:
            ops.activation(first, ys, s.activation)
        return self.shared_down(ctx, ys, "moe.shared_out")

    def _forward_tiles(self, ctx, x, first, choice, weight, add=None):
        s = self.spec
        T, H = x.shape
        ws = ctx.workspace
        tile = ops.grouped_tile_rows(T * s.top, s.experts, (2 if s.gated else 1) * s.intermediate_size * H)
        n_tiles = (T * s.top) // tile + s.experts            # every expert wastes less than one tile
        rows_cap = n_tiles * tile
        heads = ws.get("moe.heads", 2, s.experts + 1, torch.int32, reserve=2)
        group_of_tile = ws.get("moe.group_of_tile", n_tiles, 1, torch.int32, reserve=0).view(-1)
        pair_of_row = ws.get("moe.pair_of_row", rows_cap, 1, torch.int32, reserve=0).view(-1)
        row_of_pair = ws.get("moe.row_of_pair", T, s.top, torch.int32).view(-1)
        ops.moe_sort(choice, s.experts, heads[0], heads[1], pair_of_row, row_of_pair, tile_rows=tile,
                     group_of_tile=group_of_tile)
        xs = ws.get("moe.xs", rows_cap, H, ctx.dtype, reserve=0)
        ops.moe_gather_rows(x, pair_of_row, s.top, xs, pair_scale=weight if s.weight_on_input else None)
        y = ws.get("moe.y_tiles", rows_cap, s.intermediate_size, ctx.dtype, reserve=0)
        if s.gated:
            ops.gemm_tn_tcgen05_grouped(xs, self.gate_up, y, group_of_tile, glu=True, limit=self.limit, alpha=s.glu_alpha,
                                        tile_rows=tile)
        else:
            ops.gemm_tn_tcgen05_grouped(xs, self.gate_up, y, group_of_tile, act=s.activation, tile_rows=tile)
        rows = ws.get("moe.rows_tiles", rows_cap, H, torch.float32, reserve=0)
        ops.gemm_tn_tcgen05_grouped(y, self.down, rows, group_of_tile, tile_rows=tile)
        out = ws.get("moe.out", T, H, ctx.dtype)
        ops.moe_combine(rows, row_of_pair.view(T, s.top), None if s.weight_on_input else weight,
                        add if add is not None else self._shared(ctx, first), out)
        return out
