"""Attention over a cached latent.

Per token the pages hold one vector: the RMS-normed latent c (kv_rank elements) and, behind it, one
rotated key part (rot_dim elements) that all heads share.  Head h's unrotated key is U_k,h c and its
value U_v,h c; the score of query i on key j is (q_i . U_k,h c_j + qr_i . kr_j) * scale.  Neither keys
nor values are formed: the up projection of the keys is folded into the query (U_k,h^T q_i), the
attention runs over [c | kr] with the values being c itself, and the up projection of the values is
applied to the attended latent.  With ``output_gate`` each head's output is multiplied by the sigmoid of a
projection of the mixer's input before the output projection.  With ``q_rank`` the queries pass a latent of their
own: q = W_uq N(w, W_dq h).  With ``window`` a query sees itself and the window - 1 tokens before it, and the
pages behind the widest window of the entry's readers go back to the pool.  A mixer without a down projection
(``own_kv`` False) reads the latent and the rotated key part that the run step whose cache entry it names
cached, with up projections, queries and window of its own.

Prompts in bfloat16 (steps with an entry of more than four tokens) take the other road when the sizes
fit the tensor-core kernel: the latents of the entries' whole contexts are gathered from the pages, one
matrix product with [U_k; U_v] forms every head's unrotated keys and values for this step only, and the
attention runs in the heads' own space (dim + rot_dim per key, vdim per value: a third of the latent
form's arithmetic); the rotated key part is read from the pages.  What the pages hold is the same on
both roads, so a request may change between them from step to step; the float32 path always attends
in the latent space and its logits do not depend on the cutting.
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import PAGED_ALL, PAGED_WINDOW
from ..config.spec import LatentAttentionSpec, RunStep
from ..errors import ConfigError, Unsupported
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import POSITION_ENCODINGS, ROTATION, CacheNeed, Part, lookup, register_mixer
from .linear import Linear


@register_mixer("latent_attention")
class LatentAttention(Part):
    def __init__(self, spec: LatentAttentionSpec, prefix: str, tensors: dict, mctx):
        self.spec = s = spec
        p, nm = prefix, spec.names
        # one product for everything that reads the mixer's input: the queries (or their latent), the down projection
        # (layers that cache a latent of their own), the gate; float32 result
        q_rows = s.q_rank if s.q_rank else s.heads * (s.head_dim + s.rot_dim)
        rows = [tensors[p + (nm.q_down if s.q_rank else nm.q)]]
        if s.own_kv:
            rows.append(tensors[p + nm.down])
        if s.output_gate:
            rows.append(tensors[p + nm.gate])
        self.proj = Linear(torch.cat(rows, dim=0).contiguous(), p + "q_down_gate")
        self.c_off = q_rows
        self.g_off = q_rows + (s.kv_rank + s.rot_dim if s.own_kv else 0) if s.output_gate else -1
        self.q_norm_w = self.q_up = None
        if s.q_rank:
            self.q_norm_w = tensors[p + nm.q_norm]
            self.q_up = Linear(tensors[p + nm.q_up], p + nm.q_up)
        self.latent_norm_w = tensors[p + nm.latent_norm] if s.own_kv else None
        self.uk = tensors[p + nm.up_k].view(s.heads, s.head_dim, s.kv_rank).contiguous()
        # per head [kv_rank, v_head_dim]: a thread of the expanding kernel owns one output column
        self.uv_t = tensors[p + nm.up_v].view(s.heads, s.v_head_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.out = Linear(tensors[p + nm.o], p + nm.o)
        # [U_k; U_v] as one weight, for prompts that form per-head keys and values (bfloat16 only)
        self.up_kv = None
        if mctx.dtype == torch.bfloat16 and tensors[p + nm.up_k].dtype == torch.bfloat16:
            self.up_kv = torch.cat([tensors[p + nm.up_k], tensors[p + nm.up_v]], dim=0).contiguous()
        self.position = None
        if s.position is not None:
            self.position = lookup(POSITION_ENCODINGS, s.position.kind, "position encoding")(s.position, mctx)
            if getattr(self.position, "applies", ROTATION) != ROTATION:
                raise Unsupported(f"position encoding {s.position.kind!r} is not a rotation")

    @classmethod
    def tensor_decls(cls, s: LatentAttentionSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.names
        hd = s.heads * (s.head_dim + s.rot_dim)
        if s.q_rank:
            decls = [TensorDecl(p + nm.q_down, (s.q_rank, s.hidden_size), MATRIX),
                     TensorDecl(p + nm.q_norm, (s.q_rank,), VECTOR),
                     TensorDecl(p + nm.q_up, (hd, s.q_rank), MATRIX)]
        else:
            decls = [TensorDecl(p + nm.q, (hd, s.hidden_size), MATRIX)]
        if s.own_kv:
            decls += [TensorDecl(p + nm.down, (s.kv_rank + s.rot_dim, s.hidden_size), MATRIX),
                      TensorDecl(p + nm.latent_norm, (s.kv_rank,), VECTOR)]
        decls += [TensorDecl(p + nm.up_k, (s.heads * s.head_dim, s.kv_rank), MATRIX),
                  TensorDecl(p + nm.up_v, (s.heads * s.v_head_dim, s.kv_rank), MATRIX)]
        if s.output_gate:
            decls.append(TensorDecl(p + nm.gate, (s.heads, s.hidden_size), MATRIX))
        decls.append(TensorDecl(p + nm.o, (s.hidden_size, s.heads * s.v_head_dim), MATRIX))
        return decls

    @classmethod
    def cache_need_of(cls, s: LatentAttentionSpec) -> CacheNeed:
        # one KV head of kv_rank + rot_dim elements per token, and no value pool: the values are the latent
        if s.window and s.cache_window and s.cache_window < s.window:
            raise ConfigError("a latent attention's cache keeps fewer keys than its window sees")
        keeps = s.cache_window if s.window else None
        return CacheNeed(PAGED_WINDOW if keeps else PAGED_ALL, 1, s.kv_rank + s.rot_dim, keeps, v_head_dim=0)

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep) -> torch.Tensor:
        s = self.spec
        T = x.shape[0]
        if run_step.writes_cache != s.own_kv:
            raise ConfigError("a latent attention writes its cache entry exactly when it has a down projection of its own")
        proj = self.proj(ctx, x, "latent.proj", out_dtype=torch.float32)
        cache, _, group = ctx.cache.kv_of_entry(run_step.cache)
        rot = self.position.rotation(ctx) if self.position is not None else None
        cq = ctx.workspace.get("latent.cq", T, s.q_rank, ctx.dtype) if s.q_rank else None
        if s.own_kv:       # the kernel that norms and appends the latent norms the queries' latent too
            ops.latent_append(proj, self.c_off, self.latent_norm_w, s.latent_norm_eps, rot, cache, ctx.kv_slot[group],
                              s.kv_rank, s.rot_dim, q_norm=(0, s.q_rank, self.q_norm_w, cq) if s.q_rank else None)
        elif s.q_rank:
            ops.rmsnorm_columns(proj, 0, s.q_rank, self.q_norm_w, s.latent_norm_eps, cq)
        q_heads = proj                 # heads x [dim | rot_dim] lead the row
        if s.q_rank:
            q_heads = self.q_up(ctx, cq, "latent.q_heads_raw", out_dtype=torch.float32)
        gated = ctx.workspace.get("latent.out", T, s.heads * s.v_head_dim, ctx.dtype)
        if (self.up_kv is not None and ctx.max_q_len > 4
                and ops.latent_prompt_takes(s.head_dim, s.rot_dim, s.v_head_dim, s.kv_rank)):
            self._attend_in_head_space(ctx, proj, q_heads, cache, group, rot, gated)
            return self.out(ctx, gated, "latent.proj_out")
        qd = s.kv_rank + s.rot_dim
        q = ctx.workspace.get("latent.q", T, s.heads * qd, torch.float32)
        ops.latent_absorb(q_heads, self.uk, rot, q, s.heads, s.head_dim, s.rot_dim, s.kv_rank)
        o_lat = ctx.workspace.get("latent.o", T, s.heads * s.kv_rank, torch.float32)
        ops.paged_attention_general(ctx, q, cache, None, o_lat, ctx.block_tables[group], None, s.heads, 1, qd,
                                    s.kv_rank, s.softmax_scale, s.window or 0)
        ops.latent_expand(o_lat, self.uv_t, proj, self.g_off, gated, s.heads, s.kv_rank, s.v_head_dim)
        return self.out(ctx, gated, "latent.proj_out")

    def _attend_in_head_space(self, ctx, proj, q_heads, cache, group, rot, gated) -> None:
        """Prompts: gather the contexts' latents (from the first key that the step's rows still see), form all heads'
        unrotated keys and values with one product, attend per head, gate.  Key j of entry e lies in row cu_kv[e] + j
        of the gathered matrices."""
        s = self.spec
        T = proj.shape[0]
        key = ("latent.cu_kv", s.window)
        if key not in ctx.tables:
            cu, first, total = [], [], 0
            for n, q_len in zip(ctx.host["kv_lens"], ctx.host["q_lens"]):
                f = max(0, n - q_len - s.window + 1) if s.window else 0
                cu.append(total - f)
                first.append(f)
                total += n - f
            both = torch.tensor([cu, first], dtype=torch.int32).pin_memory().to(proj.device, non_blocking=True)
            ctx.tables[key] = (both[0], both[1], total)
        cu_kv, kv_first, keys = ctx.tables[key]
        latents = ctx.workspace.get("latent.gathered", keys, s.kv_rank, ctx.dtype)
        ops.latent_gather(ctx, cache, latents, ctx.block_tables[group], cu_kv, s.kv_rank, kv_first)
        kv_rows = ctx.workspace.get("latent.kv_rows", keys, s.heads * (s.head_dim + s.v_head_dim), ctx.dtype)
        ops.gemm(latents, self.up_kv, kv_rows)
        q = ctx.workspace.get("latent.q_heads", T, s.heads * (s.head_dim + s.rot_dim), torch.float32)
        ops.latent_rotate_q(q_heads, rot, q, s.heads, s.head_dim, s.rot_dim)
        # without a gate the attention writes the output projection's input itself
        attended = ctx.workspace.get("latent.o_heads", T, s.heads * s.v_head_dim, torch.float32) if s.output_gate else gated
        ops.latent_prefill_attention(ctx, q, cache, kv_rows, cu_kv, attended, ctx.block_tables[group], s.heads,
                                     s.head_dim, s.rot_dim, s.v_head_dim, s.kv_rank, s.heads * s.head_dim, s.softmax_scale,
                                     s.window or 0)
        if s.output_gate:
            ops.head_gate(attended, proj, self.g_off, gated, s.heads, s.v_head_dim)
