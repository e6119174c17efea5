"""Dovorax: config.json keys -> ModelSpec.

A Dovorax model is a list of layers that norm AFTER the sum: x <- norm(alpha x + sublayer(x)), once for the mixer
and, if the layer has one, once for the feed-forward (``postln_alpha``; the norm's weight is stored around zero and
applied as 1 + w).  The sublayers read the stream itself.  ``type`` names the mixer:

* ``latent_attention``: attention over a cached latent and one shared rotated key part, queries through a latent of
  their own (``q_rank``), a sliding window (``mask.size``), rotary pairs (i, i + dims/2) with the frequencies ramped
  down (``rot.scaling``).  With ``kv_from: j`` the layer has no down projection and reads what layer j cached.
* ``parallel``: two mixers on the same input, added with the weights ``left_scale`` and ``right_scale`` --
  ``left``, grouped-query attention behind short convolutions with a per-head norm of q and k, a rotation of the
  leading ``rot.dims`` elements and one more term in the softmax denominator; ``right``, a matrix memory with
  exponential gates.
* ``rglru``: a gated linear recurrence per channel behind a short convolution, beside a gate branch.

``mlp`` is null, ``kind: dense`` (down(gelu(up h))) or ``kind: moe`` (routed experts of that form, chosen among the
best groups by a softmax over all experts, plus a shared expert).  The output head is the embedding table.  Tensor
names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.mlp.*``, ``final.norm``.  No key has a
default: what config.json does not give, the model does not have.
"""
from __future__ import annotations

import dataclasses
import math

from ..errors import ConfigError, Unsupported
from .spec import (ConvAttentionNames, ConvAttentionSpec, DenseNames, DenseSpec, GatedRecurrenceNames,
                   GatedRecurrenceSpec, LatentAttentionNames, LatentAttentionSpec, LayerSpec, MatrixMemoryNames,
                   MatrixMemorySpec, ModelSpec, NormSpec, PositionSpec, RoutedExpertsSpec, RunStep, SideBySideSpec)

ARCHITECTURE = "Dovorax"
MAX_LAYERS = 4096
MAX_POSITIONS = 1 << 24       # the design sets no limit; angles are formed in double precision


def _int(d: dict, key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}{key!r} must be a positive integer, got {v!r}")
    return v


def _num(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise ConfigError(f"config.json: {where}{key!r} must be a finite positive number, got {v!r}")
    return float(v)


def _real(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"config.json: {where}{key!r} must be a finite number, got {v!r}")
    return float(v)


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


def _position(m: dict, dim: int, where: str) -> PositionSpec:
    rot = _obj(m, "rot", where)
    dims = _int(rot, "dims", where + "rot.")
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most {dim}")
    ramp = None
    if rot.get("scaling") is not None:
        sc, w = _obj(rot, "scaling", where + "rot."), where + "rot.scaling."
        ramp = (_num(sc, "factor", w), _num(sc, "original", w), _num(sc, "fast", w), _num(sc, "slow", w))
    return PositionSpec("rotary_half", theta=_num(rot, "base", where + "rot."), rotary_dim=dims, head_dim=dim, ramp=ramp)


def _window(m: dict, where: str):
    return _int(_obj(m, "mask", where), "size", where + "mask.") if m.get("mask") is not None else None


def _latent(m: dict, width: int, eps: float, where: str) -> LatentAttentionSpec:
    rot_dim = _int(m, "rot_dim", where)
    position = _position(m, rot_dim, where)
    if position.rotary_dim != rot_dim:
        raise ConfigError(f"config.json: {where}rot.dims must equal rot_dim {rot_dim}")
    window = _window(m, where)
    return LatentAttentionSpec(
        kind="latent_attention", hidden_size=width, heads=_int(m, "heads", where), head_dim=_int(m, "dim", where),
        rot_dim=rot_dim, v_head_dim=_int(m, "vdim", where), kv_rank=_int(m, "kv_rank", where),
        softmax_scale=_num(m, "scale", where), position=position, latent_norm_eps=eps, output_gate=False,
        q_rank=_int(m, "q_rank", where), window=window, cache_window=window, own_kv="kv_from" not in m,
        names=LatentAttentionNames(q_down="mix.dq", q_norm="mix.dq.norm", q_up="mix.uq", down="mix.dkv",
                                   latent_norm="mix.dkv.norm", up_k="mix.uk", up_v="mix.uv", o="mix.o"))


def _conv_attention(m: dict, width: int, eps: float, where: str, prefix: str) -> ConvAttentionSpec:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}heads {heads} is not a multiple of kv_heads {kv}")
    dim = _int(m, "dim", where)
    return ConvAttentionSpec(
        kind="conv_attention", hidden_size=width, heads=heads, kv_heads=kv, head_dim=dim,
        v_head_dim=_int(m, "vdim", where), softmax_scale=_num(m, "scale", where), conv_taps=_int(m, "conv", where),
        qk_norm_eps=eps, position=_position(m, dim, where) if m.get("rot") is not None else None, unit_sink=True,
        window=_window(m, where),
        names=ConvAttentionNames(prefix + "q", prefix + "k", prefix + "v", prefix + "o", ".conv", ".norm"))


def _matrix_memory(m: dict, width: int, eps: float, where: str, prefix: str) -> MatrixMemorySpec:
    return MatrixMemorySpec(
        kind="matrix_memory", hidden_size=width, heads=_int(m, "heads", where), head_dim=_int(m, "dim", where),
        v_head_dim=_int(m, "vdim", where), gate_cap=_num(m, "gate_cap", where), norm_eps=eps,
        names=MatrixMemoryNames(prefix + "q", prefix + "k", prefix + "v", prefix + "g", prefix + "i", prefix + "f",
                                prefix + "norm", prefix + "o"))


def _recurrence(m: dict, width: int, where: str) -> GatedRecurrenceSpec:
    channels, blocks = _int(m, "width", where), _int(m, "blocks", where)
    if channels % blocks:
        raise ConfigError(f"config.json: {where}width {channels} is not a multiple of blocks {blocks}")
    return GatedRecurrenceSpec(kind="gated_linear_recurrence", hidden_size=width, width=channels, blocks=blocks,
                               conv_taps=_int(m, "conv", where), decay_scale=8.0, names=GatedRecurrenceNames())


def _feed_forward(mlp: dict, width: int, where: str):
    kind = mlp.get("kind")
    if kind == "dense":
        return DenseSpec("dense", width, _int(mlp, "ff", where), "gelu", dense_names=DenseNames("mlp.up", "mlp.down"))
    if kind != "moe":
        raise Unsupported(f"config.json: {where}kind {kind!r}: a Dovorax feed-forward is 'dense' or 'moe'")
    expert, router = _obj(mlp, "expert", where), _obj(mlp, "router", where)
    experts, top = _int(router, "experts", where + "router."), _int(router, "top", where + "router.")
    groups = kept = 1
    if router.get("groups") is not None:
        g = _obj(router, "groups", where + "router.")
        groups, kept = _int(g, "count", where + "router.groups."), _int(g, "keep", where + "router.groups.")
    if experts % groups or kept > groups:
        raise ConfigError(f"config.json: {where}router: {experts} experts in {groups} groups of which {kept} are kept")
    if top > experts // groups * kept:
        raise ConfigError(f"config.json: {where}router.top {top} exceeds the experts of the kept groups")
    shared = _int(_obj(mlp, "shared", where), "ff", where + "shared.") if mlp.get("shared") is not None else 0
    return RoutedExpertsSpec("routed_experts", width, _int(expert, "ff", where + "expert."), "gelu", experts=experts,
                             top=top, router_bias=False, shared_size=shared, scoring="softmax_over_all", groups=groups,
                             groups_kept=kept, gated=False)


def read_spec(root: dict) -> ModelSpec:
    if root.get("architecture") != ARCHITECTURE:
        raise ConfigError(f"config.json: architecture {root.get('architecture')!r} is not {ARCHITECTURE}")
    width, vocab = _int(root, "width", ""), _int(root, "vocab", "")
    eps = _num(_obj(root, "norm", ""), "eps", "norm.")
    alpha = _real(root, "postln_alpha", "")
    entries = root.get("layers")
    if not isinstance(entries, list) or not entries or len(entries) > MAX_LAYERS:
        raise ConfigError(f"config.json: 'layers' must list 1 to {MAX_LAYERS} layers")
    norm = NormSpec("rmsnorm", width, eps, unit_offset=True)

    mixers = []
    for i, entry in enumerate(entries):
        where = f"layers[{i}]."
        if not isinstance(entry, dict) or not isinstance(entry.get("type"), str):
            raise ConfigError(f"config.json: {where[:-1]} must be an object with a 'type'")
        m, w = _obj(entry, "mixer", where), where + "mixer."
        if entry["type"] == "latent_attention":
            mixers.append(_latent(m, width, eps, w))
        elif entry["type"] == "parallel":
            left = _conv_attention(_obj(m, "left", w), width, eps, w + "left.", "mix.left.")
            right = _matrix_memory(_obj(m, "right", w), width, eps, w + "right.", "mix.right.")
            mixers.append(SideBySideSpec(kind="side_by_side", hidden_size=width, mixers=(left, right),
                                         combine="weighted_sum",
                                         weights=(_real(m, "left_scale", w), _real(m, "right_scale", w))))
        elif entry["type"] == "rglru":
            mixers.append(_recurrence(m, width, w))
        else:
            raise Unsupported(f"config.json: {where[:-1]} has type {entry['type']!r}; a Dovorax layer is "
                              f"'latent_attention', 'parallel' or 'rglru'")

    # a layer that reads layer j's latent and key part reads j's cache entry; the entry keeps the widest window
    source = {}
    for i, entry in enumerate(entries):
        if entry["type"] == "latent_attention" and "kv_from" in entry["mixer"]:
            j, where = entry["mixer"]["kv_from"], f"layers[{i}].mixer."
            if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
                raise ConfigError(f"config.json: {where}'kv_from' must name an earlier layer, got {j!r}")
            a, b = mixers[i], mixers[j]
            if not isinstance(b, LatentAttentionSpec) or not b.own_kv:
                raise ConfigError(f"config.json: {where}kv_from {j}: that layer caches no latent of its own")
            if (a.kv_rank, a.rot_dim, a.position) != (b.kv_rank, b.rot_dim, b.position):
                raise ConfigError(f"config.json: {where}kv_from {j}: kv_rank, rot_dim and rotation must equal that layer's")
            source[i] = j
    for j in set(source.values()):
        readers = [j] + [i for i in source if source[i] == j]
        windows = [mixers[i].window for i in readers]
        widest = None if any(w is None for w in windows) else max(windows)
        for i in readers:
            mixers[i] = dataclasses.replace(mixers[i], cache_window=widest)

    from .. import parts  # noqa: F401  (registers the mixers)
    from ..parts.base import MIXERS, lookup       # how many cache entries a mixer's run step names
    layers, run_order, entry_of, next_entry = [], [], {}, 0
    for i, entry in enumerate(entries):
        where = f"layers[{i}]."
        ff = _feed_forward(_obj(entry, "mlp", where), width, where + "mlp.") if entry.get("mlp") is not None else None
        layers.append(LayerSpec(block="post_norm", mixer=mixers[i], feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=norm if ff else None, weight_prefix=f"l{i}.",
                                mixer_norm_name="norm1", feed_forward_norm_name="norm2", residual_scale=alpha))
        if i in source:
            run_order.append(RunStep(i, entry_of[source[i]], writes_cache=False))
            continue
        need = lookup(MIXERS, mixers[i].kind, "mixer").cache_need_of(mixers[i])
        n = len(need) if isinstance(need, tuple) else 1
        entry_of[i] = next_entry
        run_order.append(RunStep(i, next_entry, True, more_caches=tuple(range(next_entry + 1, next_entry + n))))
        next_entry += n
    return ModelSpec(architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab,
                     max_position_embeddings=MAX_POSITIONS, layers=tuple(layers), run_order=tuple(run_order),
                     final_norm=norm, tie_word_embeddings=True, eos_token_ids=(),
                     embed_name="embed", final_norm_name="final.norm", head_name="head")
