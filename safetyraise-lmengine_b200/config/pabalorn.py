"""Pabalorn: config.json keys -> ModelSpec.

A Pabalorn model is a list of parallel layers: one norm (its weight stored around zero, applied as 1 + w), whose
output both the mixer and the feed-forward read; their sum joins the stream.  ``type`` names the mixer:

* ``attention``: rotated attention (pairs (i, i + dims/2) of the first ``rot.dims`` elements of a head), scores
  capped by a tanh (``softcap``), a sliding window (``mask.size``), no biases.  With ``kv_from: j`` the layer
  has no key and value projections and attends over what layer j cached.
* ``parallel``: two mixers side by side on the same input -- ``left``, rotated attention with biases on q, k
  and v, interleaved pairs (2i, 2i + 1) and optionally rescaled frequencies (``rot.scaling``); ``right``, a
  selective scan -- each output RMS-normed with a plain weight, then averaged.

``mlp`` is a feed-forward of routed experts (``kind: moe``) or null.  The router scores are logistic, the
chosen scores are the weights as they are, and a weight multiplies its expert's input.  The embedded tokens
are normed before the first layer and the output head is the embedding table.  Tensor names: ``embed``,
``embed.norm``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.  No key has a default: what
config.json does not give, the model does not have.
"""
from __future__ import annotations

import math

from ..errors import ConfigError, Unsupported
from .spec import (LayerSpec, ModelSpec, NormSpec, PositionSpec, RotatedAttentionNames, RotatedAttentionSpec,
                   RoutedExpertsSpec, RunStep, SelectiveScanNames, SelectiveScanSpec, SideBySideSpec)

ARCHITECTURE = "Pabalorn"
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


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


def _position(m: dict, dim: int, kind: str, where: str):
    if m.get("rot") is None:
        return None
    rot = _obj(m, "rot", where)
    dims = _int(rot, "dims", where + "rot.")
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most the head size {dim}")
    scaling = None
    if rot.get("scaling") is not None:
        sc = _obj(rot, "scaling", where + "rot.")
        w = where + "rot.scaling."
        scaling = (_num(sc, "factor", w), _num(sc, "low", w), _num(sc, "high", w), _num(sc, "original", w))
        if scaling[2] <= scaling[1]:
            raise ConfigError(f"config.json: {w}high must exceed low")
    return PositionSpec(kind, theta=_num(rot, "base", where + "rot."), rotary_dim=dims, head_dim=dim, scaling=scaling)


def _attention(m: dict, width: int, where: str, prefix: str, bias: bool, rotary: str) -> RotatedAttentionSpec:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}heads {heads} is not a multiple of kv_heads {kv}")
    dim = _int(m, "dim", where)
    window = _int(_obj(m, "mask", where), "size", where + "mask.") if m.get("mask") is not None else None
    return RotatedAttentionSpec(
        kind="rotated_attention", hidden_size=width, heads=heads, kv_heads=kv, head_dim=dim,
        v_head_dim=_int(m, "vdim", where), softmax_scale=_num(m, "scale", where),
        position=_position(m, dim, rotary, where),
        softcap=_num(m, "softcap", where) if m.get("softcap") is not None else None,
        window=window, cache_window=window, bias=bias, own_kv="kv_from" not in m,
        names=RotatedAttentionNames(prefix + "q", prefix + "k", prefix + "v", prefix + "o", ".b"))


def _scan(m: dict, width: int, where: str, prefix: str) -> SelectiveScanSpec:
    return SelectiveScanSpec(
        kind="selective_scan", hidden_size=width, inner=_int(m, "inner", where), state=_int(m, "state", where),
        dt_rank=_int(m, "dt_rank", where), conv_taps=_int(m, "conv", where),
        names=SelectiveScanNames(prefix + "in", prefix + "conv", prefix + "x", prefix + "dt", prefix + "A_log",
                                 prefix + "D", prefix + "o"))


def _feed_forward(mlp: dict, width: int, where: str):
    if mlp.get("kind") != "moe":
        raise Unsupported(f"config.json: {where}kind {mlp.get('kind')!r}: a Pabalorn feed-forward is 'moe'")
    expert, router = _obj(mlp, "expert", where), _obj(mlp, "router", where)
    experts, top = _int(router, "experts", where + "router."), _int(router, "top", where + "router.")
    if top > experts:
        raise ConfigError(f"config.json: {where}router.top {top} exceeds router.experts {experts}")
    return RoutedExpertsSpec("routed_experts", width, _int(expert, "ff", where + "expert."), "silu", experts=experts,
                             top=top, router_bias=False, scoring="logistic", weight_on_input=True)


def read_spec(root: dict) -> ModelSpec:
    if root.get("architecture") != ARCHITECTURE:
        raise ConfigError(f"config.json: architecture {root.get('architecture')!r} is not {ARCHITECTURE}")
    width, vocab = _int(root, "width", ""), _int(root, "vocab", "")
    eps = _num(_obj(root, "norm", ""), "eps", "norm.")
    entries = root.get("layers")
    if not isinstance(entries, list) or not entries or len(entries) > MAX_LAYERS:
        raise ConfigError(f"config.json: 'layers' must list 1 to {MAX_LAYERS} layers")
    norm = NormSpec("rmsnorm", width, eps, unit_offset=True)

    mixers = []
    for i, entry in enumerate(entries):
        where = f"layers[{i}]."
        if not isinstance(entry, dict) or not isinstance(entry.get("type"), str):
            raise ConfigError(f"config.json: {where[:-1]} must be an object with a 'type'")
        m = _obj(entry, "mixer", where)
        if entry["type"] == "attention":
            mixers.append(_attention(m, width, where + "mixer.", "mix.", bias=False, rotary="rotary_half"))
        elif entry["type"] == "parallel":
            left = _attention(_obj(m, "left", where + "mixer."), width, where + "mixer.left.", "mix.left.", bias=True,
                              rotary="rotary_interleaved")
            if not left.own_kv:
                raise Unsupported(f"config.json: {where}mixer.left takes its keys and values from another layer")
            right = _scan(_obj(m, "right", where + "mixer."), width, where + "mixer.right.", "mix.right.")
            mixers.append(SideBySideSpec(kind="side_by_side", hidden_size=width, mixers=(left, right),
                                         out_norm_names=("mix.left.out", "mix.right.out"), out_norm_eps=eps))
        else:
            raise Unsupported(f"config.json: {where[:-1]} has type {entry['type']!r}; a Pabalorn layer is "
                              f"'attention' or 'parallel'")

    # a layer that takes its keys and values from layer j reads j's cache entry; the entry keeps the widest
    # window of its readers
    source = {}
    for i, entry in enumerate(entries):
        if entry["type"] == "attention" and "kv_from" in entry["mixer"]:
            j = entry["mixer"]["kv_from"]
            where = f"layers[{i}].mixer."
            if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
                raise ConfigError(f"config.json: {where}'kv_from' must name an earlier layer, got {j!r}")
            a, b = mixers[i], mixers[j]
            if not isinstance(b, RotatedAttentionSpec) or not b.own_kv:
                raise ConfigError(f"config.json: {where}kv_from {j}: that layer has no keys and values of its own")
            if (a.kv_heads, a.head_dim, a.v_head_dim, a.position) != (b.kv_heads, b.head_dim, b.v_head_dim, b.position):
                raise ConfigError(f"config.json: {where}kv_from {j}: key / value heads, sizes and rotation must equal "
                                  f"that layer's")
            source[i] = j
    for j in set(source.values()):
        windows = [mixers[j].window] + [mixers[i].window for i in source if source[i] == j]
        widest = None if any(w is None for w in windows) else max(windows)
        for i in [j] + [i for i in source if source[i] == j]:
            m = mixers[i]
            mixers[i] = RotatedAttentionSpec(**{**m.__dict__, "cache_window": widest})

    layers, run_order, entry_of, next_entry = [], [], {}, 0
    for i, entry in enumerate(entries):
        where = f"layers[{i}]."
        ff = _feed_forward(_obj(entry, "mlp", where), width, where + "mlp.") if entry.get("mlp") is not None else None
        layers.append(LayerSpec(block="parallel", mixer=mixers[i], feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=None, weight_prefix=f"l{i}.", mixer_norm_name="norm1"))
        if i in source:
            run_order.append(RunStep(i, entry_of[source[i]], writes_cache=False))
        elif isinstance(mixers[i], SideBySideSpec):
            n = len(mixers[i].mixers)
            run_order.append(RunStep(i, next_entry, True, more_caches=tuple(range(next_entry + 1, next_entry + n))))
            next_entry += n
        else:
            entry_of[i] = next_entry
            run_order.append(RunStep(i, next_entry, True))
            next_entry += 1
    return ModelSpec(architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab,
                     max_position_embeddings=MAX_POSITIONS, layers=tuple(layers), run_order=tuple(run_order),
                     final_norm=norm, tie_word_embeddings=True, eos_token_ids=(),
                     embed_name="embed", final_norm_name="final.norm", head_name="head",
                     embed_norm=norm, embed_norm_name="embed.norm")
