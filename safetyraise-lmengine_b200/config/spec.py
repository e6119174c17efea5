"""Typed specifications of a model: what the parts are built from.

A ``ModelSpec`` is a list of ``LayerSpec`` (each names its mixer, feed-forward
and norms by ``kind`` plus their sizes and constants) and a *run order*: the
list of steps a forward takes.  A step names the layer whose weights it uses
and the cache entry it writes or reads, so a layer may run twice, and a layer
may read the cache another layer wrote.  Nothing here knows an architecture:
readers such as ``config/qwen3.py`` fill these records from config.json keys.

Counterpart of ModelSpec/AttentionSpec/RopeSpec/LayerKind in the reference
(src/model/spec.rs:9-78), generalised so that every layer carries its own
part specifications.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    kind: str            # registry key in parts.NORMS
    size: int
    eps: float
    unit_offset: bool = False   # weight + 1 (not used by Qwen3: src/model/native.rs:534)


@dataclass(frozen=True)
class PositionSpec:
    kind: str            # registry key in parts.POSITION_ENCODINGS
    theta: float = 0.0   # the fields of a rotary encoding; another kind adds its own in a subclass
    rotary_dim: int = 0
    head_dim: int = 0
    # rescaled frequencies (factor, low, high, original): with wavelength l = 2 pi / f, f is kept where
    # l < original / high, divided by factor where l > original / low, and blended between the two with
    # s = (original / l - low) / (high - low): (1 - s) f / factor + s f.  None: the plain frequencies.
    scaling: Optional[Tuple[float, float, float, float]] = None
    # a ramp over the pair index (factor, original, fast, slow): with index(n) = rotary_dim ln(original / (2 pi n)) /
    # (2 ln theta), lo = max(floor(index(fast)), 0), hi = min(ceil(index(slow)), rotary_dim - 1) and r_i = clamp((i - lo) /
    # max(hi - lo, 0.001), 0, 1), pair i turns at f_i (1 - r_i) + f_i r_i / factor, and cos and sin are multiplied by
    # 0.1 ln(factor) + 1.  None: the plain frequencies and unit length.
    ramp: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class AttentionNames:
    """Tensor names of an attention mixer, each appended to its layer's ``weight_prefix``."""
    q: str = "self_attn.q_proj.weight"
    k: str = "self_attn.k_proj.weight"
    v: str = "self_attn.v_proj.weight"
    o: str = "self_attn.o_proj.weight"
    q_norm: str = "self_attn.q_norm.weight"
    k_norm: str = "self_attn.k_norm.weight"


@dataclass(frozen=True)
class GatedDenseNames:
    """Tensor names of a gated dense feed-forward, each appended to its layer's ``weight_prefix``."""
    gate: str = "mlp.gate_proj.weight"
    up: str = "mlp.up_proj.weight"
    down: str = "mlp.down_proj.weight"


@dataclass(frozen=True)
class MixerSpec:
    """Common header of every mixer specification."""
    kind: str            # registry key in parts.MIXERS


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    hidden_size: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    qk_norm: Optional[NormSpec] = None      # per-head norm of q and k before the position encoding
    position: Optional[PositionSpec] = None
    softmax_scale: float = 0.0
    window: Optional[int] = None            # None: every earlier key is visible
    bias: bool = False
    names: AttentionNames = AttentionNames()


@dataclass(frozen=True)
class SinkAttentionNames:
    """Tensor names of an attention mixer with biases, sinks and value mixing; a bias is its weight's name + ``bias_suffix``."""
    q: str = "mix.q"
    k: str = "mix.k"
    v: str = "mix.v"
    o: str = "mix.o"
    sink: str = "mix.sink"
    value_mix: str = "mix.vmix"
    bias_suffix: str = ".b"


@dataclass(frozen=True)
class SinkAttentionSpec(MixerSpec):
    """Grouped-query attention whose keys and values may differ in size, without a position encoding."""
    hidden_size: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0                       # query / key size
    v_head_dim: int = 0                     # value size
    softmax_scale: float = 0.0
    bias: bool = True                       # q, k and v projections carry biases
    sink: bool = True                       # one learned term per head in the softmax denominator
    value_mix: str = ""                     # "": values as projected; "keep": also kept for later layers;
                                            # "mix": (1 - lambda) v + lambda (the values a "keep" layer kept)
    window: Optional[int] = None
    names: SinkAttentionNames = SinkAttentionNames()


@dataclass(frozen=True)
class LatentAttentionNames:
    q: str = "mix.q"
    q_down: str = "mix.dq"                  # with q_rank: the queries' own latent, its norm, and the up projection
    q_norm: str = "mix.dq.norm"
    q_up: str = "mix.uq"
    down: str = "mix.dkv"                   # rows: the latent (kv_rank), then the shared rotated key part (rot_dim)
    latent_norm: str = "mix.dkv.norm"
    up_k: str = "mix.uk"
    up_v: str = "mix.uv"
    gate: str = "mix.g"
    o: str = "mix.o"


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Attention whose cache holds one normed latent and one rotated key part per token; per-head keys
    and values are up projections of the latent."""
    hidden_size: int = 0
    heads: int = 0
    head_dim: int = 0                       # unrotated query / key size per head
    rot_dim: int = 0                        # rotated query / key size per head (the key part is shared by the heads)
    v_head_dim: int = 0
    kv_rank: int = 0
    softmax_scale: float = 0.0
    position: Optional[PositionSpec] = None  # rotation of the rot_dim part (its first rotary_dim elements)
    latent_norm_eps: float = 1e-6
    output_gate: bool = True                # head outputs times sigmoid of a per-head projection of the input
    q_rank: int = 0                         # > 0: q = W_uq N(w, W_dq h), a latent of this size; 0: q = W_q h
    window: Optional[int] = None            # what a query sees (None: every earlier key)
    cache_window: Optional[int] = None      # what the cache keeps: the widest window of the steps that read the entry
    own_kv: bool = True                     # False: no down projection; it reads the latent and key part another step cached
    names: LatentAttentionNames = LatentAttentionNames()


@dataclass(frozen=True)
class DeltaRuleNames:
    q: str = "mix.q"
    k: str = "mix.k"
    v: str = "mix.v"
    conv_suffix: str = ".conv"              # the short convolution of a projection: its weight's name + this
    beta: str = "mix.b"
    decay: str = "mix.a"
    decay_log: str = "mix.A_log"
    decay_bias: str = "mix.dt_bias"
    out_norm: str = "mix.norm"
    gate: str = "mix.g"
    o: str = "mix.o"


@dataclass(frozen=True)
class DeltaRuleSpec(MixerSpec):
    """The gated delta rule: a matrix of state per head, written and read token by token."""
    hidden_size: int = 0
    heads: int = 0                          # value heads; q / k heads are shared by heads / kv_heads of them
    kv_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    conv_taps: int = 1
    norm_eps: float = 1e-6                  # of the per-head norm of the read-out
    unit_eps: float = 1e-6                  # inside the root that makes q and k unit vectors
    names: DeltaRuleNames = DeltaRuleNames()


@dataclass(frozen=True)
class DistanceAttentionNames:
    """Tensor names of an attention mixer with a distance penalty, each appended to its layer's ``weight_prefix``."""
    q: str = "mix.q"
    k: str = "mix.k"
    v: str = "mix.v"
    o: str = "mix.o"
    gate: str = "mix.g"                     # [heads, hidden]: one gate logit per head
    temperature: str = "mix.temp"           # [heads]
    penalty_weight: str = "mix.r1"          # [heads]
    penalty_rate: str = "mix.r2"            # [heads]


@dataclass(frozen=True)
class DistanceAttentionSpec(MixerSpec):
    """Grouped-query attention without a rotation, whose scores fall with the distance to the key:

        score(i, j) = (q_i . k_j) * softmax_scale * temperature_h - weight_h * ln(1 + rate_h * (i - j))

    over the keys 0 <= i - j < window (all earlier keys when window is None); q and k are divided by their
    root mean square per head when ``unit_norm_eps`` is given; a head's output is multiplied by the
    logistic of a per-head projection of the mixer's input when ``output_gate`` is set."""
    hidden_size: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0                       # query / key size
    v_head_dim: int = 0                     # value size
    softmax_scale: float = 0.0
    window: Optional[int] = None
    unit_norm_eps: Optional[float] = None   # None: q and k as projected
    temperature: bool = True                # a learned factor per head on the scores
    distance_penalty: bool = True           # the logarithmic penalty above, two learned numbers per head
    output_gate: bool = True
    names: DistanceAttentionNames = DistanceAttentionNames()


@dataclass(frozen=True)
class RotatedAttentionNames:
    """Tensor names of a rotated attention mixer, each appended to its layer's ``weight_prefix``; a bias is its
    weight's name + ``bias_suffix``."""
    q: str = "mix.q"
    k: str = "mix.k"
    v: str = "mix.v"
    o: str = "mix.o"
    bias_suffix: str = ".b"


@dataclass(frozen=True)
class RotatedAttentionSpec(MixerSpec):
    """Grouped-query attention whose keys and values may differ in size, with a rotary encoding on the leading
    part of q and k, optional biases on q, k and v, an optional cap on the scores and an optional window:

        score(i, j) = cap((q_i . k_j) * softmax_scale),  cap(s) = softcap * tanh(s / softcap),  0 <= i - j < window

    ``own_kv`` False: the mixer has no key and value projections; it attends over the keys (as cached, rotated)
    and values of the run step whose cache entry its own run step reads."""
    hidden_size: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0                       # query / key size
    v_head_dim: int = 0                     # value size
    softmax_scale: float = 0.0
    position: Optional[PositionSpec] = None
    softcap: Optional[float] = None
    window: Optional[int] = None            # what a query sees
    cache_window: Optional[int] = None      # what the cache keeps: the widest window of the steps that read the entry
    bias: bool = False
    own_kv: bool = True
    names: RotatedAttentionNames = RotatedAttentionNames()


@dataclass(frozen=True)
class SelectiveScanNames:
    inp: str = "mix.in"                     # [2 inner, hidden]: x rows, then z rows
    conv: str = "mix.conv"                  # [inner, taps]; its bias: this name + ".b"
    x: str = "mix.x"                        # [dt_rank + 2 state, inner]: dt, B, C rows
    dt: str = "mix.dt"                      # [inner, dt_rank]; its bias: this name + ".b"
    a_log: str = "mix.A_log"                # [inner, state]
    d: str = "mix.D"                        # [inner]
    o: str = "mix.o"                        # [hidden, inner]


@dataclass(frozen=True)
class SelectiveScanSpec(MixerSpec):
    """The selective scan: per channel c of ``inner`` and state n of ``state``,
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c;  out = W_o (y * silu(z)),
    x behind a short causal convolution and SiLU, dt = softplus(W_dt (low-rank part) + bias), A = -exp(A_log)."""
    hidden_size: int = 0
    inner: int = 0
    state: int = 0
    dt_rank: int = 0
    conv_taps: int = 1
    names: SelectiveScanNames = SelectiveScanNames()


@dataclass(frozen=True)
class ConvAttentionNames:
    """Tensor names of an attention behind short convolutions, each appended to its layer's ``weight_prefix``; the
    convolution of a projection is its weight's name + ``conv_suffix``, the per-head norm's weight + ``norm_suffix``."""
    q: str = "mix.q"
    k: str = "mix.k"
    v: str = "mix.v"
    o: str = "mix.o"
    conv_suffix: str = ".conv"
    norm_suffix: str = ".norm"


@dataclass(frozen=True)
class ConvAttentionSpec(MixerSpec):
    """Grouped-query attention whose q, k and v each pass a short causal convolution over time (per channel, no bias)
    right behind their projection; then a per-head RMS norm of q and k (one weight of head_dim for all heads), the
    rotary encoding, and

        p_ij = exp(s_ij) / (sink + sum_j' exp(s_ij')),   s_ij = (q_i . k_j) * softmax_scale,   0 <= i - j < window

    with sink = 1 when ``unit_sink`` (one more key of score 0 and no value) and 0 otherwise.  The last conv_taps - 1
    projected rows of a request are part of its state."""
    hidden_size: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    softmax_scale: float = 0.0
    conv_taps: int = 1
    qk_norm_eps: Optional[float] = None     # None: q and k as convolved
    position: Optional[PositionSpec] = None
    unit_sink: bool = False
    window: Optional[int] = None
    names: ConvAttentionNames = ConvAttentionNames()


@dataclass(frozen=True)
class MatrixMemoryNames:
    q: str = "mix.q"
    k: str = "mix.k"
    v: str = "mix.v"
    gate: str = "mix.g"                     # [heads * v_head_dim, hidden]: the output gate
    write: str = "mix.i"                    # [heads, hidden] and a bias (name + ".b"): the logarithm of the input gate
    forget: str = "mix.f"                   # likewise: the forget gate ahead of its log-logistic
    out_norm: str = "mix.norm"              # [heads * v_head_dim]
    o: str = "mix.o"


@dataclass(frozen=True)
class MatrixMemorySpec(MixerSpec):
    """A matrix of state S [head_dim, v_head_dim] and a vector n [head_dim] per head, with a running maximum m of the
    gates' logarithms (m, S, n start at 0):  i = cap tanh((W_i h + b_i) / cap),  f = log logistic(cap tanh((W_f h + b_f) / cap)),

        m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;  n likewise with k;
        o = S^T q / (max(|n . q|, exp(-m')) + denominator_floor),   q = W_q h / sqrt(head_dim)

    then each head's o over its root mean square, times a weight over all heads, times logistic(W_g h), then W_o."""
    hidden_size: int = 0
    heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    gate_cap: float = 0.0
    norm_eps: float = 1e-6
    denominator_floor: float = 1e-6
    names: MatrixMemoryNames = MatrixMemoryNames()


@dataclass(frozen=True)
class GatedRecurrenceNames:
    gate_branch: str = "mix.y"              # [width, hidden] and a bias (name + ".b")
    recurrent_branch: str = "mix.x"         # likewise
    conv: str = "mix.conv"                  # [width, taps] and a bias (name + ".b")
    decay_gate: str = "mix.ra"              # [blocks, width / blocks, width / blocks] ([out, in]) and a bias [blocks, width / blocks]
    input_gate: str = "mix.ri"              # likewise
    decay: str = "mix.lam"                  # [width]
    o: str = "mix.o"


@dataclass(frozen=True)
class GatedRecurrenceSpec(MixerSpec):
    """A linear recurrence per channel with gates from block-diagonal products of its own input:

        y = gelu_tanh(W_y h + b_y);   u = conv(W_x h + b_x) + b_conv      (a short causal convolution per channel)
        r = logistic(R_a u + b_a);  i = logistic(R_i u + b_i)             (R block-diagonal, ``blocks`` square blocks)
        a = exp(-decay_scale r softplus(lam));   S <- a S + sqrt(1 - a^2) i u;   out = W_o (S y)

    S starts at zero, also for a request's first token.  S and the convolution's last taps - 1 inputs are the state."""
    hidden_size: int = 0
    width: int = 0
    blocks: int = 1
    conv_taps: int = 1
    decay_scale: float = 8.0
    names: GatedRecurrenceNames = GatedRecurrenceNames()


@dataclass(frozen=True)
class SideBySideSpec(MixerSpec):
    """Several mixers that read the same input; the result is the mean of their outputs, each first RMS-normed
    over the model width with a weight of its own (``out_norm_names``, appended to the layer's prefix)."""
    hidden_size: int = 0
    mixers: Tuple[MixerSpec, ...] = ()
    out_norm_names: Tuple[str, ...] = ()
    out_norm_eps: float = 1e-6
    # "normed_mean": as above.  "weighted_sum": sum_k weights[k] * mixer_k(h), nothing normed (no out_norm_names).
    combine: str = "normed_mean"
    weights: Tuple[float, ...] = ()


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str            # registry key in parts.FEED_FORWARDS
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    names: GatedDenseNames = GatedDenseNames()   # read by the gated dense part; other kinds name their own


@dataclass(frozen=True)
class DenseNames:
    up: str = "mlp.up"
    down: str = "mlp.down"


@dataclass(frozen=True)
class DenseSpec(FeedForwardSpec):
    """down(act(up(x))): no gate.  ``activation``: "gelu" (the exact one, with erf)."""
    dense_names: DenseNames = DenseNames()


@dataclass(frozen=True)
class RoutedExpertsNames:
    """Tensor names of a routed feed-forward; expert e's tensors start with ``expert.format(e)``."""
    router: str = "mlp.router"
    router_bias: str = "mlp.router.b"
    expert: str = "mlp.e{}."
    shared: str = "mlp.shared."
    gate: str = "gate"
    up: str = "up"
    down: str = "down"


@dataclass(frozen=True)
class RoutedExpertsSpec(FeedForwardSpec):
    """``experts`` small gated feed-forwards of which every token uses the ``top`` with the largest router
    logits, weighted by the softmax over those logits alone; plus, optionally, one that every token uses.
    ``activation`` "clamped_glu": y = g * logistic(glu_alpha * g) * (u + 1) with g = min(gate, limit),
    u = clamp(up, -limit, limit).  intermediate_size is one expert's."""
    experts: int = 0
    top: int = 0
    limit: float = 0.0
    glu_alpha: float = 1.702
    router_bias: bool = True
    shared_size: int = 0                    # 0: no expert that every token uses
    shared_limit: float = 0.0
    # "softmax_of_chosen": weights = softmax over the chosen logits; "logistic": the logistic of each chosen
    # logit, not renormalised.  activation "silu": y = gate * logistic(gate) * up, no clamp (limit unused).
    # "softmax_over_all": scores = softmax over every expert's logit; the experts form ``groups`` equal groups of
    # neighbours, a group counts as its largest score, only experts of the best ``groups_kept`` groups can be chosen;
    # weights = the chosen scores over their sum (+ 1e-20).
    scoring: str = "softmax_of_chosen"
    weight_on_input: bool = False           # a weight multiplies its expert's input instead of its output
    groups: int = 1
    groups_kept: int = 1
    gated: bool = True                      # False: an expert is W_down act(W_up h) (activation "gelu"), and so is the shared one
    expert_names: RoutedExpertsNames = RoutedExpertsNames()


@dataclass(frozen=True)
class LayerSpec:
    block: str                               # registry key in parts.BLOCKS
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]  # None: a layer of a mixer alone (blocks that allow it)
    mixer_norm: NormSpec
    feed_forward_norm: Optional[NormSpec]
    weight_prefix: str                       # e.g. "model.layers.3."
    mixer_norm_name: str = "input_layernorm.weight"              # appended to weight_prefix
    feed_forward_norm_name: str = "post_attention_layernorm.weight"
    # blocks that also norm a sublayer's result and gate it before it joins the residual stream:
    mixer_post_norm: Optional[NormSpec] = None
    feed_forward_post_norm: Optional[NormSpec] = None
    mixer_post_norm_name: str = "norm1b"
    feed_forward_post_norm_name: str = "norm2b"
    mixer_gate_name: str = "rg1"             # weight [hidden, hidden]; its bias: this name + ".b"
    feed_forward_gate_name: str = "rg2"
    residual_scale: float = 1.0              # block "post_norm": x <- norm(residual_scale * x + sublayer(x))


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order."""
    layer: int                 # index into ModelSpec.layers: whose weights run
    cache: int                 # cache entry (per-step key/value or state storage) it uses
    writes_cache: bool = True  # False: reads what another step wrote under ``cache``
    more_caches: Tuple[int, ...] = ()   # a mixer made of several (side by side): the entries of the second, third, ...


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position_embeddings: int
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunStep, ...]
    final_norm: NormSpec
    tie_word_embeddings: bool
    eos_token_ids: Tuple[int, ...] = ()
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    embed_position: Optional[PositionSpec] = None   # an encoding that adds to the embedded tokens (none in Qwen3)
    embed_position_name: str = "model.embed_positions.weight"
    embed_norm: Optional[NormSpec] = None           # a norm of the embedded tokens before the first layer
    embed_norm_name: str = "embed.norm"
    logit_softcap: Optional[float] = None           # logits <- cap * tanh(logits / cap)
    extra: dict = field(default_factory=dict, compare=False)

    def to_json(self) -> dict:
        return asdict(self)

    @property
    def num_cache_entries(self) -> int:
        return 1 + max(max((s.cache,) + s.more_caches) for s in self.run_order) if self.run_order else 0
