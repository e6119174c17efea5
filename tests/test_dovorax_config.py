"""The Dovorax config reader: keys, run order, declared tensors, cache needs, refusals; the plain implementation's
mechanisms on inputs whose answer is known.  No GPU."""
import copy
import math

import pytest
import torch

import plain_dovorax as P
from safetyraise_lmengine_b200 import spec_from_config
from safetyraise_lmengine_b200.errors import ConfigError, Unsupported
from safetyraise_lmengine_b200.parts.model import cache_groups_of, tensor_decls
from safetyraise_lmengine_b200.parts.position import ramped_frequencies

ROT = {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}


def latent(window=20, **more):
    m = {"heads": 4, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 32, "q_rank": 20, "scale": 0.3, "mask": {"size": window},
         "rot": ROT}
    m.update(more)
    return m


MOE = {"kind": "moe", "expert": {"ff": 24}, "shared": {"ff": 40},
       "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}
LEFT = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "conv": 4, "scale": 0.35, "rot": {"dims": 4, "base": 100.0}}
RIGHT = {"heads": 2, "dim": 12, "vdim": 20, "gate_cap": 6.0}
CFG = {"architecture": "Dovorax", "width": 48, "vocab": 100, "norm": {"eps": 1e-5}, "postln_alpha": 2.0,
       "layers": [{"type": "latent_attention", "mixer": latent(), "mlp": {"kind": "dense", "ff": 64}},
                  {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT, "left_scale": 0.8, "right_scale": 0.5}, "mlp": MOE},
                  {"type": "rglru", "mixer": {"width": 36, "blocks": 3, "conv": 3}, "mlp": None},
                  {"type": "latent_attention", "mixer": latent(window=33, kv_from=0, heads=2, q_rank=9), "mlp": MOE}]}


def test_layers_run_order_and_constants():
    spec = spec_from_config(CFG)
    assert spec.architecture == "Dovorax" and spec.hidden_size == 48 and spec.vocab_size == 100
    assert spec.tie_word_embeddings and spec.embed_norm is None and spec.final_norm.unit_offset and spec.final_norm.eps == 1e-5
    assert all(l.block == "post_norm" and l.residual_scale == 2.0 and l.mixer_norm.unit_offset for l in spec.layers)
    # the pair keeps pages, carried rows and a memory; the layer without a down projection reads layer 0's entry
    assert [(s.layer, s.cache, s.more_caches, s.writes_cache) for s in spec.run_order] == \
        [(0, 0, (), True), (1, 1, (2, 3), True), (2, 4, (), True), (3, 0, (), False)]
    a, b = spec.layers[0].mixer, spec.layers[3].mixer
    assert (a.kind, a.heads, a.head_dim, a.rot_dim, a.v_head_dim, a.kv_rank, a.q_rank, a.window, a.softmax_scale) == \
        ("latent_attention", 4, 16, 8, 24, 32, 20, 20, 0.3)
    assert a.own_kv and not b.own_kv and not a.output_gate and b.heads == 2 and b.q_rank == 9
    assert a.cache_window == b.cache_window == 33 and b.window == 33 and a.latent_norm_eps == 1e-5
    assert (a.position.kind, a.position.rotary_dim, a.position.theta, a.position.ramp) == ("rotary_half", 8, 10000.0, (4.0, 64.0, 8.0, 1.0))
    pair = spec.layers[1].mixer
    left, right = pair.mixers
    assert (pair.kind, pair.combine, pair.weights, pair.out_norm_names) == ("side_by_side", "weighted_sum", (0.8, 0.5), ())
    assert (left.kind, left.heads, left.kv_heads, left.head_dim, left.v_head_dim, left.conv_taps, left.unit_sink, left.window,
            left.qk_norm_eps) == ("conv_attention", 4, 2, 16, 8, 4, True, None, 1e-5)
    assert left.position.rotary_dim == 4 and left.position.ramp is None
    assert (right.kind, right.heads, right.head_dim, right.v_head_dim, right.gate_cap, right.norm_eps) == \
        ("matrix_memory", 2, 12, 20, 6.0, 1e-5)
    r = spec.layers[2].mixer
    assert (r.kind, r.width, r.blocks, r.conv_taps, r.decay_scale) == ("gated_linear_recurrence", 36, 3, 3, 8.0)
    d, ff = spec.layers[0].feed_forward, spec.layers[1].feed_forward
    assert (d.kind, d.intermediate_size, d.activation) == ("dense", 64, "gelu")
    assert (ff.kind, ff.experts, ff.top, ff.intermediate_size, ff.activation, ff.scoring, ff.groups, ff.groups_kept, ff.gated,
            ff.shared_size, ff.router_bias, ff.weight_on_input) == \
        ("routed_experts", 6, 2, 24, "gelu", "softmax_over_all", 3, 2, False, 40, False, False)
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None


def test_declared_tensors():
    names = {d.name: tuple(d.shape) for d in tensor_decls(spec_from_config(CFG))}
    assert names["embed"] == (100, 48) and names["final.norm"] == (48,) and "head" not in names and "embed.norm" not in names
    assert names["l0.norm1"] == names["l0.norm2"] == (48,) and "l2.norm2" not in names
    assert names["l0.mix.dq"] == (20, 48) and names["l0.mix.dq.norm"] == (20,) and names["l0.mix.uq"] == (96, 20)
    assert names["l0.mix.dkv"] == (40, 48) and names["l0.mix.dkv.norm"] == (32,)
    assert names["l0.mix.uk"] == (64, 32) and names["l0.mix.uv"] == (96, 32) and names["l0.mix.o"] == (48, 96)
    assert "l3.mix.dkv" not in names and "l3.mix.dkv.norm" not in names and names["l3.mix.uq"] == (48, 9)
    assert names["l3.mix.uk"] == (32, 32) and names["l3.mix.o"] == (48, 48)
    assert names["l0.mlp.up"] == (64, 48) and names["l0.mlp.down"] == (48, 64)
    assert names["l1.mix.left.q"] == (64, 48) and names["l1.mix.left.k"] == (32, 48) and names["l1.mix.left.v"] == (16, 48)
    assert names["l1.mix.left.q.conv"] == (64, 4) and names["l1.mix.left.v.conv"] == (16, 4)
    assert names["l1.mix.left.q.norm"] == names["l1.mix.left.k.norm"] == (16,) and names["l1.mix.left.o"] == (48, 32)
    assert names["l1.mix.right.q"] == names["l1.mix.right.k"] == (24, 48)
    assert names["l1.mix.right.v"] == names["l1.mix.right.g"] == (40, 48) and names["l1.mix.right.norm"] == (40,)
    assert names["l1.mix.right.i"] == names["l1.mix.right.f"] == (2, 48) and names["l1.mix.right.i.b"] == names["l1.mix.right.f.b"] == (2,)
    assert names["l1.mix.right.o"] == (48, 40)
    assert names["l2.mix.y"] == names["l2.mix.x"] == (36, 48) and names["l2.mix.y.b"] == names["l2.mix.conv.b"] == (36,)
    assert names["l2.mix.conv"] == (36, 3) and names["l2.mix.ra"] == names["l2.mix.ri"] == (3, 12, 12)
    assert names["l2.mix.ra.b"] == (3, 12) and names["l2.mix.lam"] == (36,) and names["l2.mix.o"] == (48, 36)
    assert names["l1.mlp.e5.up"] == (24, 48) and names["l3.mlp.e0.down"] == (48, 24) and "l1.mlp.e6.up" not in names
    assert "l1.mlp.e0.gate" not in names and "l1.mlp.shared.gate" not in names
    assert names["l1.mlp.router"] == (6, 48) and names["l1.mlp.shared.up"] == (40, 48) and names["l1.mlp.shared.down"] == (48, 40)
    assert not any("l2.mlp" in n for n in names)


def test_cache_groups_follow_windows_sizes_and_states():
    groups = cache_groups_of(spec_from_config(CFG))
    by = {(g.kind, g.window, g.kv_heads, g.head_dim, g.v_head_dim, tuple(g.state_shape)): g.entries for g in groups}
    assert by[("paged_window", 33, 1, 40, 0, ())] == (0,)                        # the latent and the key part; the widest reader
    assert by[("paged_all", None, 2, 16, 8, ())] == (1,)                         # the attention behind convolutions sees everything
    assert by[("fixed_state", None, 0, 0, None, (3 * (64 + 32 + 16),))] == (2,)  # its carried rows
    assert by[("fixed_state", None, 0, 0, None, (2 * 12 * 20 + 2 * 12 + 2,))] == (3,)
    assert by[("fixed_state", None, 0, 0, None, (36 * 3,))] == (4,)
    one_tap = copy.deepcopy(CFG)
    one_tap["layers"][1]["mixer"]["left"]["conv"] = 1
    spec = spec_from_config(one_tap)
    assert spec.run_order[1].more_caches == (2,) and len(cache_groups_of(spec)) == 4      # nothing to carry
    assert ("l1.mix.left.q.conv", (64, 1)) in {(d.name, tuple(d.shape)) for d in tensor_decls(spec)}


@pytest.mark.parametrize("change,error", [
    (lambda c: c.update(architecture="Other"), Unsupported),
    (lambda c: c.pop("postln_alpha"), ConfigError),
    (lambda c: c["norm"].pop("eps"), ConfigError),
    (lambda c: c["layers"][0].update(type="attention"), Unsupported),
    (lambda c: c["layers"][0]["mixer"].pop("q_rank"), ConfigError),
    (lambda c: c["layers"][0]["mixer"].update(rot_dim=6), ConfigError),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), ConfigError),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), ConfigError),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=16), ConfigError),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), ConfigError),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), ConfigError),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("gate_cap"), ConfigError),
    (lambda c: c["layers"][2]["mixer"].update(blocks=5), ConfigError),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), Unsupported),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), ConfigError),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), ConfigError),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=4), ConfigError),
])
def test_refusals(change, error):
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(error):
        spec_from_config(cfg)


def test_ramped_frequencies_by_hand():
    # dims 8, base 10^4, original 64: index(n) = 8 ln(64 / (2 pi n)) / (2 ln 10^4): index(8) = 0.105 -> lo 0, index(1) = 1.008 -> hi 2
    f, length = ramped_frequencies(10000.0, 8, (4.0, 64.0, 8.0, 1.0))
    plain = [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    assert f[0] == plain[0] and math.isclose(f[1], plain[1] * (0.5 + 0.5 / 4)) and math.isclose(f[2], plain[2] / 4)
    assert math.isclose(f[3], plain[3] / 4) and math.isclose(length, 0.1 * math.log(4.0) + 1.0)
    pf, pl = P.rotary({"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    assert torch.allclose(pf, torch.tensor(f, dtype=torch.float64)) and pl == length
    # a ramp of no width (lo = hi = 0): pair 0 keeps its frequency, every pair behind it is divided
    f, _ = ramped_frequencies(100.0, 4, (2.0, 1000.0, 1000.0, 999.0))
    assert f == [1.0, 0.1 / 2.0]


def test_plain_mechanisms_on_known_inputs():
    # one more term in the denominator: scores of 0 over two keys weigh 1/3 each
    s = torch.zeros(1, 2, 2, dtype=torch.float64)
    a = P.softmax_rows(s, P.visible(2, None), one_more=True)
    assert torch.allclose(a[0], torch.tensor([[0.5, 0.0], [1 / 3, 1 / 3]], dtype=torch.float64))
    # the window: a query sees itself and window - 1 keys before it
    assert P.visible(4, 2).tolist() == [[True, False, False, False], [True, True, False, False], [False, True, True, False],
                                         [False, False, True, True]]
    # the convolution: the last column is the current token's
    y = P.short_conv(torch.tensor([[1.0], [2.0], [3.0]]), torch.tensor([[100.0, 10.0, 1.0]]))
    assert y.flatten().tolist() == [1.0, 12.0, 123.0]
    # the router: the best group wins even when a losing group holds the second best expert
    z = torch.tensor([[5.0, 0.0, 4.9, 4.8, 0.1, 0.2]])
    chosen, w = P.route(z, {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert chosen.tolist() == [[0, 1]] and math.isclose(float(w.sum()), 1.0)
    chosen, _ = P.route(z, {"experts": 6, "top": 2})
    assert chosen.tolist() == [[0, 2]]
    # the memory's first token: m = max(f, i) from m = 0, not from minus infinity
    W = {"p.q": torch.eye(2), "p.k": torch.eye(2), "p.v": torch.eye(2), "p.g": torch.zeros(2, 2), "p.o": torch.eye(2),
         "p.i": torch.zeros(1, 2), "p.f": torch.zeros(1, 2), "p.i.b": torch.tensor([-3.0]), "p.f.b": torch.tensor([0.0]),
         "p.norm": torch.ones(2)}
    h = torch.tensor([[1.0, 2.0]])
    out = P.matrix_memory(h, W, "p.", {"heads": 1, "dim": 2, "vdim": 2, "gate_cap": 10.0}, 1e-6)
    gi, gf = 10 * math.tanh(-0.3), -math.log(2.0)
    m = max(gf, gi)
    write = math.exp(gi - m)
    nq = write * 5.0 / math.sqrt(2.0)
    o = torch.tensor([1.0, 2.0]) * write * 5.0 / math.sqrt(2.0) / (max(nq, math.exp(-m)) + 1e-6)
    want = o / torch.sqrt((o * o).mean() + 1e-6) * 0.5
    assert torch.allclose(out[0], want.double(), atol=1e-9)
