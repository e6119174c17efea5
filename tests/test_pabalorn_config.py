"""The Pabalorn config reader: keys, run order, declared tensors, cache needs, refusals; the plain
implementation's mechanisms on inputs whose answer is known.  No GPU."""
import copy
import math

import pytest
import torch

import plain_pabalorn as P
from safetyraise_lmengine_b200 import spec_from_config
from safetyraise_lmengine_b200.errors import ConfigError, Unsupported
from safetyraise_lmengine_b200.parts.model import cache_groups_of, tensor_decls
from safetyraise_lmengine_b200.parts.position import rescaled_frequencies


def att(heads=4, kv=2, dim=16, vdim=24, window=20, softcap=30.0, rot=8, **more):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": 0.3, "mask": {"size": window},
         "softcap": softcap, "rot": {"dims": rot, "base": 10000.0}}
    m.update(more)
    return m


MOE = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}
LEFT = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.35, "mask": {"size": 9},
        "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}}
RIGHT = {"inner": 40, "state": 6, "dt_rank": 3, "conv": 4}
CFG = {"architecture": "Pabalorn", "width": 48, "vocab": 100, "norm": {"eps": 1e-5},
       "layers": [{"type": "attention", "mixer": att(), "mlp": MOE},
                  {"type": "parallel", "mixer": {"left": LEFT, "right": RIGHT}, "mlp": None},
                  {"type": "attention", "mixer": att(window=33, kv_from=0), "mlp": MOE},
                  {"type": "attention", "mixer": att(heads=2, kv=2, dim=8, vdim=8, window=7), "mlp": None}]}


def test_layers_run_order_and_constants():
    spec = spec_from_config(CFG)
    assert spec.architecture == "Pabalorn" and spec.hidden_size == 48 and spec.vocab_size == 100
    assert spec.tie_word_embeddings and spec.logit_softcap is None
    assert spec.embed_norm.eps == 1e-5 and spec.embed_norm.unit_offset and spec.final_norm.unit_offset
    assert all(l.block == "parallel" and l.feed_forward_norm is None for l in spec.layers)
    # the pair of mixers has an entry each; the layer without keys and values reads layer 0's
    assert [(s.layer, s.cache, s.more_caches, s.writes_cache) for s in spec.run_order] == \
        [(0, 0, (), True), (1, 1, (2,), True), (2, 0, (), False), (3, 3, (), True)]
    a, b = spec.layers[0].mixer, spec.layers[2].mixer
    assert (a.kind, a.heads, a.kv_heads, a.head_dim, a.v_head_dim, a.window, a.softcap, a.softmax_scale) == \
        ("rotated_attention", 4, 2, 16, 24, 20, 30.0, 0.3)
    assert a.own_kv and not b.own_kv and not a.bias
    assert a.cache_window == b.cache_window == 33 and b.window == 33       # the entry keeps its widest reader's keys
    assert (a.position.kind, a.position.rotary_dim, a.position.theta, a.position.scaling) == ("rotary_half", 8, 10000.0, None)
    pair = spec.layers[1].mixer
    left, right = pair.mixers
    assert pair.kind == "side_by_side" and pair.out_norm_names == ("mix.left.out", "mix.right.out") and pair.out_norm_eps == 1e-5
    assert left.bias and left.softcap is None and left.window == 9 and left.position.kind == "rotary_interleaved"
    assert left.position.scaling == (8.0, 1.0, 4.0, 64.0) and left.position.rotary_dim == 4
    assert (right.kind, right.inner, right.state, right.dt_rank, right.conv_taps) == ("selective_scan", 40, 6, 3, 4)
    ff = spec.layers[0].feed_forward
    assert (ff.kind, ff.experts, ff.top, ff.intermediate_size, ff.activation, ff.scoring, ff.weight_on_input,
            ff.shared_size, ff.router_bias) == ("routed_experts", 5, 2, 24, "silu", "logistic", True, 0, False)
    assert spec.layers[1].feed_forward is None and spec.layers[3].feed_forward is None


def test_declared_tensors():
    names = {d.name: tuple(d.shape) for d in tensor_decls(spec_from_config(CFG))}
    assert names["embed"] == (100, 48) and names["embed.norm"] == (48,) and names["final.norm"] == (48,)
    assert "head" not in names and not any(".norm2" in n for n in names)
    assert names["l0.mix.q"] == (64, 48) and names["l0.mix.k"] == (32, 48) and names["l0.mix.v"] == (48, 48)
    assert names["l0.mix.o"] == (48, 96) and "l0.mix.q.b" not in names
    assert "l2.mix.k" not in names and "l2.mix.v" not in names and names["l2.mix.q"] == (64, 48)
    assert names["l1.mix.left.q"] == (16, 48) and names["l1.mix.left.k.b"] == (8,) and names["l1.mix.left.v.b"] == (8,)
    assert names["l1.mix.left.out"] == names["l1.mix.right.out"] == (48,)
    assert names["l1.mix.right.in"] == (80, 48) and names["l1.mix.right.conv"] == (40, 4)
    assert names["l1.mix.right.conv.b"] == names["l1.mix.right.dt.b"] == names["l1.mix.right.D"] == (40,)
    assert names["l1.mix.right.x"] == (15, 40) and names["l1.mix.right.dt"] == (40, 3)
    assert names["l1.mix.right.A_log"] == (40, 6) and names["l1.mix.right.o"] == (48, 40)
    assert names["l0.mlp.e4.gate"] == (24, 48) and names["l2.mlp.e0.down"] == (48, 24) and "l0.mlp.e5.up" not in names
    assert names["l0.mlp.router"] == (5, 48) and "l0.mlp.router.b" not in names and not any("l1.mlp" in n for n in names)


def test_cache_groups_follow_windows_sizes_and_states():
    groups = cache_groups_of(spec_from_config(CFG))
    by = {(g.kind, g.window, g.kv_heads, g.head_dim, g.v_head_dim, tuple(g.state_shape)): g.entries for g in groups}
    assert by == {("paged_window", 33, 2, 16, 24, ()): (0,), ("paged_window", 9, 1, 8, None, ()): (1,),
                  ("fixed_state", None, 0, 0, None, (40 * (6 + 3),)): (2,), ("paged_window", 7, 2, 8, None, ()): (3,)}


def test_a_model_without_windows_caps_rotation_or_experts():
    cfg = copy.deepcopy(CFG)
    for key in ("mask", "softcap", "rot"):
        del cfg["layers"][3]["mixer"][key]
    del cfg["layers"][1]["mixer"]["left"]["mask"]
    del cfg["layers"][1]["mixer"]["left"]["rot"]["scaling"]
    spec = spec_from_config(cfg)
    a, left = spec.layers[3].mixer, spec.layers[1].mixer.mixers[0]
    assert a.window is None and a.cache_window is None and a.softcap is None and a.position is None
    assert left.window is None and left.position.scaling is None
    kinds = {g.entries: g.kind for g in cache_groups_of(spec)}
    assert kinds[(1,)] == "paged_all" and kinds[(3,)] == "paged_all"


@pytest.mark.parametrize("change,error", [
    (lambda c: c.update(width=0), ConfigError),
    (lambda c: c["norm"].pop("eps"), ConfigError),
    (lambda c: c["layers"][0].update(type="convolution"), Unsupported),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), ConfigError),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), Unsupported),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), ConfigError),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), ConfigError),             # not an earlier layer
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), ConfigError),             # a pair of mixers has no such keys
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=1), ConfigError),            # heads must equal the owner's
    (lambda c: c["layers"][2]["mixer"]["rot"].update(base=500.0), ConfigError),     # so must the rotation
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_from=0), Unsupported),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("state"), ConfigError),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"]["scaling"].update(high=1.0), ConfigError),
])
def test_refusals(change, error):
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(error):
        spec_from_config(cfg)


def test_a_reader_of_a_reader_is_refused_and_two_readers_share_an_entry():
    cfg = copy.deepcopy(CFG)
    cfg["layers"].append({"type": "attention", "mixer": att(window=5, kv_from=0), "mlp": None})
    spec = spec_from_config(cfg)
    assert [s.cache for s in spec.run_order] == [0, 1, 0, 3, 0] and not spec.run_order[4].writes_cache
    assert [spec.layers[i].mixer.cache_window for i in (0, 2, 4)] == [33, 33, 33]
    assert [spec.layers[i].mixer.window for i in (0, 2, 4)] == [20, 33, 5]
    cfg["layers"][4]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError):
        spec_from_config(cfg)


def test_rescaled_frequencies_against_the_rule_and_the_plain_implementation():
    rot = {"dims": 16, "base": 50.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}}
    got = rescaled_frequencies(50.0, 16, (4.0, 1.0, 4.0, 40.0))
    plain = P.rotary_frequencies(rot).tolist()
    assert got == pytest.approx(plain, rel=1e-14)
    kinds = set()
    for i, f in enumerate(got):
        base = 50.0 ** (-2.0 * i / 16)
        wave = 2 * math.pi / base
        if wave < 10:
            kinds.add("kept")
            assert f == base
        elif wave > 40:
            kinds.add("divided")
            assert f == pytest.approx(base / 4)
        else:
            kinds.add("blended")
            assert base / 4 < f < base
    assert kinds == {"kept", "divided", "blended"}               # the example has waves of all three kinds
    assert rescaled_frequencies(50.0, 16, None) == [50.0 ** (-2.0 * i / 16) for i in range(8)]


def test_plain_rotation_pairs_and_the_untouched_tail():
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0                    # element 0: paired with 1 when interleaved, with 2 otherwise (dims 4)
    x[:, 0, 5] = 7.0
    rot = {"dims": 4, "base": 10000.0}
    inter, half = P.rotate(x, rot, True), P.rotate(x, rot, False)
    for p in range(3):
        assert inter[p, 0, 0] == pytest.approx(math.cos(p)) and inter[p, 0, 1] == pytest.approx(math.sin(p))
        assert half[p, 0, 0] == pytest.approx(math.cos(p)) and half[p, 0, 2] == pytest.approx(math.sin(p))
        assert inter[p, 0, 2] == 0 and half[p, 0, 1] == 0 and inter[p, 0, 5] == half[p, 0, 5] == 7.0


def test_plain_scan_of_one_channel_by_hand():
    """One channel, one state, no convolution history: S_t = exp(dt A) S_{t-1} + dt x_t B_t by hand."""
    W = {"in": torch.tensor([[1.0], [0.0]]), "conv": torch.tensor([[0.0, 1.0]]), "conv.b": torch.tensor([0.0]),
         "x": torch.tensor([[0.0], [1.0], [1.0]]), "dt": torch.tensor([[0.0]]), "dt.b": torch.tensor([0.3]),
         "A_log": torch.tensor([[0.5]]), "D": torch.tensor([2.0]), "o": torch.tensor([[1.0]])}
    h = torch.tensor([[1.0], [-0.5], [2.0]], dtype=torch.float64)
    got = P.selective_scan(h, W, "", {"inner": 1, "state": 1, "dt_rank": 1})
    dt, A = math.log1p(math.exp(0.3)), -math.exp(0.5)
    S, want = 0.0, []
    for t in range(3):
        x = float(h[t]) / (1 + math.exp(-float(h[t])))            # silu of the convolution's output (the current tap only)
        S = math.exp(dt * A) * S + dt * x * x                       # B = C = x
        want.append((S * x + 2.0 * x) * 0.0)                        # z = 0: silu(z) = 0
    assert got[:, 0].tolist() == pytest.approx(want)
    W["in"] = torch.tensor([[1.0], [1.0]])                         # z = h
    got = P.selective_scan(h, W, "", {"inner": 1, "state": 1, "dt_rank": 1})
    S = 0.0
    for t in range(3):
        v = float(h[t])
        x = v / (1 + math.exp(-v))
        S = math.exp(dt * A) * S + dt * x * x
        assert float(got[t, 0]) == pytest.approx((S * x + 2.0 * x) * x)


def test_plain_router_weighs_the_input_with_logistic_scores():
    torch.manual_seed(3)
    h = torch.randn(4, 6, dtype=torch.float64)
    W = {"router": torch.randn(3, 6)}
    for e in range(3):
        W.update({f"e{e}.gate": torch.randn(5, 6), f"e{e}.up": torch.randn(5, 6), f"e{e}.down": torch.randn(6, 5)})
    idx, w = P.route(h, W, "", 2)
    s = torch.sigmoid(h @ W["router"].double().T)
    assert torch.equal(idx, s.topk(2).indices) and torch.allclose(w, s.topk(2).values)
    assert float(w.sum(-1).max()) > 1.0 or float(w.sum(-1).min()) < 1.0          # not renormalised
    out = P.routed_ff(h, W, "", {"router": {"top": 2}})
    t = 1
    want = sum(P.expert(w[t, c] * h[t:t + 1], W, f"e{int(idx[t, c])}.")[0] for c in range(2))
    assert torch.allclose(out[t], want)
    other = sum(w[t, c] * P.expert(h[t:t + 1], W, f"e{int(idx[t, c])}.")[0] for c in range(2))
    assert not torch.allclose(out[t], other, rtol=1e-3)              # a weight on the output would be another model
