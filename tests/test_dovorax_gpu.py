"""Dovorax in the engine against the plain implementation (tests/plain_dovorax.py): every mechanism alone and the
layers stacked, under every way of cutting the work, with pages and slots used again, and through the generation
loop.  The configurations are made here; weights are random, then sharpened so that a key at a window's edge, the
extra term of a softmax, a carried state, a carried convolution input or a router's choice shows in the result."""
import copy
import json
import math
import os

import numpy as np
import pytest
import torch
from helpers import TOL, cut_bulk_tail, cut_portions, cut_whole, note_error, random_tokens, replay

import plain_dovorax as P

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def dense(ff=48):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, groups=(3, 2), shared=40):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if groups:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def rot_of(dims, base=10000.0, scaling=(4.0, 64, 8.0, 1.0)):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def latent(heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=32, q_rank=20, window=24, base=10000.0, scaling=(4.0, 64, 8.0, 1.0),
           mlp="moe", **more):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": 2.0 * (dim + rot_dim) ** -0.5, "rot": rot_of(rot_dim, base, scaling)}
    if window:
        m["mask"] = {"size": window}
    m.update(more)
    return {"type": "latent_attention", "mixer": m, "mlp": moe() if mlp == "moe" else mlp}


def pair(heads=4, kv_heads=2, dim=16, vdim=8, rot=8, base=100.0, scaling=(8.0, 40, 4.0, 0.5), conv=4, scale=None,
         mheads=2, mdim=12, mvdim=20, cap=6.0, left_scale=0.8, right_scale=0.5, mlp="moe"):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
            "scale": scale if scale is not None else 1.5 * dim ** -0.5}
    if rot:
        left["rot"] = rot_of(rot, base, scaling)
    right = {"heads": mheads, "dim": mdim, "vdim": mvdim, "gate_cap": cap}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": moe() if mlp == "moe" else mlp}


def rec(width=48, blocks=3, conv=3, mlp="moe"):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": moe() if mlp == "moe" else mlp}


def config(layers, width=64, vocab=200, eps=1e-6, alpha=1.5):
    return {"architecture": "Dovorax", "layers": layers, "norm": {"eps": eps}, "postln_alpha": alpha, "vocab": vocab,
            "width": width}


CONFIGS = {
    # each kind of layer alone
    "latent": config([latent(mlp=dense())]),
    "pair": config([pair()]),
    "recurrence": config([rec()]),
    # stacked: readers of another layer's latent through a wider and a narrower window than their owner's, layers
    # without a feed-forward, a dense one, routers with and without groups, several taps and block counts
    "stack": config([latent(), pair(), rec(), latent(window=41, kv_from=0, heads=2, dim=8, vdim=8, q_rank=12),
                     pair(heads=2, kv_heads=2, dim=8, vdim=8, rot=4, scaling=None, conv=2, mheads=1, mdim=8, mvdim=8, mlp=None),
                     rec(width=32, blocks=1, conv=2, mlp=dense(40)),
                     latent(window=9, kv_from=0, mlp=moe(experts=3, top=1, ff=40, groups=None, shared=None))],
                    alpha=2.0),
    # sizes that the tensor-core forms take: a latent whose keys are a multiple of 16 and whose values one of 64; heads
    # of 128 in the attention with one more term (prompts on the tensor-memory kernel); windows that end inside and
    # outside a tile of keys; a memory of 64 x 128
    "wide": config([latent(heads=4, dim=32, rot_dim=16, vdim=64, kv_rank=64, q_rank=48, window=40,
                           mlp=moe(experts=8, top=2, ff=32, groups=(4, 2), shared=64)),
                    pair(heads=4, kv_heads=2, dim=128, vdim=128, rot=64, base=5000.0, scaling=(4.0, 128, 16.0, 1.0),
                         mheads=2, mdim=64, mvdim=128, mlp=dense(256)),
                    rec(width=256, blocks=2, conv=4, mlp=moe(experts=4, top=4, ff=16, groups=None, shared=None)),
                    latent(heads=8, dim=32, rot_dim=16, vdim=64, kv_rank=64, q_rank=48, window=150, kv_from=0, mlp=dense(64))],
                   width=128, vocab=260, alpha=2.5),
    # sizes that are 1, odd or no multiple of 8; a window of one token, a window longer than any request; every expert
    # chosen, one expert alone, one group kept; one tap; one block; the whole head rotated, no rotation; no scaling
    "odd": config([latent(heads=3, dim=10, rot_dim=6, vdim=7, kv_rank=9, q_rank=5, window=1, scaling=None,
                          mlp=moe(experts=3, top=3, ff=20, groups=None, shared=9)),
                   pair(heads=3, kv_heads=3, dim=10, vdim=7, rot=10, scaling=None, conv=1, mheads=3, mdim=5, mvdim=9, cap=2.0,
                        mlp=moe(experts=4, top=1, ff=9, groups=(2, 1), shared=None)),
                   latent(heads=1, dim=24, rot_dim=2, vdim=33, kv_rank=40, q_rank=1, window=5000,
                          mlp=moe(experts=1, top=1, ff=12, groups=None, shared=3)),
                   rec(width=27, blocks=1, conv=1, mlp=None),
                   pair(heads=1, kv_heads=1, dim=6, vdim=12, rot=None, conv=5, mheads=1, mdim=1, mvdim=1, left_scale=1.0,
                        right_scale=1.0, mlp=dense(5)),
                   rec(width=10, blocks=10, conv=6, mlp=dense(1))],
                  width=36, vocab=131, eps=1e-5, alpha=0.7),
}


def sharpen(tensors, cfg, seed):
    """Random N(0, 0.02) matrices hide faults: scores near zero make every key weigh the same, a router whose logits
    all lie within 0.2 always takes the same experts, gates that never leave the middle forget at one rate, and a
    sublayer whose output is small adds next to nothing to a stream that is normed right behind it.  Queries, keys,
    gates and routers are scaled up, decays are spread from channels that keep a token for hundreds of steps to
    channels that forget it in two, the block norms' weights lie around zero (they are applied as 1 + w)."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *shape: torch.randn(*shape, generator=g)
    uni = lambda shape, lo, hi: lo + (hi - lo) * torch.rand(*shape, generator=g)
    scaled = lambda t, f: (t.float() * f).to(torch.bfloat16)
    bf = lambda t: t.to(torch.bfloat16).float()          # what a bfloat16 file would hold
    for name in list(tensors):
        t = tensors[name]
        if name == "embed":
            tensors[name] = scaled(t, 25.0)
        elif name.endswith(("norm1", "norm2", "final.norm")):
            tensors[name] = bf(0.3 * rnd(*t.shape))
        elif name.endswith((".conv",)):
            tensors[name] = bf(0.6 * rnd(*t.shape))
        elif name.endswith((".right.i", ".right.f")):
            tensors[name] = scaled(t, 8.0)
        elif name.endswith(".right.i.b"):
            # input gates mostly below one: the running maximum stays near zero and the read-out's denominator is its floor
            # exp(-m) more often than |n . q|, a sum that random keys let cancel to nearly nothing now and then (every
            # rounding then shows a hundredfold)
            tensors[name] = bf(-1.0 + rnd(*t.shape))
        elif name.endswith((".right.q", ".right.k")):
            tensors[name] = scaled(t, 4.0)
        elif name.endswith(".right.f.b"):
            tensors[name] = bf(uni(t.shape, 0.5, 4.0))
        elif name.endswith(".mix.lam"):
            tensors[name] = bf(uni(t.shape, -4.0, 1.0))
        elif name.endswith((".ra", ".ri")):
            tensors[name] = scaled(t, 12.0)
        elif name.endswith(".b"):
            tensors[name] = bf(0.4 * rnd(*t.shape))
        elif name.endswith(".mlp.router"):
            tensors[name] = scaled(t, 12.0)
        elif name.endswith((".dq", ".uq", ".dkv", ".uk", ".left.q", ".left.k", ".right.q", ".right.k")):
            tensors[name] = scaled(t, 9.0)
        elif ".mlp." in name:
            tensors[name] = scaled(t, 8.0 if name.endswith(".up") else 5.0)
        elif t.dtype == torch.bfloat16 and t.dim() == 2:
            tensors[name] = scaled(t, 6.0)
    return tensors


_folders = {}


def make_folder(cfg, out, seed):
    from safetyraise_lmengine_b200.weights.random_init import write_model_folder
    from safetyraise_lmengine_b200.weights.safetensors_io import WeightFolder, write_safetensors
    out = write_model_folder(cfg, seed, out)
    src = WeightFolder(out)
    tensors = sharpen({n: src.get(n).clone() for n in src.names()}, cfg, seed + 7)
    del src
    write_safetensors(os.path.join(out, "model.safetensors"), tensors)
    return out, tensors


def folder_of(name, tmp_path_factory):
    """(folder, config, weights) of a configuration, written once per session."""
    if name not in _folders:
        cfg = CONFIGS[name]
        seed = 410 + 10 * list(CONFIGS).index(name) + int(os.environ.get("DOVORAX_TEST_SEED", "0"))
        out, tensors = make_folder(cfg, str(tmp_path_factory.mktemp("dovorax_" + name)), seed)
        _folders[name] = (out, cfg, tensors)
    return _folders[name]


@pytest.fixture(scope="session", params=list(CONFIGS))
def model(request, tmp_path_factory):
    return (request.param,) + folder_of(request.param, tmp_path_factory)


_plain = {}


def plain(name, cfg, W, tokens):
    key = (name, tuple(tokens))
    if key not in _plain:
        _plain[key] = P.forward(cfg, W, tokens).numpy()
    return _plain[key]


def build(folder, dtype, num_pages=64, page_size=16, **kw):
    from safetyraise_lmengine_b200 import Engine
    kw.setdefault("max_context", 1024)
    kw.setdefault("max_batch_tokens", 512)
    return Engine.from_folder(folder, dtype=dtype, page_size=page_size, num_pages=num_pages, max_requests=4, **kw)


def check(got, model, requests, dtype):
    name, _, cfg, W = model
    for rid, tokens in requests.items():
        ref = plain(name, cfg, W, tokens)
        rows = np.stack([got[(rid, p)] for p in range(len(tokens))])
        err = np.abs(rows.astype(np.float64) - ref).max(axis=1) / np.abs(ref).max()
        # float32: every position within the tolerance.  bfloat16: a router is a discrete choice, and rounding tips it
        # between two experts at a few positions in a hundred; the stream is off behind the routed layer at such a
        # position, and its keys, values and state colour the positions after it.  So one position in six may be off
        # and the median must lie within half the tolerance: a fault of the cache or the state, which is wrong
        # everywhere after it, still shows.  The tolerance, set for models that add to their stream four times, grows with
        # the root of the number of sums: every sublayer of this design rewrites the whole stream behind its sum, and the
        # next sublayer reads the activation dtype's rounding of it.
        sums = sum(2 if layer.get("mlp") else 1 for layer in cfg["layers"])
        tol = TOL[dtype] * (max(1.0, (sums / 4) ** 0.5) if dtype == "bfloat16" else 1.0)
        bad = np.nonzero(err > tol)[0]
        allowed = len(tokens) // 6 + 2 if dtype == "bfloat16" else 0
        assert dtype == "float32" or np.median(err) <= tol / 2, (name, rid, float(np.median(err)))
        assert bad.size <= allowed, (
            f"{name} request {rid}: first wrong position {bad[0]} of {len(tokens)} "
            f"(rel err {err[bad[0]]:.3e} > {tol:.1e}); wrong positions {bad[:20]}")
        label = dtype if dtype == "float32" else ("bfloat16, Dovorax: median over positions; the tolerance grows with the root "
                                                  "of the depth, one position in six may exceed it")
        note_error(label, float(err.max() if dtype == "float32" else np.median(err)), "dovorax " + name)


def all_pages_free(eng, n):
    return eng.cache.audit() == 0 and all(eng.cache.free_pages(g.name) == n for g in eng.cache.paged_groups)


def requests_for(cfg, lens=(1, 7, 33, 64, 100), seed=0):
    rng = np.random.default_rng(1700 + seed)
    return {f"r{i}": random_tokens(rng, n, cfg["vocab"]) for i, n in enumerate(lens)}


def test_the_sharpened_models_use_what_they_have(model, monkeypatch):
    """The tests below mean something only if a window's edge, the extra term of the softmax, the carried states and
    convolution inputs and the routed weights change the logits by far more than the tolerances: the plain
    implementation with each of them changed differs."""
    name, _, cfg, W = model
    toks = requests_for(cfg, lens=(60,), seed=1)["r0"]
    ref = plain(name, cfg, W, toks)
    big = np.abs(ref).max()
    differs = lambda other_cfg, other_W=W: np.abs(P.forward(other_cfg, other_W, toks).numpy() - ref).max()
    with_zeroed = lambda key, how: {**W, key: how(W[key].clone())}
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            size = (m.get("mask") or {}).get("size")
            if size and size < 60:
                other = copy.deepcopy(cfg)
                other["layers"][i]["mixer"]["mask"]["size"] = size + 1
                assert differs(other) > 50 * TOL["float32"] * big, (i, "window")
        elif layer["type"] == "parallel":
            with monkeypatch.context() as mp:
                plain_rows = P.softmax_rows
                mp.setattr(P, "softmax_rows", lambda s, mask, one_more=False: plain_rows(s, mask, False))
                assert differs(cfg) > 50 * TOL["float32"] * big, (i, "the softmax's extra term")
            if m["left"]["conv"] > 1:
                key = f"l{i}.mix.left.k.conv"
                assert differs(cfg, with_zeroed(key, lambda t: t.index_fill_(1, torch.tensor([0]), 0))) > 50 * TOL["float32"] * big
            # a memory that forgets at once: the forget gate's bias far below zero
            key = f"l{i}.mix.right.f.b"
            assert differs(cfg, with_zeroed(key, lambda t: t.fill_(-30.0))) > 0.003 * big, (i, "memory")
        else:
            key = f"l{i}.mix.lam"
            assert differs(cfg, with_zeroed(key, lambda t: t.fill_(6.0))) > 0.003 * big, (i, "state")
            if m["conv"] > 1:
                key = f"l{i}.mix.conv"
                assert differs(cfg, with_zeroed(key, lambda t: t.index_fill_(1, torch.tensor([0]), 0))) > 0.001 * big
        mlp = layer.get("mlp")
        if mlp and mlp["kind"] == "moe" and mlp["router"]["experts"] > mlp["router"]["top"]:
            key = f"l{i}.mlp.router"
            assert differs(cfg, {**W, key: -W[key].float()}) > 0.003 * big, (i, "router")


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_requests_alone(model, dtype):
    eng = build(model[1], dtype)
    reqs = requests_for(model[2])
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_whole(rid, toks)))
    check(got, model, reqs, dtype)
    assert all_pages_free(eng, 64)


def test_the_stream_after_every_layer(model):
    """float32, layer by layer: the engine's model is cut off behind its first k run steps and its stream (which a
    block of this design leaves normed, with nothing pending) compared with the plain one's."""
    name, folder, cfg, W = model
    toks = requests_for(cfg, lens=(40,), seed=7)["r0"]
    streams = []
    P.forward(cfg, W, toks, streams)
    from safetyraise_lmengine_b200 import StepEntry
    eng = build(folder, "float32")
    order = eng.model.spec.run_order
    for k in range(1, len(order) + 1):
        object.__setattr__(eng.model.spec, "run_order", order[:k])
        slot = eng.open_request()
        eng.step([StepEntry(slot, toks, [])])
        x = eng.workspace.get("residual", len(toks), cfg["width"], torch.float32).cpu().double()
        eng.close_request(slot)
        want = streams[k - 1]
        assert (x - want).abs().max() <= 2e-5 * want.abs().max(), (name, k, float((x - want).abs().max()))
    object.__setattr__(eng.model.spec, "run_order", order)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_then_token_by_token(model, dtype):
    """Most of a prompt in one step, the rest decoded one by one (replayed from CUDA graphs): windows pass over decoded
    tokens, pages behind them are given back, states and carried inputs go from step to step."""
    eng = build(model[1], dtype)
    reqs = {k: v for k, v in requests_for(model[2]).items() if len(v) >= 33}
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_bulk_tail(rid, toks, 32)))
    check(got, model, reqs, dtype)
    assert eng.graph_replays > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_token_at_a_time_from_the_start(model, dtype):
    """The first tokens of a sequence: convolutions with nothing but zeros before them, states that start at zero, a
    running maximum that starts at zero."""
    eng = build(model[1], dtype)
    reqs = requests_for(model[2], lens=(45,), seed=2)
    got = replay(eng, cut_bulk_tail("r0", reqs["r0"], 44))
    check(got, model, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page_size", [4, 16])
def test_portions_of_changing_size(model, dtype, page_size):
    """Portions down to two tokens (shorter than the convolutions' taps), cut in the middle of pages, of key blocks,
    of windows and of the memory's chunks."""
    eng = build(model[1], dtype, num_pages=40, page_size=page_size)
    reqs = {k: v for k, v in requests_for(model[2]).items() if len(v) >= 2}
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_portions(rid, toks)))
        got.update({(rid + "b", p): row for (_, p), row in
                    replay(eng, cut_portions(rid, toks, sizes=(2, 2, 3, 2, 29, 2, 2, 35, 2))).items()})
    check(got, model, reqs, dtype)
    check(got, model, {rid + "b": toks for rid, toks in reqs.items()}, dtype)
    assert eng.cache.audit() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_and_reuse_of_pages_and_slots(model, dtype):
    """Up to four live requests: portions of some beside single tokens of others; requests end and new ones take their
    slots (whose states must start at zero again) and pages (few pages, so the page freed last is used next)."""
    cfg = model[2]
    rng = np.random.default_rng(9)
    lens = {"a": 70, "b": 23, "c": 41, "d": 9, "e": 55, "f": 30, "g": 12}
    reqs = {k: random_tokens(rng, n, cfg["vocab"]) for k, n in lens.items()}
    fed = {k: 0 for k in reqs}

    def take(rid, n):
        lo = fed[rid]
        hi = min(len(reqs[rid]), lo + n)
        fed[rid] = hi
        return (rid, reqs[rid][lo:hi], list(range(hi - lo)))

    steps = [
        {"entries": [take("a", 20), take("b", 5)]},
        {"entries": [take("a", 1), take("b", 18), take("c", 2), take("d", 8)], "end": ["b"]},
        {"entries": [take("a", 1), take("c", 30), take("d", 1), take("e", 7)], "end": ["d"]},
        {"entries": [take("f", 30), take("a", 48), take("c", 1), take("e", 2)], "end": ["a", "f"]},
        {"entries": [take("g", 3), take("c", 8), take("e", 1)], "end": ["c"]},
        {"entries": [take("e", 45), take("g", 1)]},
        {"entries": [take("g", 8)], "end": ["e", "g"]},
    ]
    assert all(fed[k] == len(reqs[k]) for k in reqs)
    eng = build(model[1], dtype, num_pages=24, page_size=8)
    got = replay(eng, steps)
    check(got, model, reqs, dtype)
    opened, reused = eng.cache.reuse_counts()
    assert (reused > 0 or not eng.cache.paged_groups) and all_pages_free(eng, 24)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model, dtype):
    """300 tokens, the last 260 one by one: pages fill, windows move on and their pages turn over, the states are
    renewed 260 times."""
    reqs = requests_for(model[2], lens=(300,), seed=3)
    eng = build(model[1], dtype, num_pages=24, page_size=16)
    got = replay(eng, cut_bulk_tail("r0", reqs["r0"], 260))
    check(got, model, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_in_portions_and_in_one_step(model, dtype):
    """700 tokens in portions of 48 (the later portions stand behind hundreds of cached keys, most of them behind the
    window and their pages gone, and behind states that 600 tokens have written), then at once beside a short request."""
    if model[0] == "odd":
        pytest.skip("one configuration of each kernel is enough")
    reqs = requests_for(model[2], lens=(700, 40), seed=6)
    eng = build(model[1], dtype, num_pages=56, page_size=16, max_batch_tokens=1024)
    got = replay(eng, cut_portions("r0", reqs["r0"], sizes=(48,)))
    check(got, model, {"r0": reqs["r0"]}, dtype)
    got = replay(eng, [{"entries": [("r1", reqs["r1"], list(range(40))), ("r0", reqs["r0"], list(range(700)))],
                        "end": ["r0", "r1"]}])
    check(got, model, reqs, dtype)
    assert all_pages_free(eng, 56)


def test_cuttings_agree_bit_for_bit_in_float32(model):
    """In float32 no sum depends on the cutting or on the batch: the logits of a position are the same bits."""
    reqs = requests_for(model[2], lens=(90, 37), seed=4)
    toks, other = reqs["r0"], reqs["r1"]
    eng = build(model[1], "float32")
    whole = replay(eng, cut_whole("r0", toks))
    tail = replay(eng, cut_bulk_tail("r0", toks, 40))
    parts = replay(eng, cut_portions("r0", toks))
    beside = replay(eng, [{"entries": [("x", other[:30], []), ("r0", toks[:50], list(range(50)))]},
                          {"entries": [("r0", toks[50:], list(range(40))), ("x", other[30:31], [])]}])
    for p in range(len(toks)):
        assert np.array_equal(whole[("r0", p)], tail[("r0", p)]), p
        assert np.array_equal(whole[("r0", p)], parts[("r0", p)]), p
        assert np.array_equal(whole[("r0", p)], beside[("r0", p)]), p


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_refused_step_leaves_nothing_behind(model, dtype):
    """A step that is refused after another one ran: the states of the slot and the pages are as before."""
    from safetyraise_lmengine_b200 import StepEntry
    from safetyraise_lmengine_b200.errors import ShapeError
    reqs = requests_for(model[2], lens=(30,), seed=5)
    toks = reqs["r0"]
    eng = build(model[1], dtype)
    slot = eng.open_request()
    rows = [eng.step([StepEntry(slot, toks[:11], list(range(11)))]).cpu().numpy().copy()]
    with pytest.raises(ShapeError):
        eng.step([StepEntry(slot, [model[2]["vocab"] + 5, 1], [0])])
    rows.append(eng.step([StepEntry(slot, toks[11:], list(range(19)))]).cpu().numpy().copy())
    check({("r0", p): r for p, r in enumerate(np.concatenate(rows))}, model, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_scheduler(model, dtype):
    from safetyraise_lmengine_b200 import LLM, SamplingParams
    name, folder, cfg, W = model
    rng = np.random.default_rng(21)
    prompts = [random_tokens(rng, n, cfg["vocab"]) for n in (5, 19, 11, 3, 26)]        # more requests than slots
    llm = LLM.from_folder(folder, dtype=dtype, page_size=4, num_pages=64, max_active=3, max_batch_tokens=48,
                          prefill_chunk=8, max_context=128, queue_capacity=8)
    llm.eos = set()
    res = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=10))
    for prompt, r in zip(prompts, res):
        assert r.finish_reason == "length" and len(r.tokens) == 10
        toks = list(prompt) + list(r.tokens)
        ref = P.forward(cfg, W, toks[:-1]).numpy()
        for i, tok in enumerate(r.tokens):
            row = ref[len(prompt) - 1 + i]
            if dtype == "float32":
                assert tok == int(np.argmax(row)) or row[tok] >= row.max() - 1e-5 * np.abs(row).max(), (i, tok)
            else:
                assert row[tok] >= row.max() - 3 * TOL[dtype] * np.abs(row).max(), (i, tok)
    assert all_pages_free(llm.engine, 64)


# ---- mechanisms alone, with inputs made so that a fault shows --------------------------------------------------

class _Ctx:
    """The fields of a step's context that the kernels' wrappers read."""
    def __init__(self, q_lens, kv_lens, dev, slots=None):
        self.n_entries, self.max_q_len = len(q_lens), max(q_lens)
        self.cu_q = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32, device=dev)
        self.kv_lens = torch.tensor(kv_lens, dtype=torch.int32, device=dev)
        self.slots = torch.tensor(slots if slots is not None else list(range(len(q_lens))), dtype=torch.int32, device=dev)
        self.entry_of_token = torch.tensor(np.repeat(np.arange(len(q_lens)), q_lens), dtype=torch.int32, device=dev)
        from safetyraise_lmengine_b200.parts import Workspace
        self.kv_bound, self.workspace = max(kv_lens), Workspace(torch.device(dev), 64)
        self.host = {"q_lens": list(q_lens), "kv_lens": list(kv_lens), "starts": [k - q for q, k in zip(q_lens, kv_lens)]}
        self.tables = {}


def _in_steps(total, cuts):
    """Portion sizes that add up to total, cycling through cuts."""
    out, k = [], 0
    while sum(out) < total:
        out.append(min(cuts[k % len(cuts)], total - sum(out)))
        k += 1
    return out


@pytest.mark.parametrize("C,taps", [(40, 4), (27, 1), (64, 2), (130, 6)])
def test_short_convolution_carried_through_steps_and_slots(C, taps):
    """Two requests in slots 2 and 0, cut into portions shorter than the taps, against the convolution of each whole
    sequence; then slot 2 is zeroed and used again."""
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(C + taps)
    w, b_in, b_out = torch.randn(C, taps, generator=g), torch.randn(C, generator=g), torch.randn(C, generator=g)
    lens = {2: 37, 0: 23}
    seqs = {s: torch.randn(n, C + 5, generator=g) for s, n in lens.items()}      # the channels are columns 5.. of a wider row
    want = {s: P.short_conv(x[:, 5:].double() + b_in.double(), w, b_out).float() for s, x in seqs.items()}
    state = torch.zeros(3, 7 + (taps - 1) * C, device=dev)
    wd, bi, bo = w.to(dev), b_in.to(dev), b_out.to(dev)
    for round_ in range(2):
        fed = {s: 0 for s in lens}
        got = {s: [] for s in lens}
        cuts = {2: _in_steps(37, (1, 2, 1, 5, 3, 11)), 0: _in_steps(23, (2, 1, 1, 9))}
        while any(cuts.values()):
            live = [s for s in lens if cuts[s]]
            sizes = [cuts[s].pop(0) for s in live]
            rows = torch.cat([seqs[s][fed[s]:fed[s] + n] for s, n in zip(live, sizes)]).to(dev).contiguous()
            ctx = _Ctx(sizes, [fed[s] + n for s, n in zip(live, sizes)], dev, slots=live)
            out = torch.empty(rows.shape[0], C, device=dev)
            low = torch.empty(rows.shape[0], C, device=dev, dtype=torch.bfloat16)
            ops.short_conv(ctx, rows, 5, C, wd, state, 7, out, in_bias=bi, out_bias=bo, out_low=low)
            ops.conv_carry(ctx, rows, 5, C, taps, state, 7, in_bias=bi)
            at = 0
            for s, n in zip(live, sizes):
                got[s].append(out[at:at + n].cpu())
                assert torch.equal(low[at:at + n].float().cpu(), out[at:at + n].bfloat16().float().cpu())
                at, fed[s] = at + n, fed[s] + n
        for s in lens:
            assert (torch.cat(got[s]) - want[s]).abs().max() <= 1e-5 * want[s].abs().max(), (round_, s)
        assert state[1].abs().max() == 0 and state[:, :7].abs().max() == 0      # nobody's slot, and what lies ahead of the carry
        state.zero_()                                                             # new occupants


@pytest.mark.parametrize("q_dtype,cache_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                                 (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("nq,nkv,dk,dv,pairs,interleaved,taps", [(4, 2, 16, 8, 4, False, 4), (3, 3, 10, 7, 5, False, 1),
                                                                 (2, 1, 64, 64, 16, True, 3), (1, 1, 6, 12, 0, False, 5)])
def test_convolution_norm_rotation_and_append_in_one_kernel(q_dtype, cache_dtype, nq, nkv, dk, dv, pairs, interleaved, taps):
    """A sequence in two portions (the second starts inside the taps' reach) against the plain formulas: q as written,
    k and v as the pages hold them."""
    from safetyraise_lmengine_b200.kernels import ops
    from safetyraise_lmengine_b200.parts import Rotation
    dev, page = "cuda:0", 4
    g = torch.Generator().manual_seed(nq * 100 + dk)
    L, C = 11, nq * dk + nkv * (dk + dv)
    proj = torch.randn(L, C, generator=g)
    w = torch.randn(C, taps, generator=g)
    qw, kw = 1 + 0.3 * torch.randn(dk, generator=g), 1 + 0.3 * torch.randn(dk, generator=g)
    ang = torch.arange(L, dtype=torch.float64)[:, None] * (0.3 ** torch.arange(max(pairs, 1), dtype=torch.float64))[None, :]
    cos, sin = (1.3 * torch.cos(ang)).float(), (1.3 * torch.sin(ang)).float()
    y = P.short_conv(proj, w)

    def turned(x, weight):
        x = P.rms_norm(x, weight, 1e-5)
        if not pairs:
            return x
        out = x.clone()
        c, s = cos.double()[:, None, :], sin.double()[:, None, :]
        if interleaved:
            u, v = x[..., 0:2 * pairs:2], x[..., 1:2 * pairs:2]
            out[..., 0:2 * pairs:2], out[..., 1:2 * pairs:2] = u * c - v * s, v * c + u * s
        else:
            u, v = x[..., :pairs], x[..., pairs:2 * pairs]
            out[..., :pairs], out[..., pairs:2 * pairs] = u * c - v * s, v * c + u * s
        return out
    q_ref = turned(y[:, :nq * dk].reshape(L, nq, dk), qw)
    k_ref = turned(y[:, nq * dk:(nq + nkv) * dk].reshape(L, nkv, dk), kw)
    v_ref = y[:, (nq + nkv) * dk:].reshape(L, nkv, dv)

    pages = [2, 0, 3]
    k_pool = torch.zeros(4, nkv, page, dk, device=dev, dtype=cache_dtype)
    v_pool = torch.zeros(4, nkv, page, dv, device=dev, dtype=cache_dtype)
    state = torch.zeros(2, (taps - 1) * C + 1, device=dev)
    rot = Rotation(cos.to(dev), sin.to(dev), pairs, interleaved) if pairs else None
    q_got = []
    for lo, hi in ((0, 6), (6, 8), (8, 11)):
        ctx = _Ctx([hi - lo], [hi], dev, slots=[1])
        rows = proj[lo:hi].to(dev).contiguous()
        kv_slot = torch.tensor([pages[t // page] * page + t % page for t in range(lo, hi)], dtype=torch.int32, device=dev)
        r = Rotation(rot.cos[lo:hi].contiguous(), rot.sin[lo:hi].contiguous(), pairs, interleaved) if pairs else None
        q = torch.empty(hi - lo, nq * dk, device=dev, dtype=q_dtype)
        ops.conv_norm_rope_append(ctx, rows, w.to(dev), state, 1, qw.to(dev), kw.to(dev), 1e-5, r, q, k_pool, v_pool, kv_slot,
                                  nq, nkv, dk, dv)
        ops.conv_carry(ctx, rows, 0, C, taps, state, 1)
        q_got.append(q.float().cpu())
    tol = 1e-5 if cache_dtype == torch.float32 else 1e-2
    q_tol = 1e-5 if q_dtype == torch.float32 else 1e-2
    assert (torch.cat(q_got).reshape(L, nq, dk) - q_ref).abs().max() <= q_tol * q_ref.abs().max()
    for t in range(L):
        kk = k_pool[pages[t // page], :, t % page].float().cpu()
        vv = v_pool[pages[t // page], :, t % page].float().cpu()
        assert (kk - k_ref[t]).abs().max() <= tol * k_ref.abs().max(), t
        assert (vv - v_ref[t]).abs().max() <= tol * v_ref.abs().max(), t
    assert k_pool[1].abs().max() == 0 and state[0].abs().max() == 0


def _plain_memory(proj, bi, bf, H, d, dv, cap, S=None, n=None, m=None):
    """The recurrence of plain_dovorax.matrix_memory on a stacked projection row q | k | v | gate | i | f."""
    T = proj.shape[0]
    proj = proj.double()
    q = proj[:, :H * d].reshape(T, H, d) * d ** -0.5
    k = proj[:, H * d:2 * H * d].reshape(T, H, d)
    v = proj[:, 2 * H * d:2 * H * d + H * dv].reshape(T, H, dv)
    gi = cap * torch.tanh((proj[:, -2 * H:-H] + bi.double()) / cap)
    gf = P.logsigmoid(cap * torch.tanh((proj[:, -H:] + bf.double()) / cap))
    S = torch.zeros(H, d, dv, dtype=torch.float64) if S is None else S
    n = torch.zeros(H, d, dtype=torch.float64) if n is None else n
    m = torch.zeros(H, dtype=torch.float64) if m is None else m
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        new = torch.maximum(gf[t] + m, gi[t])
        keep, write = torch.exp(gf[t] + m - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + write[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + write[:, None] * k[t]
        m = new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    return out.reshape(T, H * dv), S, n, m


@pytest.mark.parametrize("H,d,dv,cap", [(2, 12, 20, 6.0), (3, 5, 9, 2.0), (1, 1, 1, 12.0), (2, 64, 128, 8.0), (1, 48, 48, 12.0),
                                        (1, 130, 200, 5.0)])
def test_matrix_memory_carried_through_steps_and_slots(H, d, dv, cap):
    """Gates far from zero in both directions (the running maximum moves, the denominator's floor exp(-m) takes over
    and gives way), a sequence in portions down to one token beside another request, against the plain recurrence."""
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(H * 1000 + d)
    width = 2 * H * d + 2 * H * dv + 2 * H
    lens = {1: 61, 3: 19}
    seqs = {}
    for s, n in lens.items():
        x = torch.randn(n, width, generator=g)
        x[:, H * d:2 * H * d] = 0.8 * x[:, :H * d] + 0.2 * x[:, H * d:2 * H * d]      # k near q: n . q does not cancel
        x[:, -2 * H:] *= 6.0                                   # gate logits up to the cap and beyond
        x[n // 2:, -2 * H:-H] -= 8.0                           # then a stretch of small input gates
        seqs[s] = x
    bi, bf = torch.randn(H, generator=g), 2.0 + torch.randn(H, generator=g)
    want = {s: _plain_memory(x, bi, bf, H, d, dv, cap) for s, x in seqs.items()}
    state = torch.zeros(4, H * d * dv + H * d + H, device=dev)
    fed, got = {s: 0 for s in lens}, {s: [] for s in lens}
    cuts = {1: _in_steps(61, (17, 1, 1, 2, 16, 3)), 3: _in_steps(19, (1, 5, 1, 1))}
    while any(cuts.values()):
        live = [s for s in lens if cuts[s]]
        sizes = [cuts[s].pop(0) for s in live]
        rows = torch.cat([seqs[s][fed[s]:fed[s] + n] for s, n in zip(live, sizes)]).to(dev).contiguous()
        ctx = _Ctx(sizes, [fed[s] + n for s, n in zip(live, sizes)], dev, slots=live)
        o = torch.empty(rows.shape[0], H * dv, device=dev)
        ops.matrix_memory_recurrence(ctx, rows, bi.to(dev), bf.to(dev), cap, 1e-6, state, o, H, d, dv)
        at = 0
        for s, n in zip(live, sizes):
            got[s].append(o[at:at + n].cpu())
            at, fed[s] = at + n, fed[s] + n
    for s in lens:
        ref, S, n, m = want[s]
        # a quotient whose denominator |n . q| is a sum of up to 130 products that may nearly cancel: its largest values
        # are the worst conditioned ones
        assert (torch.cat(got[s]) - ref).abs().max() <= 2e-4 * ref.abs().max(), s
        row = state[s].cpu().double()
        assert (row[:H * d * dv].reshape(H, dv, d).transpose(1, 2) - S).abs().max() <= 2e-5 * max(S.abs().max(), 1e-30)
        assert (row[H * d * dv:H * d * dv + H * d].reshape(H, d) - n).abs().max() <= 2e-5 * max(n.abs().max(), 1e-30)
        assert (row[-H:] - m).abs().max() <= 1e-5 * max(m.abs().max(), 1.0)
    assert state[0].abs().max() == 0 and state[2].abs().max() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_memory_read_out_normed_and_gated(dtype):
    from safetyraise_lmengine_b200.kernels import ops
    dev, T, H, dv = "cuda:0", 9, 3, 20
    g = torch.Generator().manual_seed(5)
    o, w, proj = torch.randn(T, H * dv, generator=g), torch.randn(H * dv, generator=g), torch.randn(T, 7 + H * dv, generator=g)
    ref = P.rms_norm(o.reshape(T, H, dv), None, 1e-4).reshape(T, H * dv) * w.double() * torch.sigmoid(proj[:, 7:].double())
    out = torch.empty(T, H * dv, device=dev, dtype=dtype)
    ops.matrix_memory_output(o.to(dev), w.to(dev), 1e-4, proj.to(dev), 7, out, H, dv)
    assert (out.float().cpu() - ref).abs().max() <= (1e-5 if dtype == torch.float32 else 1e-2) * ref.abs().max()


@pytest.mark.parametrize("segments", [False, True])
@pytest.mark.parametrize("C,blocks,w_dtype", [(48, 3, torch.float32), (27, 1, torch.bfloat16), (10, 10, torch.float32),
                                              (256, 2, torch.bfloat16), (130, 1, torch.float32)])
def test_gated_recurrence_carried_through_steps_and_slots(C, blocks, w_dtype, segments):
    """Decays from nearly one to nearly zero; a sequence in portions beside another request, against the plain loop;
    token by token, and with every portion cut into segments that are walked side by side."""
    from safetyraise_lmengine_b200.kernels import ops
    dev, Cb = "cuda:0", C // blocks
    g = torch.Generator().manual_seed(C)
    Ra = (0.5 * torch.randn(blocks, Cb, Cb, generator=g)).to(w_dtype)
    Ri = (0.5 * torch.randn(blocks, Cb, Cb, generator=g)).to(w_dtype)
    ba, bi, yb = torch.randn(C, generator=g), torch.randn(C, generator=g), torch.randn(C, generator=g)
    lam = -5.0 + 7.0 * torch.rand(C, generator=g)
    rate = (8.0 * torch.nn.functional.softplus(lam.double())).float()
    lens = {2: 75, 0: 21}
    u = {s: torch.randn(n, C, generator=g) for s, n in lens.items()}
    y = {s: torch.randn(n, C + 3, generator=g) for s, n in lens.items()}

    def reference(s):
        ub = u[s].double().reshape(-1, blocks, Cb)
        r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, Ra.double()).reshape(-1, C) + ba.double())
        i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, Ri.double()).reshape(-1, C) + bi.double())
        a = torch.exp(-rate.double() * r)
        S, out = torch.zeros(C, dtype=torch.float64), []
        for t in range(lens[s]):
            S = a[t] * S + torch.sqrt(1 - a[t] ** 2) * i[t] * u[s][t].double()
            out.append(S * P.gelu_tanh(y[s][t, 3:].double() + yb.double()))
        return torch.stack(out), S
    state = torch.zeros(3, C + 5, device=dev)
    fed, got = {s: 0 for s in lens}, {s: [] for s in lens}
    cuts = {2: _in_steps(75, (30, 1, 1, 2, 5, 3)), 0: _in_steps(21, (1, 6, 1))}
    while any(cuts.values()):
        live = [s for s in lens if cuts[s]]
        sizes = [cuts[s].pop(0) for s in live]
        uu = torch.cat([u[s][fed[s]:fed[s] + n] for s, n in zip(live, sizes)]).to(dev).contiguous()
        yy = torch.cat([y[s][fed[s]:fed[s] + n] for s, n in zip(live, sizes)]).to(dev).contiguous()
        ctx = _Ctx(sizes, [fed[s] + n for s, n in zip(live, sizes)], dev, slots=live)
        a, b = torch.empty_like(uu), torch.empty_like(uu)
        ops.recurrence_gates(uu, Ra.to(dev), Ri.to(dev), ba.to(dev), bi.to(dev), rate.to(dev), a, b, blocks)
        out = torch.empty_like(uu)
        ops.linear_recurrence(ctx, a, b, yy, 3, yb.to(dev), state, out, in_segments=segments)
        at = 0
        for s, n in zip(live, sizes):
            got[s].append(out[at:at + n].cpu())
            at, fed[s] = at + n, fed[s] + n
    for s in lens:
        ref, S = reference(s)
        assert (torch.cat(got[s]) - ref).abs().max() <= 3e-5 * ref.abs().max(), s
        assert (state[s, :C].cpu().double() - S).abs().max() <= 3e-5 * S.abs().max()
    assert state[1].abs().max() == 0 and state[:, C:].abs().max() == 0


@pytest.mark.parametrize("E,top,groups", [(12, 3, (3, 2)), (6, 2, (1, 1)), (8, 2, (4, 1)), (40, 5, (5, 3)), (3, 3, (1, 1)), (1, 1, (1, 1))])
def test_router_over_all_experts_with_groups(E, top, groups):
    """Logits made so that the best expert overall sits in a group that also wins, that a strong expert of a losing
    group is passed over, and that no two scores are close; both the routing kernel and the one that also orders."""
    from safetyraise_lmengine_b200.kernels import ops
    dev, T = "cuda:0", 70
    g = torch.Generator().manual_seed(E * 10 + top)
    z = torch.randn(T, 4 + E, generator=g) * 3.0
    z[:, 4:] += torch.linspace(0, 0.37, E)[None, :]            # no ties
    cfg = {"experts": E, "top": top}
    if groups != (1, 1):
        cfg["groups"] = {"count": groups[0], "keep": groups[1]}
    want_c, want_w = P.route(z[:, 4:], cfg)
    zd = z.to(dev).contiguous()
    for ordering in (False, True):
        choice = torch.full((T, top), -1, dtype=torch.int32, device=dev)
        weight = torch.zeros(T, top, device=dev)
        if ordering:
            offsets, tiles = torch.zeros(E + 1, dtype=torch.int32, device=dev), torch.zeros(E + 1, dtype=torch.int32, device=dev)
            por, rop = torch.zeros(T * top, dtype=torch.int32, device=dev), torch.zeros(T * top, dtype=torch.int32, device=dev)
            ops.moe_sort(choice, E, offsets, tiles, por, rop, route=(zd, 4, None, weight), scoring="softmax_over_all", groups=groups)
        else:
            ops.moe_route(zd, None, top, choice, weight, column=4, experts=E, scoring="softmax_over_all", groups=groups)
        assert torch.equal(choice.cpu().long(), want_c), ordering
        assert (weight.cpu().double() - want_w).abs().max() <= 1e-6
    if groups[1] < groups[0]:
        free_c, _ = P.route(z[:, 4:], {"experts": E, "top": top})
        assert not torch.equal(free_c, want_c)                   # the groups did change some choice


@pytest.mark.parametrize("out_dtype", [None, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,delta_dtype", [(64, torch.float32), (36, torch.bfloat16), (2048, torch.bfloat16), (1, torch.float32)])
def test_norm_behind_the_scaled_sum(H, delta_dtype, out_dtype):
    from safetyraise_lmengine_b200.kernels import ops
    dev, T = "cuda:0", 5
    g = torch.Generator().manual_seed(H)
    x, d, w = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g).to(delta_dtype), 0.3 * torch.randn(H, generator=g)
    ref = P.rms_norm(1.7 * x.double() + d.double(), w, 1e-5, one_plus=True)
    res = x.to(dev)
    out = torch.empty(T, H, device=dev, dtype=out_dtype) if out_dtype else None
    ops.postnorm_scale_add(res, d.to(dev), w.to(dev), 1.7, 1e-5, True, out)
    assert (res.cpu() - ref).abs().max() <= 1e-5 * ref.abs().max()
    if out is not None:
        assert torch.equal(out.cpu(), res.cpu().to(out_dtype))
    # two results summed with weights on their way in
    d2 = torch.randn(T, H, generator=g).to(delta_dtype)
    ref = P.rms_norm(1.7 * x.double() + 0.8 * d.double() - 0.5 * d2.double(), w, 1e-5, one_plus=True)
    res = x.to(dev)
    ops.postnorm_scale_add(res, None, w.to(dev), 1.7, 1e-5, True, out, terms=((d.to(dev), 0.8), (d2.to(dev), -0.5)))
    assert (res.cpu() - ref).abs().max() <= 1e-5 * ref.abs().max()


def test_ramped_rotary_table_and_norm_of_columns():
    from safetyraise_lmengine_b200.config.spec import PositionSpec
    from safetyraise_lmengine_b200.kernels import ops
    from safetyraise_lmengine_b200.parts import ModelContext
    from safetyraise_lmengine_b200.parts.position import RotaryHalf
    dev = torch.device("cuda:0")
    for rot in (rot_of(12, 30000.0, (6.0, 512, 16.0, 2.0)), rot_of(6, 100.0, (3.0, 30, 2.0, 0.25)), rot_of(8, 10000.0, None)):
        sc = rot.get("scaling")
        spec = PositionSpec("rotary_half", theta=rot["base"], rotary_dim=rot["dims"], head_dim=rot["dims"],
                            ramp=(sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None)
        enc = RotaryHalf(spec, ModelContext(dev, torch.float32, 64))
        ctx = _Ctx([5], [2000], "cuda:0")
        ctx.T, ctx.positions = 5, torch.tensor([0, 1, 77, 1030, 1999], dtype=torch.int32, device=dev)
        got = enc.rotation(ctx)
        f, mag = P.rotary(rot)
        ang = ctx.positions.cpu().double()[:, None] * f[None, :]
        assert (got.cos.cpu().double() - mag * torch.cos(ang)).abs().max() <= 2e-7 * mag
        assert (got.sin.cpu().double() - mag * torch.sin(ang)).abs().max() <= 2e-7 * mag
    g = torch.Generator().manual_seed(3)
    x, w = torch.randn(6, 50, generator=g), torch.randn(20, generator=g)
    for dt in (torch.float32, torch.bfloat16):
        out = torch.empty(6, 20, device=dev, dtype=dt)
        ops.rmsnorm_columns(x.to(dev), 11, 20, w.to(dev), 1e-5, out)
        ref = P.rms_norm(x[:, 11:31], w, 1e-5)
        assert (out.float().cpu() - ref).abs().max() <= (1e-5 if dt == torch.float32 else 1e-2) * ref.abs().max()


@pytest.mark.parametrize("heads,kv_heads,dk,dv,window,dtype", [(4, 2, 16, 8, 0, torch.float32), (4, 2, 64, 64, 0, torch.bfloat16),
                                                               (2, 1, 128, 128, 0, torch.bfloat16), (3, 3, 10, 7, 29, torch.float32),
                                                               (4, 2, 64, 64, 45, torch.bfloat16), (4, 1, 32, 64, 64, torch.bfloat16)])
def test_attention_with_one_more_term_and_a_far_key(heads, kv_heads, dk, dv, window, dtype):
    """Hundreds of keys of which one, far back, carries nearly all the weight of one query, and a query whose scores are
    all so low that the extra term carries it: prompt rows and a decoded token, against the plain softmax."""
    from safetyraise_lmengine_b200.kernels import ops
    dev, page, L = "cuda:0", 16, 331
    g = torch.Generator().manual_seed(dk)
    k, v = torch.randn(L, kv_heads, dk, generator=g), torch.randn(L, kv_heads, dv, generator=g)
    q = torch.randn(L, heads, dk, generator=g)
    scale = dk ** -0.5
    far = 3 if not window else L - window                          # just inside the window when there is one
    rep = heads // kv_heads
    k[:, :, 0] = 3.0 + 0.3 * k[:, :, 0]                           # every key points the same way along element 0 ...
    k[far] *= 3.0
    if window:                                                    # the same key just outside the window, with a value that would show
        k[L - 1 - window], v[L - 1 - window] = k[far], 50.0
    q[L - 1] = 14.0 * k[far].repeat_interleave(rep, dim=0) / ((k[far] ** 2).sum(-1).repeat_interleave(rep)[:, None] * scale)
    q[L - 2] = 0.0
    q[L - 2, :, 0] = -10.0 / (3.0 * scale)                        # ... so this query's scores all lie near -10
    if dtype == torch.bfloat16:
        k, v = k.bfloat16().float(), v.bfloat16().float()
    kk, vv = k.repeat_interleave(heads // kv_heads, dim=1).double(), v.repeat_interleave(heads // kv_heads, dim=1).double()
    s = torch.einsum("ihd,jhd->hij", q.double(), kk) * scale
    a = P.softmax_rows(s, P.visible(L, window or None), one_more=True)
    ref = torch.einsum("hij,jhd->ihd", a, vv).reshape(L, heads * dv)
    assert a[:, L - 1, far].min() > 0.5 and a[:, L - 2].sum(-1).max() < 0.5
    n_pages = (L + page - 1) // page
    order = torch.randperm(n_pages, generator=g).tolist()
    k_pool = torch.zeros(n_pages, kv_heads, page, dk, device=dev, dtype=dtype)
    v_pool = torch.zeros(n_pages, kv_heads, page, dv, device=dev, dtype=dtype)
    for t in range(L):
        k_pool[order[t // page], :, t % page] = k[t].to(dev)
        v_pool[order[t // page], :, t % page] = v[t].to(dev)
    table = torch.tensor([order], dtype=torch.int32, device=dev)
    sink = torch.zeros(heads, device=dev)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for first in (0, L - 40, L - 1):                             # the whole prompt, a portion behind a context, one token
        ctx = _Ctx([L - first], [L], dev)
        out = torch.empty(L - first, heads * dv, device=dev, dtype=dtype)
        ops.paged_attention_general(ctx, q[first:].reshape(L - first, -1).to(dev).contiguous(), k_pool, v_pool, out, table, sink,
                                    heads, kv_heads, dk, dv, scale, window)
        assert (out.float().cpu() - ref[first:]).abs().max() <= tol * ref.abs().max(), first


@pytest.mark.parametrize("window", [45, 0])
def test_latent_attention_on_both_roads_at_a_window_edge(window):
    """Pages of [latent | key part] for 200 keys; the last query's weight sits on a key just inside its window (far back
    without one), the same key part just outside it belongs to a latent whose values would show; the pages wholly behind
    the step's reach are gone.  In the latent space (decode steps, float32) and in the heads' own space (bfloat16 prompts),
    whole, as a portion and as one token, against the plain per-head attention."""
    from safetyraise_lmengine_b200.kernels import ops
    dev, page, L = "cuda:0", 16, 200
    H, dim, rot, dv, rank = 4, 32, 16, 64, 64
    g = torch.Generator().manual_seed(7 + window)
    bf = lambda t: t.bfloat16().float()
    c, kr = bf(torch.randn(L, rank, generator=g)), bf(torch.randn(L, rot, generator=g))
    uk, uv = bf(0.2 * torch.randn(H * dim, rank, generator=g)), bf(0.2 * torch.randn(H * dv, rank, generator=g))
    q = torch.randn(L, H, dim + rot, generator=g)
    scale = 0.7 * (dim + rot) ** -0.5
    far = L - window if window else 5
    kr[far] *= 3.0
    q[L - 1, :, :dim] = 0.0
    q[L - 1, :, dim:] = 14.0 * kr[far] / ((kr[far] ** 2).sum() * scale)
    if window:
        kr[L - 1 - window], c[L - 1 - window] = kr[far], 6.0
    kn = (c.double() @ uk.double().T).view(L, H, dim)
    v = (c.double() @ uv.double().T).view(L, H, dv)
    s_ = (torch.einsum("ihd,jhd->hij", q[..., :dim].double(), kn) + torch.einsum("ihd,jd->hij", q[..., dim:].double(), kr.double())) * scale
    a = P.softmax_rows(s_, P.visible(L, window or None))
    ref = torch.einsum("hij,jhd->ihd", a, v).reshape(L, H * dv)
    assert a[:, L - 1, far].min() > 0.5
    n_pages = (L + page - 1) // page
    order = torch.randperm(n_pages, generator=g).tolist()
    uk_d = uk.to(dev).bfloat16()
    uv_d = uv.to(dev).bfloat16()
    up_kv = torch.cat([uk_d, uv_d]).contiguous()
    for dtype in (torch.float32, torch.bfloat16):
        cache = torch.zeros(n_pages, 1, page, rank + rot, device=dev, dtype=dtype)
        for t in range(L):
            cache[order[t // page], 0, t % page] = torch.cat([c[t], kr[t]]).to(dev)
        for first in (0, L - 60, L - 1):
            n = L - first
            reach = max(0, first - window + 1) if window else 0          # the first key any row of the step sees
            table = torch.tensor([[-1 if (pg + 1) * page <= reach else order[pg] for pg in range(n_pages)]],
                                 dtype=torch.int32, device=dev)
            ctx = _Ctx([n], [L], dev)
            ctx.max_kv_len = L
            qd = q[first:].reshape(n, -1).to(dev).contiguous()
            tol = 2e-5 if dtype == torch.float32 else 2e-2
            # in the latent space
            w_k = (uk_d if dtype == torch.bfloat16 else uk.to(dev)).view(H, dim, rank).contiguous()
            w_v = (uv_d if dtype == torch.bfloat16 else uv.to(dev)).view(H, dv, rank).transpose(1, 2).contiguous()
            q_lat = torch.empty(n, H * (rank + rot), device=dev)
            ops.latent_absorb(qd, w_k, None, q_lat, H, dim, rot, rank)
            o_lat = torch.empty(n, H * rank, device=dev)
            ops.paged_attention_general(ctx, q_lat, cache, None, o_lat, table, None, H, 1, rank + rot, rank, scale, window)
            out = torch.empty(n, H * dv, device=dev, dtype=dtype)
            ops.latent_expand(o_lat, w_v, qd, -1, out, H, rank, dv)
            assert (out.float().cpu() - ref[first:]).abs().max() <= tol * ref.abs().max(), (dtype, first, "latent space")
            if dtype != torch.bfloat16 or n <= 4:
                continue
            # in the heads' own space: the latents from the step's reach on, one product for all heads' keys and values
            cu_kv = torch.tensor([-reach], dtype=torch.int32, device=dev)
            kv_first = torch.tensor([reach], dtype=torch.int32, device=dev)
            latents = torch.zeros(L - reach, rank, device=dev, dtype=dtype)
            ops.latent_gather(ctx, cache, latents, table, cu_kv, rank, kv_first)
            kv_rows = torch.empty(L - reach, H * (dim + dv), device=dev, dtype=dtype)
            ops.gemm(latents, up_kv, kv_rows)
            qh = torch.empty(n, H * (dim + rot), device=dev)
            ops.latent_rotate_q(qd, None, qh, H, dim, rot)
            out = torch.empty(n, H * dv, device=dev, dtype=dtype)
            ops.latent_prefill_attention(ctx, qh, cache, kv_rows, cu_kv, out, table, H, dim, rot, dv, rank, H * dim, scale, window)
            assert (out.float().cpu() - ref[first:]).abs().max() <= tol * ref.abs().max(), (dtype, first, "head space")


def _experts_plain(x, up, down, choice, weight, shared):
    out = torch.zeros(x.shape[0], down.shape[1], dtype=torch.float64)
    for t in range(x.shape[0]):
        for e, w in zip(choice[t].tolist(), weight[t]):
            out[t] += w * (down[e].double() @ P.gelu_erf(up[e].double() @ x[t].double()))
    return out + shared.double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_without_a_gate(dtype):
    """The grouped products with the exact gelu in the first one's epilogue, rows of one token under several experts."""
    from safetyraise_lmengine_b200.kernels import ops
    dev, T, H, I, E, top = "cuda:0", 37, 64, 24, 5, 2
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g).to(dtype)
    up, down = (0.3 * torch.randn(E, I, H, generator=g)).to(dtype), (0.3 * torch.randn(E, H, I, generator=g)).to(dtype)
    choice = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).int()
    weight, shared = torch.rand(T, top, generator=g), torch.randn(T, H, generator=g).to(dtype)
    ref = _experts_plain(x.float(), up.float(), down.float(), choice, weight.double(), shared.float())
    offsets, tiles = torch.zeros(E + 1, dtype=torch.int32, device=dev), torch.zeros(E + 1, dtype=torch.int32, device=dev)
    por, rop = torch.zeros(T * top, dtype=torch.int32, device=dev), torch.zeros(T * top, dtype=torch.int32, device=dev)
    ops.moe_sort(choice.to(dev).contiguous(), E, offsets, tiles, por, rop)
    y = torch.empty(T * top, I, device=dev, dtype=dtype)
    ops.moe_grouped(x.to(dev), por, top, up.to(dev), y, offsets, tiles, act="gelu")
    rows = torch.empty(T * top, H, device=dev)
    ops.moe_grouped(y, None, 1, down.to(dev), rows, offsets, tiles)
    out = torch.empty(T, H, device=dev, dtype=dtype)
    ops.moe_combine(rows, rop.view(T, top), weight.to(dev), shared.to(dev), out)
    assert (out.float().cpu() - ref).abs().max() <= (2e-5 if dtype == torch.float32 else 2e-2) * ref.abs().max()


@pytest.mark.parametrize("tile", [128, 256])
def test_experts_without_a_gate_in_tiles_of_tensor_memory(tile):
    """Steps of many tokens: every expert's rows in whole tiles, both products on the persistent tensor-memory kernel
    with the exact gelu in the first one's epilogue."""
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(15)
    for T, E, top, H, ff in ((700, 5, 2, 64, 48), (130, 3, 1, 136, 200), (512, 4, 4, 256, 128)):
        x = torch.randn(T, H, generator=g).bfloat16()
        up = (0.4 * torch.randn(E, ff, H, generator=g)).bfloat16()
        dn = (0.3 * torch.randn(E, H, ff, generator=g)).bfloat16()
        choice = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
        weight, shared = torch.rand(T, top, generator=g), torch.randn(T, H, generator=g).bfloat16()
        n = T * top
        n_tiles = n // tile + E
        d = lambda t: t.to(dev)
        heads = torch.zeros(2, E + 1, dtype=torch.int32, device=dev)
        group = torch.full((n_tiles,), -7, dtype=torch.int32, device=dev)
        por = torch.full((n_tiles * tile,), -7, dtype=torch.int32, device=dev)
        rop = torch.zeros(n, dtype=torch.int32, device=dev)
        ops.moe_sort(d(choice), E, heads[0], heads[1], por, rop, tile_rows=tile, group_of_tile=group)
        xs = torch.empty(n_tiles * tile, H, dtype=torch.bfloat16, device=dev)
        ops.moe_gather_rows(d(x), por, top, xs)
        y = torch.zeros(n_tiles * tile, ff, dtype=torch.bfloat16, device=dev)
        ops.gemm_tn_tcgen05_grouped(xs, d(up), y, group, act="gelu", tile_rows=tile)
        rows = torch.zeros(n_tiles * tile, H, device=dev)
        ops.gemm_tn_tcgen05_grouped(y, d(dn), rows, group, tile_rows=tile)
        out = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
        ops.moe_combine(rows, rop.view(T, top), d(weight), d(shared), out)
        assert ops.gemm_error_flag(torch.device(dev)) == 0
        want = _experts_plain(x.float(), up.float(), dn.float(), choice, weight.double(), shared.float())
        err = (out.cpu().double() - want).abs().max() / want.abs().max()
        assert err < 2e-2, (T, E, top, float(err))


def test_command_line_and_trace_replay(tmp_path, tmp_path_factory):
    import subprocess
    import sys
    from conftest import ROOT
    folder, cfg, W = folder_of("stack", tmp_path_factory)
    env = dict(os.environ, PYTHONPATH=ROOT)
    cli = lambda *a: subprocess.run([sys.executable, "-m", "safetyraise_lmengine_b200", *a], env=env,
                                    capture_output=True, text=True, timeout=600)
    out = cli("inspect", "--model-path", folder, "--context", "64")
    assert out.returncode == 0, out.stderr
    info = json.loads(out.stdout)
    assert info["spec"]["architecture"] == "Dovorax"
    kinds = [g["kind"] for g in info["cache_groups"]]
    assert "fixed_state" in kinds and "paged_window" in kinds and "paged_all" in kinds
    svc, req = tmp_path / "svc.json", tmp_path / "req.json"
    svc.write_text(json.dumps({"model_path": folder, "model_name": "stack",
                               "engine": {"max_context": 128, "max_active": 2, "prefill_chunk": 4, "page_size": 4,
                                          "num_pages": 40, "dtype": "float32", "max_batch_tokens": 32}}))
    prompt = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    req.write_text(json.dumps({"prompt_ids": prompt, "max_tokens": 6, "temperature": 0.0}))
    out = cli("run", "--config", str(svc), "--request", str(req))
    assert out.returncode == 0, out.stderr
    res = json.loads(out.stdout)
    toks = list(prompt)
    for tok in res["tokens"]:
        row = P.forward(cfg, W, toks)[-1].numpy()
        assert row[tok] >= row.max() - 1e-5 * np.abs(row).max()
        toks.append(tok)
    assert len(res["tokens"]) == 6 and res["finish_reason"] == "length"

    rng = np.random.default_rng(2)
    a, b = random_tokens(rng, 50, cfg["vocab"]), random_tokens(rng, 40, cfg["vocab"])
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": [1]}, {"id": "b", "tokens": b[:39], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[39:], "want": [0]}, {"id": "a", "tokens": a[32:], "want": [17]}],
         "end": ["a", "b"]},
    ]
    ra, rb = plain("stack", cfg, W, a), plain("stack", cfg, W, b)
    biggest = max(np.abs(ra).max(), np.abs(rb).max())
    for dtype in ("float32", "bfloat16"):
        out_dir = tmp_path / ("out_" + dtype)
        proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out",
                               str(out_dir), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                              capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2"]
        read = lambda i: np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        tol = TOL[dtype] * (1.0 if dtype == "float32" else 4.0)        # seven layers, and a router's close calls (see `check`)
        for got, ref in ((read(0), ra[[0, 29]]), (read(1), ra[[31]]), (read(2), np.stack([rb[39], ra[49]]))):
            assert got.shape == ref.shape and np.abs(got - ref).max() <= tol * biggest


# ---- configurations drawn at random: layer order, sizes and constants that no other test chose -----------------

def random_config(seed):
    rng = np.random.default_rng(5000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    width = pick(40, 64, 96, 128, 160)
    layers, owners = [], []

    def some_mlp():
        r = rng.random()
        if r < 0.2:
            return None
        if r < 0.4:
            return dense(pick(8, 33, 64, 100))
        count = pick(1, 2, 3, 4)
        per = pick(1, 2, 3)
        keep = int(rng.integers(1, count + 1))
        return moe(experts=count * per, top=int(rng.integers(1, min(per * keep, 4) + 1)), ff=pick(8, 16, 24, 40, 50),
                   groups=(count, keep) if rng.random() < 0.7 else None, shared=pick(None, 16, 50))

    for i in range(int(rng.integers(2, 7))):
        r = rng.random()
        if r < 0.3:
            kv = pick(1, 2, 3)
            dim, vdim = pick((8, 8), (16, 40), (24, 16), (32, 64), (64, 64), (128, 128), (48, 80), (80, 56))
            rot = pick(None, 2, dim // 2 - (dim // 2) % 2, dim)
            layers.append(pair(heads=kv * pick(1, 2, 4), kv_heads=kv, dim=dim, vdim=vdim, rot=rot or None, base=pick(50.0, 10000.0),
                               scaling=pick(None, (4.0, 64, 4.0, 1.0), (16.0, 200, 32.0, 0.5)), conv=pick(1, 2, 4), scale=pick(0.1, 0.3),
                               mheads=pick(1, 2, 5), mdim=pick(4, 16, 33, 64), mvdim=pick(4, 16, 40, 64, 100), cap=pick(3.0, 15.0),
                               left_scale=pick(0.5, 1.0, 1.2), right_scale=pick(0.3, 1.0), mlp=some_mlp()))
        elif r < 0.55:
            layers.append(rec(width=pick(12, 40, 96, 130), blocks=pick(1, 2), conv=pick(1, 2, 4), mlp=some_mlp()))
        elif owners and rng.random() < 0.4:
            j = owners[int(rng.integers(len(owners)))]
            m = copy.deepcopy(layers[j]["mixer"])
            m.pop("mask", None)
            window = pick(None, 3, 20, 75, 300)
            if window:
                m["mask"] = {"size": window}
            m.update(kv_from=j, heads=pick(1, 2, 6), dim=pick(8, 16, 40), vdim=pick(8, 24, 64), q_rank=pick(4, 16, 30))
            m["scale"] = pick(0.2, 0.5)
            layers.append({"type": "latent_attention", "mixer": m, "mlp": some_mlp()})
        else:
            dim, rot_dim, vdim, rank = pick((8, 4, 8, 16), (16, 16, 40, 48), (24, 8, 16, 20), (32, 32, 64, 64), (48, 16, 64, 48))
            layers.append(latent(heads=pick(1, 2, 4, 6), dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, q_rank=pick(4, 16, 30),
                                 window=pick(None, 1, 9, 16, 50, 129, 1000), base=pick(100.0, 20000.0),
                                 scaling=pick(None, (4.0, 64, 4.0, 1.0), (8.0, 512, 32.0, 1.0)), mlp=some_mlp()))
            owners.append(len(layers) - 1)
    return config(layers, width=width, vocab=pick(97, 160, 301), eps=pick(1e-6, 1e-5, 1e-4), alpha=pick(0.5, 1.0, 2.0, 3.0))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Whatever the order of layers and the sizes: float32 within the tolerance at every position under a cutting with
    portions, decoded tokens and a second request beside it; bfloat16 by the rule of `check`."""
    cfg = random_config(seed)
    out, W = make_folder(cfg, str(tmp_path / "m"), 900 + seed)
    rng = np.random.default_rng(seed)
    reqs = {"a": random_tokens(rng, 180, cfg["vocab"]), "b": random_tokens(rng, 37, cfg["vocab"])}
    a, b = reqs["a"], reqs["b"]
    steps = [{"entries": [("a", a[:61], list(range(61)))]},
             {"entries": [("b", b[:2], [0, 1]), ("a", a[61:64], [0, 1, 2])]},
             {"entries": [("a", a[64:150], list(range(86))), ("b", b[2:3], [0])]},
             {"entries": [("b", b[3:36], list(range(33))), ("a", a[150:151], [0])]}]
    steps += [{"entries": [("a", a[i:i + 1], [0])] + ([("b", b[36:], [0])] if i == 151 else [])} for i in range(151, 180)]
    model = (f"random {seed}", out, cfg, W)
    for dtype in DTYPES:
        eng = build(out, dtype, num_pages=20, page_size=16)
        check(replay(eng, steps), model, reqs, dtype)
        assert all_pages_free(eng, 20)
