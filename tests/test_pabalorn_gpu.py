"""Pabalorn in the engine against the plain implementation (tests/plain_pabalorn.py): every mechanism alone and
the layers stacked, under every way of cutting the work, with pages and slots used again, and through the
generation loop.  The configurations are made here; weights are random, then sharpened so that a key at a
window's edge, the cap on the scores, a carried state, a carried convolution input or a router's choice shows
in the result."""
import copy
import json
import os

import numpy as np
import pytest
import torch
from helpers import TOL, cut_bulk_tail, cut_portions, cut_whole, note_error, random_tokens, replay

import plain_pabalorn as P

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def moe(experts=6, top=2, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def att(heads=4, kv_heads=2, dim=16, vdim=24, window=24, softcap=4.0, rot=8, base=10000.0, mlp="moe", **more):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if softcap:
        m["softcap"] = softcap
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    m.update(more)
    return {"type": "attention", "mixer": m, "mlp": moe() if mlp == "moe" else mlp}


def pair(heads=4, kv_heads=1, dim=16, vdim=8, window=13, rot=16, base=100.0, scaling=(8.0, 1.0, 4.0, 64),
         inner=40, state=6, dt_rank=3, conv=4, mlp="moe"):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 1.3 * dim ** -0.5}
    if window:
        left["mask"] = {"size": window}
    if rot:
        left["rot"] = {"dims": rot, "base": base}
        if scaling:
            left["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    right = {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": moe() if mlp == "moe" else mlp}


def config(layers, width=64, vocab=200, eps=1e-6):
    return {"architecture": "Pabalorn", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


CONFIGS = {
    # each kind of layer alone
    "attention": config([att()]),
    "pair": config([pair()]),
    # stacked: layers that read another layer's keys and values through a wider and a narrower window than their
    # owner's, layers without a feed-forward, one expert of three, several states and taps
    "stack": config([att(), pair(), att(window=41, kv_from=0), pair(heads=2, kv_heads=2, dim=8, vdim=8, window=None, rot=4,
                                                                 scaling=None, inner=24, state=16, dt_rank=5, conv=2, mlp=None),
                     att(heads=2, kv_heads=2, dim=8, vdim=8, window=7, softcap=2.0, rot=8, mlp=None),
                     att(window=9, kv_from=0, mlp=moe(experts=3, top=1, ff=40)), pair(state=24, inner=72, conv=3)]),
    # sizes that the tensor-core forms of the attention take; windows that end inside and outside a tile of keys
    "wide": config([att(heads=4, kv_heads=2, dim=32, vdim=64, window=40, rot=16, mlp=moe(experts=8, top=2, ff=32)),
                    pair(heads=4, kv_heads=1, dim=64, vdim=128, window=150, rot=32, scaling=(4.0, 1.0, 2.0, 96),
                         inner=256, state=16, dt_rank=8),
                    att(heads=8, kv_heads=8, dim=16, vdim=64, window=None, softcap=9.0, rot=16, mlp=moe(experts=4, top=4, ff=16))],
                   width=128, vocab=260),
    # heads of 128 for keys and values: prompts of the capped attention on the tensor-memory kernel, the attention
    # beside the scan on the framework's kernels of equal head sizes; a reader of heads of 128; 128 states
    "heads128": config([att(heads=4, kv_heads=2, dim=128, vdim=128, window=100, softcap=6.0, rot=64),
                        pair(heads=2, kv_heads=2, dim=128, vdim=128, window=70, rot=128, base=5000.0,
                             scaling=(4.0, 1.0, 4.0, 128), inner=48, state=128, dt_rank=4, mlp=moe(experts=4, top=2, ff=32)),
                        att(heads=4, kv_heads=2, dim=128, vdim=128, window=33, softcap=3.0, rot=64, kv_from=0, mlp=None)],
                       width=128, vocab=210),
    # sizes that are 1, odd or no multiple of 8; a window of one token, a window longer than any request; all
    # experts chosen, one expert of two; one state, one tap, a step size of rank 1; the whole head rotated, no rotation
    "odd": config([att(heads=3, kv_heads=1, dim=24, vdim=8, window=1, rot=24, mlp=moe(experts=3, top=3, ff=20)),
                   pair(heads=3, kv_heads=3, dim=10, vdim=7, window=5000, rot=2, scaling=None, inner=27, state=1, dt_rank=1,
                        conv=1, mlp=moe(experts=2, top=1, ff=9)),
                   att(heads=1, kv_heads=1, dim=40, vdim=33, window=2, softcap=None, rot=None, mlp=moe(experts=1, top=1, ff=12)),
                   pair(heads=1, kv_heads=1, dim=6, vdim=12, window=3, rot=6, inner=9, state=3, dt_rank=2, conv=5, mlp=None)],
                  width=36, vocab=131, eps=1e-5),
}


def sharpen(tensors, cfg, seed):
    """Random N(0, 0.02) matrices and vectors of 1 + N(0, 0.1) hide faults: scores near zero make every key weigh
    the same and never reach a cap, a router whose logits all lie within 0.2 always takes the same experts, a scan
    whose decays are all alike forgets at one rate, and a mixer whose output weights are small adds next to nothing
    to the stream.  Queries, keys and the router are scaled up, the scan's step sizes and decays are spread from
    states that keep a token for hundreds of steps to states that forget it in two, norm weights lie around zero
    (they are applied as 1 + w), biases are of the size of what they are added to."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *shape: torch.randn(*shape, generator=g)
    uni = lambda shape, lo, hi: lo + (hi - lo) * torch.rand(*shape, generator=g)
    scaled = lambda t, f: (t.float() * f).to(torch.bfloat16)
    bf = lambda t: t.to(torch.bfloat16).float()          # what a bfloat16 file would hold
    tensors["embed"] = scaled(tensors["embed"], 25.0)
    for name in list(tensors):
        t = tensors[name]
        if name.endswith(("norm1", "embed.norm", "final.norm")):
            tensors[name] = bf(0.3 * rnd(*t.shape))
        elif name.endswith((".q", ".k")):
            tensors[name] = scaled(t, 10.0)
        elif name.endswith((".q.b", ".k.b", ".v.b")):
            tensors[name] = bf(0.7 * rnd(*t.shape))
        elif name.endswith((".left.out", ".right.out")):
            tensors[name] = bf(uni(t.shape, 0.5, 1.6))
        elif name.endswith((".mix.v", ".mix.o", ".left.v", ".left.o", ".right.o")):
            tensors[name] = scaled(t, 4.0)
        elif name.endswith(".right.in"):
            tensors[name] = scaled(t, 7.0)
        elif name.endswith(".right.conv"):
            tensors[name] = bf(0.6 * rnd(*t.shape))
        elif name.endswith((".right.conv.b", ".right.D")):
            tensors[name] = bf(0.5 * rnd(*t.shape))
        elif name.endswith(".right.x"):
            tensors[name] = scaled(t, 9.0)
        elif name.endswith(".right.dt"):
            tensors[name] = scaled(t, 20.0)
        elif name.endswith(".right.dt.b"):
            tensors[name] = bf(uni(t.shape, -5.0, 1.0))
        elif name.endswith(".right.A_log"):
            tensors[name] = bf(uni(t.shape, -4.0, 1.2))
        elif name.endswith(".mlp.router"):
            tensors[name] = scaled(t, 12.0)
        elif ".mlp.e" in name:
            tensors[name] = scaled(t, 8.0 if name.endswith((".gate", ".up")) else 3.0)
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
        seed = 170 + 10 * list(CONFIGS).index(name) + int(os.environ.get("PABALORN_TEST_SEED", "0"))
        out, tensors = make_folder(cfg, str(tmp_path_factory.mktemp("pabalorn_" + name)), seed)
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
        # position, its keys, values and state colour the positions after it, and the next norm brings most of it
        # back.  So one position in six may be off and the median must lie within half the tolerance: a fault of
        # the cache or the state, which is wrong everywhere after it, still shows.  The tolerance, set for models of
        # two layers, grows with the root of the depth.
        tol = TOL[dtype] * (max(1.0, (len(cfg["layers"]) / 2) ** 0.5) if dtype == "bfloat16" else 1.0)
        bad = np.nonzero(err > tol)[0]
        allowed = len(tokens) // 6 + 2 if dtype == "bfloat16" else 0
        assert dtype == "float32" or np.median(err) <= tol / 2, (name, rid, float(np.median(err)))
        assert bad.size <= allowed, (
            f"{name} request {rid}: first wrong position {bad[0]} of {len(tokens)} "
            f"(rel err {err[bad[0]]:.3e} > {tol:.1e}); wrong positions {bad[:20]}")
        label = dtype if dtype == "float32" else ("bfloat16, Pabalorn: median over positions; the tolerance grows with the root "
                                                  "of the depth, one position in six may exceed it")
        note_error(label, float(err.max() if dtype == "float32" else np.median(err)), "pabalorn " + name)


def all_pages_free(eng, n):
    return eng.cache.audit() == 0 and all(eng.cache.free_pages(g.name) == n for g in eng.cache.paged_groups)


def requests_for(cfg, lens=(1, 7, 33, 64, 100), seed=0):
    rng = np.random.default_rng(700 + seed)
    return {f"r{i}": random_tokens(rng, n, cfg["vocab"]) for i, n in enumerate(lens)}


def test_the_sharpened_models_use_what_they_have(model):
    """The tests below mean something only if a window's edge, the cap, the scan's memory and the routed weights
    change the logits by far more than the tolerances: the plain implementation with each of them changed differs."""
    name, _, cfg, W = model
    toks = requests_for(cfg, lens=(60,), seed=1)["r0"]
    ref = plain(name, cfg, W, toks)
    big = np.abs(ref).max()
    differs = lambda other_cfg, other_W=W: np.abs(P.forward(other_cfg, other_W, toks).numpy() - ref).max()
    for i, layer in enumerate(cfg["layers"]):
        mixers = [layer["mixer"]] if layer["type"] == "attention" else [layer["mixer"]["left"]]
        for m in mixers:
            size = (m.get("mask") or {}).get("size")
            other = copy.deepcopy(cfg)
            om = other["layers"][i]["mixer"] if layer["type"] == "attention" else other["layers"][i]["mixer"]["left"]
            if size and size < 60:
                om["mask"]["size"] = size + 1
                assert differs(other) > 50 * TOL["float32"] * big, (i, "window")
                om["mask"]["size"] = size
            if m.get("softcap") and size != 1:          # a window of one token: its only score weighs 1 whatever it is
                om["softcap"] = 3.0 * m["softcap"]
                assert differs(other) > 50 * TOL["float32"] * big, (i, "softcap")
        if layer["type"] == "parallel":
            # a scan that forgot what it carried: the state's decays set to forget at once
            W2 = dict(W)
            W2[f"l{i}.mix.right.A_log"] = torch.full_like(W[f"l{i}.mix.right.A_log"], 6.0)
            assert differs(cfg, W2) > 0.01 * big, (i, "state")
            if layer["mixer"]["right"]["conv"] > 1:
                W2 = dict(W)
                W2[f"l{i}.mix.right.conv"] = W[f"l{i}.mix.right.conv"].clone()
                W2[f"l{i}.mix.right.conv"][:, 0] = 0
                assert differs(cfg, W2) > 0.003 * big, (i, "oldest tap")
        if layer.get("mlp") and layer["mlp"]["router"]["experts"] > 1:
            W2 = dict(W)
            W2[f"l{i}.mlp.router"] = -W[f"l{i}.mlp.router"].float()
            assert differs(cfg, W2) > 0.01 * big, (i, "router")


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_requests_alone(model, dtype):
    eng = build(model[1], dtype)
    reqs = requests_for(model[2])
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_whole(rid, toks)))
    check(got, model, reqs, dtype)
    assert all_pages_free(eng, 64)


def pending_name(layer):
    """The workspace tensor that holds what a layer's last sublayer left for the next norm to add."""
    if layer.get("mlp"):
        return "moe.out"
    return "rot_attn.o" if layer["type"] == "attention" else "side.out"


def test_the_stream_after_every_layer(model):
    """float32, layer by layer: the engine's model is cut off behind its first k run steps and its stream
    compared with the plain one's."""
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
        x = x + eng.workspace.get(pending_name(cfg["layers"][k - 1]), len(toks), cfg["width"], torch.float32).cpu().double()
        eng.close_request(slot)
        want = streams[k - 1]
        assert (x - want).abs().max() <= 2e-5 * want.abs().max(), (name, k, float((x - want).abs().max()))
    object.__setattr__(eng.model.spec, "run_order", order)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_then_token_by_token(model, dtype):
    """Most of a prompt in one step, the rest decoded one by one (replayed from CUDA graphs): windows pass over
    decoded tokens, pages behind them are given back, the scan's state and carried inputs go from step to step."""
    eng = build(model[1], dtype)
    reqs = {k: v for k, v in requests_for(model[2]).items() if len(v) >= 33}
    got = {}
    for rid, toks in reqs.items():
        got.update(replay(eng, cut_bulk_tail(rid, toks, 32)))
    check(got, model, reqs, dtype)
    assert eng.graph_replays > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_token_at_a_time_from_the_start(model, dtype):
    """The first tokens of a sequence: a convolution with nothing but zeros before it, a state that starts at zero."""
    eng = build(model[1], dtype)
    reqs = requests_for(model[2], lens=(45,), seed=2)
    got = replay(eng, cut_bulk_tail("r0", reqs["r0"], 44))
    check(got, model, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page_size", [4, 16])
def test_portions_of_changing_size(model, dtype, page_size):
    """Portions down to two tokens (shorter than the convolution's taps), cut in the middle of pages, of key
    blocks, of windows and of the scan's chunks."""
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
    """Up to four live requests: portions of some beside single tokens of others; requests end and new ones take
    their slots (whose state must start at zero again) and pages (few pages, so the page freed last is used next)."""
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
    assert reused > 0 and all_pages_free(eng, 24)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model, dtype):
    """300 tokens, the last 260 one by one: pages fill, windows move on and their pages turn over, the state is
    renewed 260 times."""
    reqs = requests_for(model[2], lens=(300,), seed=3)
    eng = build(model[1], dtype, num_pages=24, page_size=16)
    got = replay(eng, cut_bulk_tail("r0", reqs["r0"], 260))
    check(got, model, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_in_portions(model, dtype):
    """700 tokens in portions of 48: the later portions stand behind hundreds of cached keys, most of them
    behind the window and their pages gone, and behind a state that 600 tokens have written."""
    if model[0] == "odd":
        pytest.skip("one configuration of each kernel is enough")
    reqs = requests_for(model[2], lens=(700,), seed=6)
    eng = build(model[1], dtype, num_pages=48, page_size=16)
    got = replay(eng, cut_portions("r0", reqs["r0"], sizes=(48,)))
    check(got, model, reqs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_in_one_step(model, dtype):
    """900 tokens at once, beside a short request: steps of many tokens run the experts' products in whole tiles on
    the tensor-memory kernel (bfloat16), the attention's row tiles stand behind hundreds of keys of their own step,
    and the scan walks 57 chunks."""
    reqs = requests_for(model[2], lens=(900, 40), seed=8)
    eng = build(model[1], dtype, num_pages=72, page_size=16, max_batch_tokens=1024)
    got = replay(eng, [{"entries": [("r1", reqs["r1"], list(range(40))), ("r0", reqs["r0"], list(range(900)))],
                        "end": ["r0", "r1"]}])
    check(got, model, reqs, dtype)
    assert all_pages_free(eng, 72)


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
    """A step that is refused after another one ran: the state of the slot and the pages are as before."""
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


def _paged(keys, page_size, order, dtype, dev, first_kept=0):
    """keys [L, heads, d] -> (pool [pages, heads, page_size, d], table); pages wholly before ``first_kept``
    are not stored and their table entries are -1, as a window group leaves them."""
    L, H, d = keys.shape
    n = (L + page_size - 1) // page_size
    pool = torch.zeros(len(order), H, page_size, d, dtype=dtype, device=dev)
    table = []
    for i in range(n):
        if (i + 1) * page_size <= first_kept:
            table.append(-1)
            continue
        chunk = keys[i * page_size:(i + 1) * page_size]
        pool[order[i], :, :chunk.shape[0]] = chunk.transpose(0, 1).to(dtype)
        table.append(order[i])
    return pool, torch.tensor([table], dtype=torch.int32, device=dev)


@pytest.mark.parametrize("cache_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,dv,heads,kv_heads,window,cap", [(24, 40, 4, 2, 100, 3.0), (48, 80, 6, 3, 37, None), (16, 16, 2, 1, 0, 5.0),
                                                             (32, 64, 4, 2, 64, 2.5), (64, 128, 8, 2, 129, 4.0), (48, 64, 3, 3, 33, 30.0),
                                                             (128, 128, 4, 2, 75, 3.5), (128, 128, 2, 2, 0, 6.0)])
def test_attention_kernel_cap_and_window_edges(cache_dtype, dk, dv, heads, kv_heads, window, cap):
    """Queries aimed at one key each, with scores far above the cap: just inside the window, just outside it (where
    a heavier key waits), far back, at page borders and at position 0.  A window one token off, a cap that is left
    out or applied to the unscaled score, or a page that was given back and read all the same changes the result
    by far more than the tolerance."""
    from safetyraise_lmengine_b200.kernels import ops
    dev, L, page = "cuda:0", 700, 16
    g = torch.Generator().manual_seed(dk * 100 + dv)
    q = 0.5 * torch.randn(L, heads, dk, generator=g)
    k = torch.randn(L, kv_heads, dk, generator=g)
    v = torch.randn(L, kv_heads, dv, generator=g)
    if cache_dtype == torch.bfloat16:
        k, v = k.bfloat16().float(), v.bfloat16().float()
    rep = heads // kv_heads
    aim = lambda row, col, f: q.__setitem__(row, f * k[col].repeat_interleave(rep, 0)
                                            / k[col].norm(dim=-1, keepdim=True).repeat_interleave(rep, 0))
    w = window or L
    pairs = [(L - 1, L - w), (L - 2, L - 2 - w), (L - 3, max(0, L - 3 - w + 1)), (650, 650 - min(w, 650) + 1), (651, 640), (40, 0), (600, 592)]
    for row, col in pairs:
        if col >= 0:
            aim(row, col, 9.0)
    scale = 0.9
    m = {"heads": heads, "kv_heads": kv_heads, "vdim": dv, "scale": scale}
    if cap:
        m["softcap"] = cap
    if window:
        m["mask"] = {"size": window}
    ref = P.attend(q.double(), k.double(), v.double(), m).view(L, heads, dv)
    if cap:
        uncapped = P.attend(q.double(), k.double(), v.double(), {k_: v_ for k_, v_ in m.items() if k_ != "softcap"}).view(L, heads, dv)
        assert (ref - uncapped).abs().max() > 0.05
    if window:
        off = P.attend(q.double(), k.double(), v.double(), dict(m, mask={"size": window + 1})).view(L, heads, dv)
        assert (ref[L - 2] - off[L - 2]).abs().max() > 0.05          # the key just outside would be seen
    order = list(reversed(range(L // page + 2)))
    tol = 2e-5 if cache_dtype == torch.float32 else 2e-2
    for q_lens in ([L], [1], [2], [3], [33], [130]):             # a whole prompt, decoded tokens, portions
        n = q_lens[0]
        first_kept = max(0, L - n - w + 1) if window else 0          # what a window group still holds before this step
        k_pool, table = _paged(k, page, order, cache_dtype, dev, first_kept)
        v_pool = _paged(v, page, order, cache_dtype, dev, first_kept)[0]
        out = torch.zeros(n, heads * dv, dtype=torch.float32, device=dev)
        ops.paged_attention_general(_Ctx(q_lens, [L], dev), q[L - n:].reshape(n, -1).contiguous().to(dev), k_pool, v_pool,
                                    out, table, None, heads, kv_heads, dk, dv, scale, window, softcap=cap)
        err = (out.cpu().double().view(n, heads, dv) - ref[L - n:]).abs().max() / ref.abs().max()
        assert err < tol, (q_lens, float(err))
        ctx = _Ctx(q_lens, [L], dev)
        if (cap and cache_dtype == torch.bfloat16 and dk == dv and n > 4
                and ops.sinks_on_tcgen05(ctx, cache_dtype, heads, kv_heads, dk, dv, page)):
            # heads of 128: the tensor-memory kernel, queries in bfloat16
            out16 = torch.zeros(n, heads * dv, dtype=torch.bfloat16, device=dev)
            ops.paged_attention(ctx, q[L - n:].reshape(n, -1).contiguous().to(dev).bfloat16(), k_pool, v_pool, out16, table,
                                heads, kv_heads, dk, page, scale, window, mods=(None, None, None, cap))
            err = (out16.cpu().double().view(n, heads, dv) - ref[L - n:]).abs().max() / ref.abs().max()
            assert err < tol, ("tensor memory", q_lens, float(err))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
def test_bias_rotation_and_append(dtype, interleaved):
    """q | k | v rows get their biases, q and k heads are turned on their first dims elements by the positions'
    angles (the rest of a head and v pass as they are), k and v land in the pages' slots: against the plain
    rotation, at positions far from zero, with rescaled frequencies, for a layer that projects q alone too."""
    from safetyraise_lmengine_b200.kernels import ops
    from safetyraise_lmengine_b200.parts.base import Rotation
    from safetyraise_lmengine_b200.parts.position import rescaled_frequencies
    dev = "cuda:0"
    g = torch.Generator().manual_seed(5)
    for T, nq, nkv, dk, dv, dims, bias, scaling in ((7, 4, 2, 24, 40, 8, True, None), (3, 1, 1, 10, 7, 10, False, (4.0, 1.0, 4.0, 32.0)),
                                                    (40, 6, 2, 48, 80, 48, True, (8.0, 1.0, 2.0, 100.0)), (5, 2, 2, 128, 128, 64, False, None)):
        rot = {"dims": dims, "base": 300.0}
        if scaling:
            rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
        positions = torch.tensor([1000 + 37 * t for t in range(T)])
        freq = torch.tensor(rescaled_frequencies(300.0, dims, scaling), dtype=torch.float64)
        ang = positions.double()[:, None] * freq[None, :]
        rotation = Rotation(torch.cos(ang).float().to(dev), torch.sin(ang).float().to(dev), dims // 2, interleaved=interleaved)
        width = nq * dk + nkv * (dk + dv)
        proj = 3 * torch.randn(T, width, generator=g)
        b = torch.randn(width, generator=g) if bias else None
        slots = torch.randperm(64, generator=g)[:T].to(torch.int32)
        kp = torch.zeros(4, nkv, 16, dk, dtype=dtype, device=dev)
        vp = torch.zeros(4, nkv, 16, dv, dtype=dtype, device=dev)
        q = torch.zeros(T, nq * dk, device=dev)
        ops.attention_bias_append(proj.to(dev), b.to(dev) if bias else None, q, kp, vp, slots.to(dev), nq, nkv, dk, dv,
                                  rotation=rotation)
        full = proj.double() + (b.double() if bias else 0)

        def turned(x, heads):           # the plain rotation, one token at a time at its own position
            return torch.cat([P.rotate(x[t:t + 1].view(1, heads, dk), rot, interleaved, first_position=int(positions[t]))
                              for t in range(T)])
        want_q = turned(full[:, :nq * dk], nq)
        want_k = turned(full[:, nq * dk:(nq + nkv) * dk], nkv)
        want_v = full[:, (nq + nkv) * dk:].view(T, nkv, dv)
        assert (want_q - full[:, :nq * dk].view(T, nq, dk)).abs().max() > 0.5          # the rotation does something
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert (q.cpu().double().view(T, nq, dk) - want_q).abs().max() < 3e-5 * want_q.abs().max()
        for t in range(T):
            page, off = int(slots[t]) // 16, int(slots[t]) % 16
            assert (kp[page, :, off].cpu().double() - want_k[t]).abs().max() < tol * want_k.abs().max()
            assert (vp[page, :, off].cpu().double() - want_v[t]).abs().max() < tol * want_v.abs().max()
        # a layer without keys and values of its own: the q columns alone, nothing written
        kp2, q2 = kp.clone(), torch.zeros_like(q)
        ops.attention_bias_append(proj[:, :nq * dk].contiguous().to(dev), b[:nq * dk].contiguous().to(dev) if bias else None, q2,
                                  kp2, vp, slots.to(dev), nq, nkv, dk, dv, write_kv=False, rotation=rotation)
        assert torch.equal(q2, q) and torch.equal(kp2, kp)


def _plain_scan(xz, W, N, R, taps):
    """The plain scan's steps on given inputs of the convolution and gates: -> (x behind the convolution, y gated)."""
    C = xz.shape[1] // 2
    x = P.silu(P.causal_conv(xz[:, :C], W["conv"], W["conv.b"]))
    dbc = x @ W["x"].double().T
    dt = P.softplus(dbc[:, :R] @ W["dt"].double().T + W["dt.b"].double())
    A = -torch.exp(W["A_log"].double())
    S = torch.zeros(C, N, dtype=torch.float64)
    ys = []
    for t in range(xz.shape[0]):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * dbc[t, R:R + N][None, :]
        ys.append(S @ dbc[t, R + N:R + 2 * N] + W["D"].double() * x[t])
    return x, torch.stack(ys) * P.silu(xz[:, C:].double()), dbc, dt


@pytest.mark.parametrize("C,N,R,taps", [(40, 6, 3, 4), (27, 1, 1, 1), (64, 16, 4, 2), (33, 24, 5, 3), (16, 128, 2, 4), (130, 40, 7, 6)])
def test_convolution_and_scan_carried_through_steps_and_slots(C, N, R, taps):
    """Two requests in slots used before (left full of other numbers, zeroed as the engine does for a new
    occupant), cut into steps of unequal sizes down to one token (shorter than the taps) and run side by side:
    against the plain recurrence over each whole sequence.  One channel keeps a large first token for hundreds
    of steps (a decay near one), one forgets within a step: a state that is lost, zeroed at the wrong time or
    mixed up between slots, or a carried input that is dropped, shows."""
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(C * 7 + N)
    rnd = lambda *s: torch.randn(*s, generator=g)
    W = {"conv": 0.6 * rnd(C, taps), "conv.b": 0.3 * rnd(C), "x": 0.4 * rnd(R + 2 * N, C) / C ** 0.5 * 4, "dt": 1.5 * rnd(C, R) / R ** 0.5,
         "dt.b": -5 + 6 * torch.rand(C, generator=g), "A_log": -4 + 5.2 * torch.rand(C, N, generator=g), "D": rnd(C)}
    W["A_log"][0] = -9.0          # channel 0 forgets next to nothing
    W["dt.b"][0] = 0.5
    W["A_log"][1] = 3.0           # channel 1 forgets at once
    lens = {"a": 330, "b": 75}
    xz = {r: rnd(n, 2 * C) for r, n in lens.items()}
    xz["a"][0, 0] = 25.0          # a large first input of the channel that remembers
    want = {r: _plain_scan(xz[r].double(), W, N, R, taps) for r in lens}
    without = xz["a"].double().clone()
    without[0, 0] = 0.0
    far = (want["a"][1][300:, 0] - _plain_scan(without, W, N, R, taps)[1][300:, 0]).abs().max()
    assert far > 0.05              # the first token still shows 300 steps later
    state = torch.randn(5, C * (N + taps - 1) + 3, generator=g).to(dev)          # rows longer than the state: a stride
    slot_of = {"a": 3, "b": 1}
    for s in slot_of.values():
        state[s].zero_()
    d = lambda t: t.float().to(dev).contiguous()
    A_dev = d(-torch.exp(W["A_log"].double()))
    cuts = {"a": [200, 1, 1, 2, 17, 1, 60, 3, 45], "b": [1, 2, 1, 30, 16, 1, 1, 20, 3]}
    assert all(sum(c) == lens[r] for r, c in cuts.items())
    fed = {r: 0 for r in lens}
    got = {r: [] for r in lens}
    for step in range(9):
        order = ["a", "b"] if step % 2 == 0 else ["b", "a"]
        q_lens = [cuts[r][step] for r in order]
        ctx = _Ctx(q_lens, q_lens, dev, slots=[slot_of[r] for r in order])
        rows = torch.cat([xz[r][fed[r]:fed[r] + cuts[r][step]] for r in order])
        T = rows.shape[0]
        x_out, y = torch.zeros(T, C, device=dev), torch.zeros(T, C, device=dev)
        xz_dev = d(rows)
        ops.scan_conv(ctx, xz_dev, d(W["conv"]), d(W["conv.b"]), state, x_out, None, C, N, taps)
        # the projections behind the convolution are not this test's matter: the plain ones, on the kernel's x
        dbc = x_out.double() @ W["x"].double().T.to(dev)
        dt_raw = (dbc[:, :R] @ W["dt"].double().T.to(dev)).float().contiguous()
        ops.selective_scan(ctx, x_out, xz_dev, dbc.float().contiguous(), R, dt_raw, d(W["dt.b"]), A_dev, d(W["D"]), state, y, C, N, taps)
        at = 0
        for r in order:
            n = cuts[r][step]
            got[r].append((x_out[at:at + n].cpu().double(), y[at:at + n].cpu().double()))
            at += n
            fed[r] += n
    for r in lens:
        x_got, y_got = torch.cat([p[0] for p in got[r]]), torch.cat([p[1] for p in got[r]])
        assert (x_got - want[r][0]).abs().max() < 2e-5 * want[r][0].abs().max(), r
        err = (y_got - want[r][1]).abs().max(dim=1).values / want[r][1].abs().max()
        assert err.max() < 5e-5, (r, int(err.argmax()), float(err.max()))
        if r == "a":
            assert (y_got[300:, 0] - want[r][1][300:, 0]).abs().max() < 1e-2 * far
    # the other slots were not touched
    assert torch.isfinite(state).all()


def test_two_normed_results_averaged():
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(3)
    for T, H in ((5, 36), (3, 328), (17, 1000), (2, 4096)):
        a, b = 7 * torch.randn(T, H, generator=g), 0.01 * torch.randn(T, H, generator=g)      # unequal sizes: each its own RMS
        wa, wb = torch.rand(H, generator=g) + 0.5, torch.randn(H, generator=g)
        want = 0.5 * (P.rms_norm(a, wa, 1e-5) + P.rms_norm(b, wb, 1e-5))
        for out_dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
            out = torch.zeros(T, H, dtype=out_dtype, device=dev)
            ops.paired_rmsnorm_mean(a.to(dev), wa.to(dev), b.to(dev), wb.to(dev), 1e-5, out)
            assert (out.cpu().double() - want).abs().max() < tol * want.abs().max()


def test_logistic_router_choice_and_weights():
    """The chosen experts are those of the largest scores, a tie goes to the lower index, and the weights are the
    chosen scores themselves: they do not sum to one."""
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(8)
    for T, E, top in ((9, 6, 2), (5, 3, 3), (33, 70, 8), (4, 2, 1), (3, 1, 1)):
        z = 2 * torch.randn(T, E, generator=g)
        if E >= 6:
            z[0, 4] = z[0, 1] = 9.0
        choice = torch.zeros(T, top, dtype=torch.int32, device=dev)
        weight = torch.zeros(T, top, device=dev)
        ops.moe_route(z.to(dev), None, top, choice, weight, scoring="logistic")
        val, idx = torch.sigmoid(z.double()).topk(top, dim=-1)
        if E >= 6:
            assert choice[0, :2].tolist() == [1, 4]
            idx[0, :2] = torch.tensor([1, 4])
        assert torch.equal(choice.cpu().long(), idx)
        assert (weight.cpu().double() - val).abs().max() < 1e-6
        if top > 1:
            assert (weight.sum(-1) - 1).abs().max() > 0.05
        # the same from columns of a wider tensor, routed by the block that orders the pairs
        wide = torch.cat([torch.randn(T, 5, generator=g), z, torch.randn(T, 2, generator=g)], dim=1).to(dev)
        choice2, weight2 = torch.zeros_like(choice), torch.zeros_like(weight)
        heads = torch.zeros(2, E + 1, dtype=torch.int32, device=dev)
        por, rop = torch.zeros(T * top, dtype=torch.int32, device=dev), torch.zeros(T * top, dtype=torch.int32, device=dev)
        assert ops.moe_sort_routes(T, E)
        ops.moe_sort(choice2, E, heads[0], heads[1], por, rop, route=(wide, 5, None, weight2), scoring="logistic")
        assert torch.equal(choice2, choice) and torch.equal(weight2, weight)


def _experts_plain(x, gu, dn, choice, weight, add):
    """sum over a token's choices of expert(weight * x), plus what is to be added."""
    ff = gu.shape[1] // 2
    want = add.double().clone()
    for t in range(x.shape[0]):
        for c in range(choice.shape[1]):
            e = int(choice[t, c])
            W = {"gate": gu[e, :ff], "up": gu[e, ff:], "down": dn[e]}
            want[t] += P.expert(weight[t, c].double() * x[t:t + 1].double(), W, "")[0]
    return want


@pytest.mark.parametrize("dtype,interleaved", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
def test_experts_with_the_weight_on_their_input(dtype, interleaved):
    """Both grouped products and the combination with the weight ahead of the activation, against loops over tokens:
    weights far from one, so that a weight on the output instead (the activation is not linear) shows; an expert
    nobody chose, an expert with more rows than a tile, one token, sizes that are no multiple of anything."""
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(12)
    sizes = ((150, 5, 2, 40, 24), (1, 4, 4, 36, 9), (70, 9, 1, 64, 32), (33, 3, 3, 24, 130))
    if interleaved:
        sizes = ((150, 5, 2, 40, 24), (1, 4, 4, 72, 8), (300, 9, 1, 64, 200), (33, 3, 3, 264, 136), (70, 2, 2, 36, 16))
    for T, E, top, H, ff in sizes:
        x = torch.randn(T, H, generator=g).to(dtype)
        gu = (0.5 * torch.randn(E, 2 * ff, H, generator=g)).to(dtype)
        dn = (0.3 * torch.randn(E, H, ff, generator=g)).to(dtype)
        choice = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
        if E == 5:
            choice[choice == 3] = 0
            choice[:, 1] = torch.where(choice[:, 0] == 4, 1, 4)
        weight = 0.15 + 0.8 * torch.rand(T, top, generator=g)
        add = torch.randn(T, H, generator=g).to(dtype)
        n = T * top
        d = lambda t: t.to(dev)
        offsets, tiles = torch.zeros(E + 1, dtype=torch.int32, device=dev), torch.zeros(E + 1, dtype=torch.int32, device=dev)
        por, rop = torch.zeros(n, dtype=torch.int32, device=dev), torch.zeros(n, dtype=torch.int32, device=dev)
        ops.moe_sort(d(choice), E, offsets, tiles, por, rop)
        y = torch.zeros(n, ff, dtype=dtype, device=dev)
        gu_dev = d(gu)
        if interleaved:        # blocks of 16 rows: 8 gate rows, then the 8 up rows of the same features
            gu_dev = torch.stack([gu_dev[:, :ff].reshape(E, ff // 8, 8, H), gu_dev[:, ff:].reshape(E, ff // 8, 8, H)],
                                 dim=2).reshape(E, 2 * ff, H).contiguous()
        ops.moe_grouped(d(x), por, top, gu_dev, y, offsets, tiles, glu=True, interleaved=interleaved, limit=0.0, alpha=1.0,
                        pair_scale=d(weight))
        rows = torch.zeros(n, H, device=dev)
        ops.moe_grouped(y, None, 1, d(dn), rows, offsets, tiles)
        out = torch.zeros(T, H, dtype=dtype, device=dev)
        ops.moe_combine(rows, rop.view(T, top), None, d(add), out)
        want = _experts_plain(x, gu, dn, choice, weight, add)
        on_output = add.double().clone()
        for t in range(T):
            for c in range(top):
                e = int(choice[t, c])
                on_output[t] += weight[t, c].double() * P.expert(x[t:t + 1], {"gate": gu[e, :ff], "up": gu[e, ff:], "down": dn[e]}, "")[0]
        assert (want - on_output).abs().max() > 0.05 * want.abs().max()
        err = (out.cpu().double() - want).abs().max() / want.abs().max()
        assert err < (2e-5 if dtype == torch.float32 else 2e-2), (T, E, top, float(err))


@pytest.mark.parametrize("tile", [128, 256])
def test_experts_in_tiles_of_tensor_memory_with_the_weight_on_their_input(tile):
    """Steps of many tokens: the gathered rows are scaled by their pair's weight, both products run on the persistent
    tensor-memory kernel with the plain gated activation in the first one's epilogue."""
    from safetyraise_lmengine_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(14)
    for T, E, top, H, ff in ((700, 5, 2, 64, 48), (130, 3, 1, 136, 200), (512, 4, 4, 256, 128)):
        x = torch.randn(T, H, generator=g).bfloat16()
        gu = (0.4 * torch.randn(E, 2 * ff, H, generator=g)).bfloat16()
        dn = (0.3 * torch.randn(E, H, ff, generator=g)).bfloat16()
        choice = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
        weight = 0.15 + 0.8 * torch.rand(T, top, generator=g)
        n = T * top
        n_tiles = n // tile + E
        d = lambda t: t.to(dev)
        heads = torch.zeros(2, E + 1, dtype=torch.int32, device=dev)
        group = torch.full((n_tiles,), -7, dtype=torch.int32, device=dev)
        por = torch.full((n_tiles * tile,), -7, dtype=torch.int32, device=dev)
        rop = torch.zeros(n, dtype=torch.int32, device=dev)
        ops.moe_sort(d(choice), E, heads[0], heads[1], por, rop, tile_rows=tile, group_of_tile=group)
        gu_dev = torch.stack([d(gu)[:, :ff].reshape(E, ff // 8, 8, H), d(gu)[:, ff:].reshape(E, ff // 8, 8, H)],
                             dim=2).reshape(E, 2 * ff, H).contiguous()
        xs = torch.empty(n_tiles * tile, H, dtype=torch.bfloat16, device=dev)
        ops.moe_gather_rows(d(x), por, top, xs, pair_scale=d(weight))
        y = torch.zeros(n_tiles * tile, ff, dtype=torch.bfloat16, device=dev)
        ops.gemm_tn_tcgen05_grouped(xs, gu_dev, y, group, glu=True, limit=0.0, alpha=1.0, tile_rows=tile)
        rows = torch.zeros(n_tiles * tile, H, device=dev)
        ops.gemm_tn_tcgen05_grouped(y, d(dn), rows, group, tile_rows=tile)
        out = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
        ops.moe_combine(rows, rop.view(T, top), None, None, out)
        assert ops.gemm_error_flag(torch.device(dev)) == 0
        want = _experts_plain(x, gu, dn, choice, weight, torch.zeros(T, H))
        err = (out.cpu().double() - want).abs().max() / want.abs().max()
        assert err < 2e-2, (T, E, top, float(err))


# ---- as a user runs it: the command line and the trace replay ---------------------------------------------------

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
    assert info["spec"]["architecture"] == "Pabalorn"
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
    rng = np.random.default_rng(3000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    width = pick(40, 64, 96, 128, 160)
    layers, owners = [], []

    def some_mlp():
        if rng.random() < 0.25:
            return None
        experts = pick(2, 3, 5, 8, 12)
        return moe(experts=experts, top=int(rng.integers(1, min(experts, 4) + 1)), ff=pick(8, 16, 24, 40, 50))

    for i in range(int(rng.integers(2, 7))):
        if rng.random() < 0.45:
            kv = pick(1, 2, 3)
            dim, vdim = pick((8, 8), (16, 40), (24, 16), (32, 64), (64, 64), (128, 128), (48, 80), (80, 56))
            rot = pick(None, 2, dim // 2, dim)
            layers.append(pair(heads=kv * pick(1, 2, 4), kv_heads=kv, dim=dim, vdim=vdim, window=pick(None, 1, 9, 40, 129),
                               rot=rot if rot is None or rot % 2 == 0 else rot - 1, base=pick(50.0, 10000.0),
                               scaling=pick(None, (4.0, 1.0, 4.0, 64), (16.0, 0.5, 3.0, 200)),
                               inner=pick(12, 40, 96, 130), state=pick(1, 4, 16, 20, 48), dt_rank=pick(1, 3, 8), conv=pick(1, 2, 4),
                               mlp=some_mlp()))
        elif owners and rng.random() < 0.35:
            j = owners[int(rng.integers(len(owners)))]
            m = {k: v for k, v in layers[j]["mixer"].items()}
            reader = {"type": "attention", "mixer": dict(m, kv_from=j), "mlp": some_mlp()}
            window = pick(None, 3, 20, 75, 300)
            reader["mixer"].pop("mask", None)
            if window:
                reader["mixer"]["mask"] = {"size": window}
            reader["mixer"]["softcap"] = pick(2.0, 30.0)
            layers.append(reader)
        else:
            kv = pick(1, 2, 3)
            dim, vdim = pick((8, 8), (16, 40), (24, 16), (32, 64), (64, 64), (128, 128), (48, 128), (80, 56))
            layers.append(att(heads=kv * pick(1, 2, 4), kv_heads=kv, dim=dim, vdim=vdim, window=pick(None, 1, 9, 16, 50, 129, 1000),
                              softcap=pick(None, 2.0, 8.0, 30.0), rot=pick(None, 2, dim // 2 - (dim // 2) % 2, dim),
                              base=pick(100.0, 20000.0), mlp=some_mlp()))
            owners.append(len(layers) - 1)
    return config(layers, width=width, vocab=pick(97, 160, 301), eps=pick(1e-6, 1e-5, 1e-4))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Whatever the order of layers and the sizes: float32 within the tolerance at every position under a cutting
    with portions, decoded tokens and a second request beside it; bfloat16 by the rule of `check`."""
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
