"""The Petelix design on the GPU against the plain implementation
(tests/plain_petelix.py): every mechanism alone, then whole models through the
engine's step function, cut and batched in every way, then greedy generation
through the scheduler.

Where both compute dtypes run: float32 must match every row; in bfloat16 a
router choice at a near tie may flip under the rounding of the router's
input, which changes that token's row (and, faintly, later ones), so whole
models are held to "nearly all rows" there.  Mechanisms alone are given inputs
without such ties and are held to every row in both.
"""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_petelix as plain
from helpers import run_trace_on_engine, trace_mixed, trace_portions, trace_tail_decoded, trace_whole
from petelix_helpers import (CFG_A, CFG_B, CFG_C, CFG_D, CONFIGS, attention_params, build, make_weights, random_config,
                             routed_params)
from potivik_helpers import PartHarness, ids_for, make_part, rel_rows

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-4, "bfloat16": 4e-2}
DEV = "cuda:0"
F64 = torch.float64


def gen(seed):
    return torch.Generator().manual_seed(seed)


def bf(t):
    return t.to(torch.bfloat16).to(torch.float32)


def dbl(W):
    return {k: v.double() for k, v in W.items()}


def check_rows(got, want, dtype: str, strict: bool = True, what: str = ""):
    e = rel_rows(got, want)
    if strict or dtype == "float32":
        assert e.max() <= TOL[dtype], f"{what}: row {int(e.argmax())} differs by {e.max():.3g} (tolerance {TOL[dtype]})"
    else:
        frac = float((e > TOL[dtype]).mean())
        assert frac <= 0.45 and np.median(e) <= 0.75 * TOL[dtype], \
            f"{what}: {frac:.1%} of the rows differ by more than {TOL[dtype]} (median {np.median(e):.3g})"


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("scale", [1.0, 0.37, 12.0])
def test_embedding_with_a_scale(dtype, scale):
    from gibbs_b200.engine.step import StepState
    g = gen(1)
    V, d = 77, 52
    table = bf(torch.randn(V, d, generator=g))
    part = make_part("embedding", "token_embedding", {"vocab": V, "dim": d, "scale": scale}, {"weight": table}, DTYPES[dtype])
    ids = torch.randint(0, V, (33,), generator=g)
    out = part.forward(ids.to(DEV, torch.int32)).cpu()
    assert out.dtype == torch.float32
    assert rel_rows(out, table[ids].double() * scale).max() < 1e-6


def _plain_mixer(h, W, m, eps):
    pos = torch.arange(h.shape[0])
    return plain.attention_mixer(h.double(), dbl(W), m, eps, pos, None)[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg,layer", [(CFG_A, 0), (CFG_A, 2), (CFG_B, 0), (CFG_B, 1), (CFG_C, 0), (CFG_C, 1),
                                       (CFG_D, 0), (CFG_D, 2), (CFG_D, 3), (CFG_D, 4)])
def test_attention_alone_whole_cut_and_decoded(cfg, layer, dtype):
    m, d, eps = cfg["layers"][layer]["mixer"], cfg["width"], cfg["norm"]["eps"]
    W = plain.sub(make_weights(cfg, 5), f"l{layer}.mix.")
    part = make_part("mixer", "gated_attention", attention_params(m, d, eps), W, DTYPES[dtype])
    T = 150
    h = bf(torch.randn(T, d, generator=gen(6)))
    want = _plain_mixer(h, W, m, eps)
    # the sink shows: the first tokens see few keys, and their weights do not add up to one
    no_sink = _attention_without_sink(h, W, m, eps)
    assert rel_rows(no_sink[:3], want[:3]).max() > 0.05
    hz = PartHarness(part, n_pages=12, page_size=16, fill=0.0)      # 12 pages: 192 positions, pages come back and go out again
    for rid, cuts in (("whole", [T]), ("cut", [2, 3, 17, 2, 31, 16, 1, 5, 64, 7]), ("decoded", [T - 45, 1])):
        got = hz.run_cut(rid, h, cuts)
        check_rows(got, want, dtype, what=f"attention, {rid}")
        hz.close(rid)


def _attention_without_sink(h, W, m, eps):
    """The same mixer with an ordinary softmax, to show that a test's inputs tell the two apart."""
    Wd, pos = dbl(W), torch.arange(h.shape[0])
    H, dim = m["heads"], m["dim"]
    rot = m.get("rot") or {}
    q = plain.rotate_pairs(plain.rms_norm(h.double() @ Wd["q"].T, Wd["q.norm"], eps).reshape(-1, H, dim), pos,
                           rot.get("base", 1.0), int(rot.get("dims", 0)))
    k, v = plain.keys_and_values(h.double(), Wd, m, eps, pos)
    T, G = h.shape[0], m["kv_heads"]
    out = torch.zeros(T, H, m["vdim"], dtype=F64)
    w = (m.get("mask") or {}).get("size")
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd // (H // G)].T) * m["scale"]
        if m.get("softcap"):
            s = m["softcap"] * torch.tanh(s / m["softcap"])
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        seen = (j <= i) & ((i - j < w) if w else True)
        out[:, hd] = torch.softmax(s.masked_fill(~seen, -math.inf), -1) @ v[:, hd // (H // G)]
    o = out.reshape(T, -1) * torch.sigmoid(h.double() @ Wd["g"].T)
    return o @ Wd["o"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_norm_is_over_the_whole_projection_and_the_cap_bends_large_scores(dtype):
    """Heads of very unequal size and scores far beyond the cap: a norm per head, or no cap, gives other rows."""
    d, eps = 48, 1e-5
    m = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 2.0, "softcap": 3.0, "mask": {"size": 50},
         "rot": {"base": 100.0, "dims": 4}}
    g = gen(31)
    W = {"q": torch.randn(32, d, generator=g) / 7, "k": torch.randn(16, d, generator=g) / 7, "v": torch.randn(16, d, generator=g) / 5,
         "q.norm": 1 + 0.2 * torch.randn(32, generator=g), "k.norm": 1 + 0.2 * torch.randn(16, generator=g),
         "g": torch.randn(32, d, generator=g) / 5, "o": torch.randn(d, 32, generator=g) / 6}
    W["q"][:8] *= 9.0                                          # head 0 carries nearly all of the projection's mean square
    W["k"][8:] *= 5.0
    W = {k: bf(v) for k, v in W.items()}
    h = bf(torch.randn(70, d, generator=g))
    want = _plain_mixer(h, W, m, eps)
    uncapped = _plain_mixer(h, W, {**m, "softcap": None}, eps)
    assert np.median(rel_rows(uncapped, want)) > 0.05
    q = h.double() @ W["q"].double().T
    per_head = plain.rms_norm(q.reshape(-1, 4, 8), 1.0, eps).reshape(-1, 32)
    assert rel_rows(per_head, plain.rms_norm(q, 1.0, eps)).max() > 0.5
    part = make_part("mixer", "gated_attention", attention_params(m, d, eps), W, DTYPES[dtype])
    hz = PartHarness(part, fill=0.0)
    check_rows(hz.run_cut("a", h, [33, 2, 1]), want, dtype, what="unequal heads, capped scores")


def _pointed_attention(window, T, hot_key, query, vdim=8, seed=7):
    """Weights and inputs for which the query position's score against ``hot_key`` stands far above all
    others (when that key is visible), and whose values tell keys apart.  Keys read the input's first 64
    entries, queries its last 64: the query token's own key is an ordinary one."""
    d, H, G, dim = 128, 2, 1, 64
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "scale": 1.0, "softcap": 100.0}
    if window:
        m["mask"] = {"size": window}
    g = gen(seed)
    W = {"q": torch.zeros(H * dim, d), "k": torch.zeros(G * dim, d), "v": bf(torch.randn(G * vdim, d, generator=g) / 8),
         "q.norm": torch.ones(H * dim), "k.norm": torch.ones(G * dim), "g": torch.zeros(H * vdim, d),
         "o": bf(torch.randn(d, H * vdim, generator=g) / 4)}
    for i in range(dim):
        W["k"][i, i] = 1.0
        for hh in range(H):
            W["q"][hh * dim + i, 64 + i] = 1.0
    h = bf(torch.randn(T, d, generator=g))
    h[query, 64:] = h[hot_key, :64]          # q of the query token points along the hot key: score 64 against about +-8
    return m, W, h


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("vdim", [8, 32])                     # 32: in bfloat16 the tensor-core kernel runs
@pytest.mark.parametrize("window,T,hot,query", [
    (40, 120, 60, 99),        # the oldest key the window keeps (99 - 60 = 39)
    (40, 120, 59, 99),        # the first one it has dropped
    (40, 120, 0, 39),         # the first token of the sequence, just inside
    (40, 120, 0, 40),         # ... and just outside
    (16, 120, 80, 95),        # a window of one page: its edge is a page's edge
    (16, 120, 79, 95),
    (32, 120, 64, 95),        # a window of one key tile
    (32, 120, 63, 95),
    (64, 200, 128, 191),      # ... of the tensor-core kernel's key tile
    (64, 200, 127, 191),
    (None, 400, 3, 399),      # no window: a key hundreds of positions back
    (None, 400, 16, 399),     # ... at a page's first row
    (None, 400, 31, 399),     # ... at a key tile's last row
    (300, 400, 100, 399),     # a long window: far but inside
    (300, 400, 99, 399),      # ... and outside
])
def test_attention_finds_the_one_key_that_matters(window, T, hot, query, vdim, decoded, dtype):
    m, W, h = _pointed_attention(window, T, hot, query, vdim)
    part = make_part("mixer", "gated_attention", attention_params(m, h.shape[1], 1e-5), W, DTYPES[dtype])
    want = _plain_mixer(h, W, m, 1e-5)
    visible = window is None or query - hot < window
    hz = PartHarness(part, n_pages=32, page_size=16, fill=0.0)
    got = hz.run_cut("r", h, [query - 10, 1] if decoded else [T])
    e = rel_rows(got, want)
    assert e[query] <= TOL[dtype], f"query row differs by {e[query]:.3g}"
    # (the other rows' scores are eight times as wide as a model's: in bfloat16 the rounding of keys and queries
    # shows in their sharp softmax)
    assert e.max() <= (TOL[dtype] if dtype == "float32" else 0.1)
    # the hot key's value dominates the output exactly when it is visible (gate logits are zero: sigmoid = 1/2)
    v_hot = (W["v"].double() @ h[hot].double()) * 0.5
    out_hot = W["o"].double() @ torch.cat([v_hot, v_hot])
    close = float((got[query].double() - out_hot).norm() / out_hot.norm())
    assert (close < 0.2) == visible, f"hot key visible={visible}, distance to its value {close:.3g}"


def _without_ties(h, W, f, margin=0.02):
    """The rows of h whose choice of experts and of groups does not hang on the last bits."""
    r = f["router"]
    s = torch.softmax(h.double() @ W["router"].double().T, -1)
    c = s + W["correction"].double()
    g = r.get("groups") or {}
    count, keep_g = g.get("count", 1), g.get("keep", g.get("count", 1))
    ok = torch.ones(h.shape[0], dtype=torch.bool)
    if count > 1 and keep_g < count:
        marks = torch.sort(c.reshape(h.shape[0], count, -1).max(-1).values, dim=1, descending=True).values
        ok &= (marks[:, keep_g - 1] - marks[:, keep_g]) > margin * marks[:, 0].abs().clamp(min=0.05)
    open_ = torch.ones_like(c, dtype=torch.bool)
    if count > 1 and keep_g < count:
        best = c.reshape(h.shape[0], count, -1).max(-1).values
        kept = torch.topk(best, keep_g, dim=-1).indices
        allowed = torch.zeros(h.shape[0], count, dtype=torch.bool).scatter_(1, kept, True)
        open_ = allowed[:, :, None].expand(-1, -1, c.shape[1] // count).reshape(h.shape[0], -1)
    cc = torch.where(open_, c, torch.full_like(c, -math.inf))
    srt = torch.sort(cc, dim=1, descending=True).values
    top = r["top"]
    if top < int(open_[0].sum()):
        ok &= (srt[:, top - 1] - srt[:, top]) > margin * 0.1
    return ok


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg,layer", [(CFG_A, 0), (CFG_A, 2), (CFG_A, 3), (CFG_B, 0), (CFG_B, 1), (CFG_C, 0), (CFG_C, 2)])
def test_routed_experts_alone(cfg, layer, dtype):
    f, d = cfg["layers"][layer]["mlp"], cfg["width"]
    W = plain.sub(make_weights(cfg, 13), f"l{layer}.mlp.")
    part = make_part("feed_forward", "routed_glu", routed_params(f, d), W, DTYPES[dtype])
    h = bf(torch.randn(160, d, generator=gen(15)))
    h = h[_without_ties(h, W, f)]
    assert h.shape[0] > 60
    want = plain.routed_experts(h.double(), dbl(W), f)
    hz = PartHarness(part)
    got = hz.feed("a", h)
    check_rows(got, want, dtype, what="routed experts")
    # one token at a time gives the same rows as the batch
    single = torch.cat([hz.feed("b", h[t:t + 1]) for t in range(6)], 0)
    assert rel_rows(single, got[:6]).max() <= (1e-5 if dtype == "float32" else 2e-2)


def test_the_routers_rule_shows():
    """Inputs made so that every clause of the rule decides something: the best output lies in a group that
    a correction closes; choice scores are negative, so a closed output (minus infinity) must not beat them;
    the weights are the scores without the correction and do not add up to one; an identity output is chosen."""
    d = 16
    r = {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 1}}
    f = {"kind": "moe", "router": r, "expert": {"ff": 8}}
    g = gen(41)
    W = {"router": torch.zeros(6, d), "correction": torch.tensor([-0.9, -0.9, -2.0, -2.0, -0.6, -0.7])}
    # logits: input entry e is output e's logit
    for e in range(6):
        W["router"][e, e] = 1.0
    for e in range(4):
        W[f"e{e}.gate"], W[f"e{e}.up"] = bf(torch.randn(8, d, generator=g)), bf(torch.randn(8, d, generator=g))
        W[f"e{e}.down"] = bf(torch.randn(d, 8, generator=g))
    h = torch.zeros(3, d)
    h[0, :6] = torch.tensor([0.0, 0.0, 3.0, 0.0, 1.0, 1.5])    # output 2 has the largest score, its group is closed
    h[1, :6] = torch.tensor([2.0, 1.0, 0.0, 0.0, 0.0, 0.0])    # group 0 wins: two real experts
    h[2, :6] = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 4.0])    # an identity output and its neighbour
    h[:, 6:] = bf(torch.randn(3, d - 6, generator=g))
    choice, weight = plain.route(h.double(), dbl(W), r)
    assert sorted(choice[0].tolist()) == [4, 5] and sorted(choice[1].tolist()) == [0, 1] and sorted(choice[2].tolist()) == [4, 5]
    assert float(weight.sum(-1).max()) < 0.999
    part = make_part("feed_forward", "routed_glu", routed_params(f, d), W, torch.float32)
    got = PartHarness(part).feed("a", h)
    want = plain.routed_experts(h.double(), dbl(W), f)
    assert rel_rows(got, want).max() < 1e-5
    # rows 0 and 2 use identity experts only: the output is the input times the two scores
    s = torch.softmax(h[2, :6].double(), -1)
    assert rel_rows(got[2:3], (s[4] + s[5]) * h[2:3].double()).max() < 1e-5


# ---------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------

_CACHE: dict = {}


def model_and_truth(name: str, dtype: str, lengths=(1, 2, 23, 61, 130)):
    """A model, some requests, and the plain implementation's logits for them."""
    key = (name, dtype)
    if key not in _CACHE:
        cfg, seed = CONFIGS[name]
        W, model = build(cfg, seed, dtype)
        reqs = {f"r{n}": ids_for(cfg, 100 + n, n) for n in lengths}
        tkey = ("truth", name)
        if tkey not in _CACHE:
            _CACHE[tkey] = {rid: plain.forward(cfg, W, ids).numpy() for rid, ids in reqs.items()}
        _CACHE[key] = (cfg, model, reqs, _CACHE[tkey])
    return _CACHE[key]


def engine_for(model, n_pages=64, page_size=16, max_requests=4, cap=512, **kw):
    from gibbs_b200 import Engine
    return Engine(model, n_pages=n_pages, page_size=page_size, max_requests=max_requests, max_step_tokens=cap,
                  max_context=cap, guard_cache=True, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_decoded_and_cut_prompts_match_the_plain_implementation(name, dtype):
    cfg, model, reqs, truth = model_and_truth(name, dtype)
    eng = engine_for(model)
    assert eng.plan is not None, eng.plan_refusal
    for what, steps in (("whole", trace_whole(reqs)), ("decoded", trace_tail_decoded(reqs, tail=40)),
                        ("cut", trace_portions(reqs)), ("cut in twos", trace_portions(reqs, sizes=(2,)))):
        got = run_trace_on_engine(eng, steps)
        for rid in reqs:
            check_rows(got[rid], truth[rid], dtype, strict=False, what=f"{name} {what} {rid}")


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_layer_by_layer_in_float32(name):
    """The residual stream after every layer, through the parts' forward methods."""
    cfg, model, reqs, _ = model_and_truth(name, "float32")
    W = make_weights(cfg, CONFIGS[name][1])
    ids = reqs["r61"]
    layers = []
    plain.forward(cfg, W, ids, layers_out=layers)
    eng = engine_for(model, use_plan=False, use_graphs=False)
    seen = []
    originals = [b.forward for b in model.blocks]
    try:
        for b, orig in zip(model.blocks, originals):
            def fw(x, step, caches, orig=orig):
                orig(x, step, caches)
                seen.append(x.tensor().clone())
            b.forward = fw
        from gibbs_b200 import StepEntry
        eng.open("x")
        eng.step([StepEntry("x", ids, [len(ids) - 1])])
        eng.close("x")
    finally:
        for b in model.blocks:
            del b.forward
    assert len(seen) == len(cfg["layers"])
    for i, x in enumerate(seen):
        assert rel_rows(x.cpu(), layers[i]).max() <= 1e-4, f"layer {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_plan_and_forward_methods_give_the_same_bits(name, dtype):
    cfg, model, reqs, _ = model_and_truth(name, dtype)
    steps = trace_mixed(reqs, capacity_tokens=320, seed=3)
    a = run_trace_on_engine(engine_for(model, n_pages=20), steps)
    b = run_trace_on_engine(engine_for(model, n_pages=20, use_plan=False, use_graphs=False), steps)
    for rid in reqs:
        assert np.array_equal(a[rid], b[rid]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_batches_with_pages_used_again(name, dtype):
    """Up to three live requests in a pool that holds little more than the live ones, portions beside
    single tokens: against the plain implementation, and against each request run alone."""
    cfg, model, reqs, truth = model_and_truth(name, dtype)
    more = dict(reqs)
    for k in range(4):                                        # the same lengths again: pages go round
        more[f"again{k}"] = ids_for(cfg, 500 + k, 40 + 17 * k)
    for seed in (0, 1):
        eng = engine_for(model, n_pages=20, max_requests=3)   # 320 tokens of pages
        got = run_trace_on_engine(eng, trace_mixed(more, capacity_tokens=320, max_live=3, seed=seed))
        assert eng.cache.free_pages() == [20] * len(eng.cache.groups)
        for rid in reqs:
            check_rows(got[rid], truth[rid], dtype, strict=False, what=f"{name} mixed {rid}")
        alone = run_trace_on_engine(engine_for(model), trace_whole(more))
        for rid in more:
            e = rel_rows(got[rid], alone[rid])
            lim = 1e-4 if dtype == "float32" else TOL[dtype]
            assert (e > lim).mean() <= (0.0 if dtype == "float32" else 0.45), f"{rid}: batch against alone {e.max():.3g}"


@pytest.mark.parametrize("seed", [2, 5, 8, 13, 21, 34, 55])
def test_random_configurations_in_float32(seed):
    """Sizes, options and the order of layers drawn at random (one to five layers; layers that read another
    layer's keys through a window of their own; windows of one token and none; one expert, all outputs chosen;
    groups; identity experts), whole, cut, decoded and in mixed batches.  Held to the plain implementation in
    float64, with room for a choice of experts that hangs on the last bits of a 32-bit softmax."""
    from gibbs_b200.config import parse_config
    from gibbs_b200.parts.model import build_model
    from gibbs_b200.weights import TensorDict
    cfg = random_config(seed)
    W = make_weights(cfg, seed)
    model = build_model(parse_config(cfg).plan(), TensorDict({k: v.to(torch.bfloat16) for k, v in W.items()}),
                        torch.float32, DEV)
    reqs = {f"r{n}": ids_for(cfg, seed * 7 + n, n) for n in (1, 2, 37, 90)}
    truth = {rid: plain.forward(cfg, W, ids).numpy() for rid, ids in reqs.items()}
    for what, steps in (("whole", trace_whole(reqs)), ("cut", trace_portions(reqs)),
                        ("decoded", trace_tail_decoded(reqs, tail=30)),
                        ("mixed", trace_mixed(reqs, capacity_tokens=256, max_live=3, seed=seed))):
        eng = engine_for(model, n_pages=16, max_requests=3, cap=256)
        got = run_trace_on_engine(eng, steps)
        for rid in reqs:
            e = rel_rows(got[rid], truth[rid])
            assert (e > 3e-4).mean() <= 0.02, f"{what} {rid}: {e.max():.3g} at row {int(e.argmax())}"


def test_long_decoding_past_windows_and_pages():
    """260 tokens decoded one by one after a two-token prompt: every window edge and page edge is passed
    by single tokens."""
    cfg, model, _, _ = model_and_truth("A", "float32")
    W = make_weights(cfg, CONFIGS["A"][1])
    ids = ids_for(cfg, 77, 262)
    truth = plain.forward(cfg, W, ids).numpy()
    eng = engine_for(model, n_pages=20)
    got = run_trace_on_engine(eng, trace_tail_decoded({"long": ids}, tail=260))
    e = rel_rows(got["long"], truth)
    assert e.max() <= TOL["float32"], f"first wrong position {int(np.nonzero(e > TOL['float32'])[0][0])}"
    assert min(eng.cache.free_pages()) == 20


def test_greedy_generation_through_the_scheduler():
    """Generator -> Scheduler -> Engine.step -> sampler: the tokens are those the plain implementation
    picks, fed back one by one; several prompts of unequal length at once."""
    from gibbs_b200 import Generator, SamplingParams
    cfg, model, _, _ = model_and_truth("B", "float32")
    W = make_weights(cfg, CONFIGS["B"][1])
    gen_ = Generator(model, ctx=256, page_size=16, n_pages=40, max_running=4, max_batch_tokens=48)
    prompts = [ids_for(cfg, 900 + k, n) for k, n in enumerate((3, 50, 19))]
    outs = gen_.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0), stop_at_eos=False)
    for p, out in zip(prompts, outs):
        seq = list(p)
        for tok in out:
            logits = plain.forward(cfg, W, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) > 1e-3:               # (no verdict on a tie)
                assert int(logits.argmax()) == tok, f"after {len(seq)} tokens"
            seq.append(tok)
        assert len(out) == 12


def test_command_line_from_a_configuration_to_tokens(tmp_path, capsys):
    """config.json -> random weights on disk -> --arch-dump, --probe-top5 and a greedy continuation, all
    through the command line's own entry point."""
    import json
    from gibbs_b200.engine.cli import main
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(CFG_A))
    folder = tmp_path / "model"
    assert main(["--random", str(cfg_path), "--save", str(folder), "--seed", "3", "--dtype", "float32"]) == 0
    capsys.readouterr()
    assert main(["-m", str(folder), "--arch-dump"]) == 0
    dump = json.loads(capsys.readouterr().out)
    assert dump["architecture"] == "Petelix"
    prompt = ids_for(CFG_A, 5, 9)
    ids = ",".join(map(str, prompt))
    assert main(["-m", str(folder), "--dtype", "float32", "--probe-top5", ids, "--ctx", "128"]) == 0
    top = json.loads(capsys.readouterr().out)
    from gibbs_b200.weights import Checkpoint
    ck = Checkpoint(folder)
    W = {n: ck.tensor(n) for n in ck.names()}
    logits = plain.forward(CFG_A, W, prompt)[-1]
    assert top["ids"][0] == int(logits.argmax())
    assert abs(top["logits"][0] - float(logits.max())) < 1e-3
    assert main(["-m", str(folder), "--dtype", "float32", "--prompt-ids", ids, "--max-tokens", "5", "--temperature", "0",
                 "--ctx", "128"]) == 0
    out = capsys.readouterr().out
    generated = [int(t) for t in out.split("Output:\n")[1].splitlines()[0].split(",")]
    assert len(generated) == 5 and generated[0] == top["ids"][0]


@pytest.mark.parametrize("cfg,layer", [(CFG_D, 0), (CFG_D, 2), (CFG_D, 3), (CFG_D, 4)])
def test_tensor_core_attention_against_the_generic_kernel(cfg, layer, monkeypatch):
    """In bfloat16 the two kernels read the same pages; they differ by the rounding of the queries and of
    the weights' second term only.  A long request, cut so that tiles hold a few rows and many."""
    from gibbs_b200.parts import gated_attention as ga
    m, d, eps = cfg["layers"][layer]["mixer"], cfg["width"], cfg["norm"]["eps"]
    W = plain.sub(make_weights(cfg, 5), f"l{layer}.mix.")
    T = 330
    h = bf(torch.randn(T, d, generator=gen(8)))
    want = _plain_mixer(h, W, m, eps)
    outs = {}
    for on in (True, False):
        monkeypatch.setattr(ga, "USE_TENSOR_CORES", on)
        part = make_part("mixer", "gated_attention", attention_params(m, d, eps), W, torch.bfloat16)
        hz = PartHarness(part, n_pages=24, page_size=16, fill=0.0)
        outs[on] = hz.run_cut("r", h, [150, 3, 1, 1, 90, 1, 64, 2, 1])
        check_rows(outs[on], want, "bfloat16", what=f"tensor cores {on}")
    assert rel_rows(outs[True], outs[False]).max() < 1.5e-2
