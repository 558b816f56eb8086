"""Shared by the Petelix tests: small configurations that differ in every size
and option, weights with realistic scales (all values exactly representable in
bfloat16, so that both compute dtypes and the plain implementation read the same
numbers), and builders."""
from __future__ import annotations

import math
import random

import torch


def _att(heads, kv_heads, dim, vdim, scale, window=None, rot=None, softcap=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if softcap is not None:
        m["softcap"] = softcap
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff, identity=0, groups=None):
    r = {"experts": experts, "top": top, "identity": identity}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": r, "expert": {"ff": ff}}


# A: three query heads a kv head, values wider than keys, a reader whose window is wider than its source's, a layer
# without a feed-forward, a source without a window read through a narrow one, experts of 64 (the tensor-core path in
# bfloat16), identity experts, groups 4 keep 2 and 2 keep 1
CFG_A = {
    "architecture": "Petelix", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [
        {"type": "attention", "mixer": _att(6, 2, 16, 24, 0.3, window=19, rot=(1000.0, 8), softcap=5.0),
         "mlp": _moe(6, 3, 40, identity=2, groups=(4, 2))},
        {"type": "attention", "mixer": _att(6, 2, 16, 24, 0.25, window=33, rot=(1000.0, 8), softcap=8.0, kv_from=0),
         "mlp": None},
        {"type": "attention", "mixer": _att(4, 4, 8, 8, 0.5, rot=(100.0, 8)), "mlp": _moe(5, 2, 64)},
        {"type": "attention", "mixer": _att(4, 4, 8, 8, 0.4, window=7, rot=(100.0, 8), softcap=50.0, kv_from=2),
         "mlp": _moe(3, 1, 16, identity=1, groups=(2, 1))},
    ],
}
# B: ten query heads a kv head (more than a block's warps), values of 40 and 72 entries, no rotation in one layer,
# every router output chosen, sixteen experts in four groups
CFG_B = {
    "architecture": "Petelix", "vocab": 257, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
    "layers": [
        {"type": "attention", "mixer": _att(20, 2, 12, 40, 0.3, window=40, rot=(50000.0, 4), softcap=30.0),
         "mlp": _moe(16, 4, 128, groups=(4, 2))},
        {"type": "attention", "mixer": _att(3, 1, 32, 72, 0.2), "mlp": _moe(2, 4, 16, identity=2)},
    ],
}
# C: sizes that are multiples of nothing, one head, a window of one token, one expert and one identity expert, a reader
# without a window on a source with one
CFG_C = {
    "architecture": "Petelix", "vocab": 97, "width": 44, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
    "layers": [
        {"type": "attention", "mixer": _att(1, 1, 10, 7, 0.4, window=1, rot=(30.0, 2), softcap=2.0), "mlp": _moe(1, 1, 9, identity=1)},
        {"type": "attention", "mixer": _att(5, 5, 6, 3, 0.5, window=5, rot=(10000.0, 6)), "mlp": None},
        {"type": "attention", "mixer": _att(5, 5, 6, 3, 0.5, rot=(10000.0, 6), kv_from=1), "mlp": _moe(7, 2, 20, groups=(7, 3))},
    ],
}
# D: sizes the tensor-core attention kernel is built for (keys and values of 32, 64, 96 and 128 entries, unequal), one,
# two, three and sixteen query heads a kv head, with and without a window, a reader with a wider window
CFG_D = {
    "architecture": "Petelix", "vocab": 211, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
    "layers": [
        {"type": "attention", "mixer": _att(4, 2, 32, 64, 0.2, window=40, rot=(1000.0, 16), softcap=10.0),
         "mlp": _moe(4, 2, 64, identity=2, groups=(3, 2))},
        {"type": "attention", "mixer": _att(4, 2, 32, 64, 0.2, window=70, rot=(1000.0, 16), softcap=10.0, kv_from=0), "mlp": None},
        {"type": "attention", "mixer": _att(6, 2, 96, 32, 0.12, rot=(10000.0, 96)), "mlp": _moe(3, 1, 128)},
        {"type": "attention", "mixer": _att(16, 1, 64, 128, 0.15, window=100, rot=(500.0, 8), softcap=4.0), "mlp": None},
        {"type": "attention", "mixer": _att(3, 3, 128, 96, 0.1, window=16), "mlp": _moe(2, 2, 64)},
    ],
}
CONFIGS = {"A": (CFG_A, 21), "B": (CFG_B, 22), "C": (CFG_C, 23), "D": (CFG_D, 24)}


def random_config(seed: int) -> dict:
    """A configuration of the design with every size, option and the order of layers drawn at random."""
    rng = random.Random(seed)
    d = rng.choice([24, 32, 40, 64, 72, 128])
    layers, sources = [], []
    for i in range(rng.randint(1, 5)):
        if sources and rng.random() < 0.4:
            j = rng.choice(sources)
            o = layers[j]["mixer"]
            m = _att(o["heads"], o["kv_heads"], o["dim"], o["vdim"], rng.choice([0.2, 0.35, 0.5]), kv_from=j)
            if "rot" in o:
                m["rot"] = dict(o["rot"])
        else:
            G = rng.choice([1, 2, 3, 5])
            dim = rng.choice([2, 4, 8, 16, 24, 32, 40, 64])
            m = _att(G * rng.choice([1, 2, 4, 9]), G, dim, rng.choice([1, 3, 8, 16, 32, 33, 64]), rng.choice([0.2, 0.35, 0.5]))
            if rng.random() < 0.8:
                m["rot"] = {"base": rng.choice([10.0, 1000.0, 500000.0]), "dims": rng.choice(range(2, dim + 1, 2))}
            sources.append(i)
        w = rng.choice([None, 1, 2, 7, 16, 17, 40, 100])
        if w:
            m["mask"] = {"size": w}
        if rng.random() < 0.6:
            m["softcap"] = rng.choice([1.5, 10.0, 30.0])
        if rng.random() < 0.2:
            f = None
        else:
            count = rng.choice([1, 1, 2, 3, 4])
            per = rng.choice([1, 2, 3, 5])
            keep = rng.randint(1, count)
            ident = rng.randint(0, min(2, count * per - 1))
            f = _moe(count * per - ident, rng.randint(1, min(4, keep * per)), rng.choice([4, 9, 16, 64]), ident, (count, keep))
        layers.append({"type": "attention", "mixer": m, "mlp": f})
    return {"architecture": "Petelix", "vocab": rng.choice([50, 97, 256]), "width": d, "norm": {"eps": rng.choice([1e-5, 1e-6])},
            "embedding": {"scale": rng.choice([1.0, 0.7, 6.0])}, "layers": layers}


def _bf16_exact(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> float32 tensor (bfloat16-exact values) for every tensor of the design."""
    g = torch.Generator().manual_seed(seed)
    d, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, out, inp, scale=1.0):
        W[name] = torch.randn(out, inp, generator=g) * (scale / math.sqrt(inp))

    def gain(name, n):
        W[name] = 1.0 + 0.15 * torch.randn(n, generator=g)

    W["embed"] = torch.randn(V, d, generator=g)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        gain(p + "norm1", d)
        mat(p + "mix.q", H * dim, d), gain(p + "mix.q.norm", H * dim)
        # (heads of unequal size: a norm over the whole projection is then not a norm per head)
        W[p + "mix.q"] *= (1.0 + torch.arange(H * dim) // dim % 3).unsqueeze(1).float()
        if m.get("kv_from") is None:
            mat(p + "mix.k", G * dim, d), gain(p + "mix.k.norm", G * dim), mat(p + "mix.v", G * vdim, d, 1.5)
            W[p + "mix.k"] *= (1.0 + torch.arange(G * dim) // dim % 2).unsqueeze(1).float()
        mat(p + "mix.g", H * vdim, d, 2.0), mat(p + "mix.o", d, H * vdim)
        f = layer.get("mlp")
        if f is not None:
            gain(p + "norm2", d)
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            n_out = E + f["router"].get("identity", 0)
            mat(p + "mlp.router", n_out, d, 2.0)
            W[p + "mlp.correction"] = torch.randn(n_out, generator=g) * (0.6 / n_out) - 0.3 / n_out
            for e in range(E):
                mat(p + f"mlp.e{e}.gate", ff, d, 1.5), mat(p + f"mlp.e{e}.up", ff, d, 1.5), mat(p + f"mlp.e{e}.down", d, ff)
    gain("final.norm", d)
    mat("head", V, d, 3.0)
    return {k: _bf16_exact(v) for k, v in W.items()}


def build(cfg: dict, seed: int, dtype: str, device="cuda:0"):
    """(weights, model on the device) of a configuration."""
    from gibbs_b200.config import parse_config
    from gibbs_b200.engine.loading import parse_dtype
    from gibbs_b200.parts.model import build_model
    from gibbs_b200.weights import TensorDict
    W = make_weights(cfg, seed)
    conf = parse_config(cfg)
    model = build_model(conf.plan(), TensorDict({k: v.to(torch.bfloat16) for k, v in W.items()}), parse_dtype(dtype), device)
    model.config = conf
    return W, model


def attention_params(m: dict, d: int, eps: float) -> dict:
    """What the design's plan hands the attention part for a mixer's config."""
    rot = m.get("rot") or {}
    w = (m.get("mask") or {}).get("size")
    return {"hidden": d, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
            "scale": m["scale"], "softcap": m.get("softcap") or 0.0, "window": w, "retain": w,
            "rot_base": rot.get("base", 1.0), "rot_dims": rot.get("dims", 0), "eps": eps, "qk_norm": "whole",
            "sink": True, "gate": True, "shares_kv": False}


def routed_params(f: dict, d: int) -> dict:
    r = f["router"]
    g = r.get("groups") or {}
    return {"hidden": d, "experts": r["experts"], "top": r["top"], "expert_inner": f["expert"]["ff"], "expert_limit": 0.0,
            "alpha": 1.0, "up_add": 0.0, "scores": "softmax", "correction": True, "identity": r.get("identity", 0),
            "groups": g.get("count", 1), "groups_keep": g.get("keep", g.get("count", 1)), "weight_on": "output"}
