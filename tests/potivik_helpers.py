"""Shared by the Potivik tests: two small configurations that differ in every
size and option, weights with realistic scales (all values exactly
representable in bfloat16, so that both compute dtypes and the plain
implementation read the same numbers), model folders, and a harness that runs
ONE mixer alone over a request cut into portions."""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch

# layers: latent attention with a window and a partly rotated part + routed experts (top 2, shared expert);
# state-space mixer with two groups and two norm groups + dense unit; a layer without a feed-forward; latent
# attention without a window + routed experts (top 3, no shared expert).  Per-token input and a soft cap.
CFG_A = {
    "architecture": "Potivik", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 10.0,
    "token_side": {"dim": 8},
    "layers": [
        {"type": "latent_attention",
         "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 40, "scale": 0.35,
                   "mask": {"size": 19}, "rot": {"base": 1000.0, "dims": 4}},
         "mlp": {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 40, "limit": 1.5},
                 "shared": {"ff": 24, "limit": 3.0}}},
        {"type": "mamba2",
         "mixer": {"heads": 4, "vdim": 12, "state": 20, "groups": 2, "conv": 4, "norm_groups": 2},
         "mlp": {"kind": "dense", "ff": 72, "limit": 0.8}},
        {"type": "mamba2",
         "mixer": {"heads": 4, "vdim": 12, "state": 20, "groups": 2, "conv": 4, "norm_groups": 2},
         "mlp": None},
        {"type": "latent_attention",
         "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 40, "scale": 0.35,
                   "rot": {"base": 1000.0, "dims": 8}},
         "mlp": {"kind": "moe", "router": {"experts": 5, "top": 3}, "expert": {"ff": 16, "limit": 2.0}}},
    ],
}
# more than eight heads, a latent wider than 64, a state wider than 64 that is no multiple of 32, a convolution
# of two taps, one expert per token, no per-token input, no soft cap
CFG_B = {
    "architecture": "Potivik", "vocab": 257, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mamba2",
         "mixer": {"heads": 2, "vdim": 40, "state": 70, "groups": 1, "conv": 2, "norm_groups": 1},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 1}, "expert": {"ff": 48, "limit": 2.5},
                 "shared": {"ff": 32, "limit": 2.5}}},
        {"type": "latent_attention",
         "mixer": {"heads": 10, "dim": 8, "rot_dim": 16, "vdim": 8, "kv_rank": 72, "scale": 0.3,
                   "mask": {"size": 33}, "rot": {"base": 50000.0, "dims": 16}},
         "mlp": {"kind": "dense", "ff": 128, "limit": 1.0}},
    ],
}
# awkward sizes: nothing is a multiple of 8 (every product runs on the 32-bit tiles, cache rows are read
# value by value), one attention head, a window of one, every expert chosen, three groups, five taps
CFG_C = {
    "architecture": "Potivik", "vocab": 97, "width": 44, "norm": {"eps": 1e-5}, "logit_softcap": 4.0,
    "token_side": {"dim": 3},
    "layers": [
        {"type": "latent_attention",
         "mixer": {"heads": 1, "dim": 10, "rot_dim": 6, "vdim": 7, "kv_rank": 21, "scale": 0.4,
                   "mask": {"size": 5}, "rot": {"base": 30.0, "dims": 2}},
         "mlp": {"kind": "moe", "router": {"experts": 2, "top": 2}, "expert": {"ff": 9, "limit": 1.0}}},
        {"type": "mamba2",
         "mixer": {"heads": 3, "vdim": 5, "state": 33, "groups": 3, "conv": 5, "norm_groups": 3},
         "mlp": {"kind": "dense", "ff": 20, "limit": 0.5}},
        {"type": "latent_attention",
         "mixer": {"heads": 5, "dim": 4, "rot_dim": 2, "vdim": 3, "kv_rank": 9, "scale": 0.5,
                   "mask": {"size": 1}, "rot": {"base": 10000.0, "dims": 2}},
         "mlp": None},
        {"type": "mamba2",
         "mixer": {"heads": 1, "vdim": 3, "state": 4, "groups": 1, "conv": 1, "norm_groups": 1},
         "mlp": {"kind": "moe", "router": {"experts": 7, "top": 1}, "expert": {"ff": 64, "limit": 3.0},
                 "shared": {"ff": 5, "limit": 3.0}}},
    ],
}
CONFIGS = {"A": (CFG_A, 11), "B": (CFG_B, 12), "C": (CFG_C, 13)}


def random_config(seed: int) -> dict:
    """A configuration of the design with every size, option and the order of layers drawn at random."""
    import random
    rng = random.Random(seed)
    d = rng.choice([24, 32, 40, 64, 72, 128])
    layers = []
    for _ in range(rng.randint(1, 5)):
        if rng.random() < 0.5:
            dr = rng.choice([2, 4, 6, 8, 16]); dims = rng.choice([x for x in range(2, dr + 1, 2)])
            m = {"heads": rng.choice([1, 2, 3, 5, 8, 17]), "dim": rng.choice([2, 4, 7, 8, 16, 24]), "rot_dim": dr,
                 "vdim": rng.choice([1, 3, 8, 16]), "kv_rank": rng.choice([4, 8, 12, 33, 64, 96]), "scale": rng.choice([0.2, 0.35, 0.5]),
                 "rot": {"base": rng.choice([10.0, 1000.0, 500000.0]), "dims": dims}}
            w = rng.choice([None, 1, 2, 7, 16, 17, 40, 100])
            if w: m["mask"] = {"size": w}
            layers.append({"type": "latent_attention", "mixer": m})
        else:
            heads = rng.choice([1, 2, 4, 6]); groups = rng.choice([g for g in (1, 2, 3, 6) if heads % g == 0])
            P = rng.choice([1, 3, 4, 8, 12, 20]); inner = heads * P
            ng = rng.choice([g for g in (1, 2, 3, 4) if inner % g == 0])
            layers.append({"type": "mamba2", "mixer": {"heads": heads, "vdim": P, "state": rng.choice([1, 4, 8, 16, 24, 33, 64, 128, 132]),
                                                        "groups": groups, "conv": rng.randint(1, 5), "norm_groups": ng}})
        k = rng.random()
        if k < 0.2: layers[-1]["mlp"] = None
        elif k < 0.5: layers[-1]["mlp"] = {"kind": "dense", "ff": rng.choice([8, 20, 64, 128]), "limit": rng.choice([0.5, 1.0, 4.0])}
        else:
            E = rng.choice([1, 2, 3, 8, 16, 33]); top = rng.randint(1, min(E, 4))
            f = {"kind": "moe", "router": {"experts": E, "top": top}, "expert": {"ff": rng.choice([4, 9, 16, 64]), "limit": rng.choice([1.0, 3.0])}}
            if rng.random() < 0.5: f["shared"] = {"ff": rng.choice([8, 24, 64]), "limit": rng.choice([1.0, 3.0])}
            layers[-1]["mlp"] = f
    cfg = {"architecture": "Potivik", "vocab": rng.choice([50, 97, 256]), "width": d, "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.6: cfg["token_side"] = {"dim": rng.choice([1, 3, 8, 16])}
    if rng.random() < 0.6: cfg["logit_softcap"] = rng.choice([5.0, 30.0])
    return cfg


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
    side = cfg.get("token_side")
    if side:
        W["side.embed"] = torch.randn(V, len(cfg["layers"]) * side["dim"], generator=g)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        gain(p + "norm1", d), gain(p + "norm1b", d)
        if layer["type"] == "latent_attention":
            H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            mat(p + "mix.q", H * (dn + dr), d, 1.6), mat(p + "mix.dkv", r + dr, d, 1.6)
            gain(p + "mix.dkv.norm", r)
            mat(p + "mix.uk", H * dn, r, 1.3), mat(p + "mix.uv", H * dv, r), mat(p + "mix.g", H, d, 2.0)
            mat(p + "mix.o", d, H * dv)
        else:
            H, P, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = H * P, H * P + 2 * G * N
            mat(p + "mix.in", 2 * inner + 2 * G * N + H, d)
            W[p + "mix.conv"] = torch.randn(ch, K, generator=g) * 0.5
            W[p + "mix.conv.b"] = torch.randn(ch, generator=g) * 0.1
            W[p + "mix.dt_bias"] = torch.randn(H, generator=g) * 0.7 - 1.5
            W[p + "mix.A_log"] = torch.log(0.3 + 3.0 * torch.rand(H, generator=g))
            W[p + "mix.D"] = 1.0 + 0.2 * torch.randn(H, generator=g)
            gain(p + "mix.norm", inner)
            mat(p + "mix.o", d, inner)
        f = layer.get("mlp")
        if f is not None:
            gain(p + "norm2", d), gain(p + "norm2b", d)
            if f["kind"] == "dense":
                mat(p + "mlp.gate", f["ff"], d, 1.5), mat(p + "mlp.up", f["ff"], d, 1.5), mat(p + "mlp.down", d, f["ff"])
            else:
                E, ff = f["router"]["experts"], f["expert"]["ff"]
                mat(p + "mlp.router", E, d, 2.0)
                for e in range(E):
                    mat(p + f"mlp.e{e}.gate", ff, d, 1.5), mat(p + f"mlp.e{e}.up", ff, d, 1.5), mat(p + f"mlp.e{e}.down", d, ff)
                if f.get("shared"):
                    sf = f["shared"]["ff"]
                    mat(p + "mlp.shared.gate", sf, d, 1.5), mat(p + "mlp.shared.up", sf, d, 1.5)
                    mat(p + "mlp.shared.down", d, sf), mat(p + "mlp.shared.sg", 1, d, 1.5)
        if side:
            mat(p + "side.gate", side["dim"], d), mat(p + "side.proj", d, side["dim"]), gain(p + "side.norm", d)
    gain("final.norm", d)
    mat("head", V, d, 3.0)
    return {k: _bf16_exact(v) for k, v in W.items()}


def write_model(folder, cfg: dict, W: dict, stored=torch.bfloat16) -> Path:
    from gibbs_b200.weights.safetensors_io import write_safetensors
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(folder / "model.safetensors", ((k, v.to(stored)) for k, v in W.items()), metadata={"format": "pt"})
    return folder


def build(name: str, dtype: str, device="cuda:0"):
    """(config dict, weights, model on the device) of a named configuration."""
    from gibbs_b200.config import parse_config
    from gibbs_b200.engine.loading import parse_dtype
    from gibbs_b200.parts.model import build_model
    from gibbs_b200.weights import TensorDict
    cfg, seed = CONFIGS[name]
    W = make_weights(cfg, seed)
    conf = parse_config(cfg)
    model = build_model(conf.plan(), TensorDict({k: v.to(torch.bfloat16) for k, v in W.items()}), parse_dtype(dtype), device)
    model.config = conf
    return cfg, W, model


def ids_for(cfg: dict, seed: int, n: int) -> list:
    rng = np.random.default_rng(seed)
    return [int(v) for v in rng.integers(0, cfg["vocab"], n)]


class PartHarness:
    """Runs one mixer alone, with a cache manager and step builder of its own, over a request cut
    into portions.  ``feed(request, h)`` runs the next tokens of a request and returns the mixer's
    output for them (float32)."""

    def __init__(self, part, n_pages=64, page_size=16, n_slots=3, max_context=1024, guard=True, fill=float("nan")):
        self.fill = fill            # what the output rows hold before the part runs (0 for a part that ADDS its output)
        from gibbs_b200.cache import CacheManager
        from gibbs_b200.engine.step import StepBuilder
        self.part, self.rt = part, part.rt
        self.cache = CacheManager([(getattr(part, 'cache_needs', list)(), None)], n_pages, page_size, n_slots, part.rt.dtype, part.rt.device,
                                  max_context, guard=guard)
        self.builder = StepBuilder(self.cache, part.rt.device, n_slots, max_context)

    def feed_many(self, portions: dict) -> dict:
        """portions: {request: h [n, hidden] float32 on the CPU}; one step for all of them."""
        from gibbs_b200.engine.step import StepEntry
        rcs, entries = [], []
        for rid, h in portions.items():
            if rid not in self.cache.live:
                self.cache.open(rid)
            rc = self.cache.live[rid]
            rcs.append(rc)
            entries.append(StepEntry(rid, [0] * h.shape[0], []))
        self.cache.reserve_all([(rc, rc.length + len(e.tokens)) for rc, e in zip(rcs, entries)])
        step, caches = self.builder.build(entries, rcs)
        h = torch.cat(list(portions.values()), 0).to(self.rt.device, self.rt.dtype).contiguous()
        out = torch.full((h.shape[0], self.part.hidden), self.fill, dtype=torch.float32, device=self.rt.device)
        self.part.forward(h, out, step, caches[0])
        torch.cuda.synchronize()
        for rc, e in zip(rcs, entries):
            self.cache.advance(rc, rc.length + len(e.tokens))
        self.cache.check()
        res, at = {}, 0
        for rid, hh in portions.items():
            res[rid] = out[at:at + hh.shape[0]].cpu()
            at += hh.shape[0]
        return res

    def feed(self, rid, h):
        return self.feed_many({rid: h})[rid]

    def close(self, rid):
        self.cache.close(rid)

    def run_cut(self, rid, h, cuts):
        """The whole of h for one request, in portions of the given sizes (the last size repeats)."""
        outs, at, k = [], 0, 0
        while at < h.shape[0]:
            n = min(cuts[min(k, len(cuts) - 1)], h.shape[0] - at)
            outs.append(self.feed(rid, h[at:at + n]))
            at, k = at + n, k + 1
        return torch.cat(outs, 0)


def make_part(category: str, kind: str, params: dict, tensors: dict, dtype=torch.float32, device="cuda:0"):
    """A part built directly from tensors (float32, bfloat16-exact), as the loader would hand them over."""
    from gibbs_b200.parts.base import MATRIX, Runtime, part_class
    cls = part_class(category, kind)
    rt = Runtime(dtype=dtype, device=torch.device(device))
    decl = cls.declare(params)
    given = {}
    for name, d in decl.items():
        t = tensors[name].reshape(d.shapes[0])
        mem = dtype if (d.role == MATRIX and dtype == torch.bfloat16) else torch.float32
        given[name] = t.to(device=device, dtype=mem).contiguous()
    return cls(params, given, rt)


def rel_rows(got, want) -> np.ndarray:
    """Per-row relative L2 error."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return np.linalg.norm(got - want, axis=-1) / (np.linalg.norm(want, axis=-1) + 1e-30)
