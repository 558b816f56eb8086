"""Configuration of the Petelix design and its plan.

Petelix is a decoder-only model whose config.json lists its layers one by one
(``layers``).  A layer is pre-norm: x += mixer(rmsnorm(x)), then, unless its
``mlp`` is null, x += ff(rmsnorm(x)).  The embedded tokens are multiplied by
``embedding.scale``; the model ends with its norm and the head.

Mixer ``attention``: grouped-query attention (``heads``, ``kv_heads``, key size
``dim``, value size ``vdim``) with an RMS norm over the whole query and the whole
key projection, a rotation of the first ``rot.dims`` entries of every head in
adjacent pairs, ``scale``, a soft cap on the scores, a sliding window
(``mask.size``), a sink in the softmax and a sigmoid gate on the concatenated
heads.  ``kv_from: j`` makes the layer read layer j's keys and values.

Feed-forward ``moe``: ``router.experts`` gated units (silu(gate) * up, then
down) of width ``expert.ff`` plus ``router.identity`` identity experts; softmax
scores over all of them, a correction added for the choice only, groups of
neighbours of which ``groups.keep`` stay open, ``router.top`` chosen, weights on
the experts' outputs and not renormalised.

Tensor names: ``embed``, ``final.norm``, ``head``; layer i's start with ``l<i>.``:
``norm1``, ``norm2``, ``mix.{q,k,v,q.norm,k.norm,g,o}``, ``mlp.router``,
``mlp.correction``, ``mlp.e<k>.{gate,up,down}``.

Constants the design fixes: the sink's score 0 (one added to the softmax's
denominator), plain norm gains, no biases.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Iterable, Optional

from .lfm2 import ConfigError
from .plan import LayerSpec, ModelPlan, OrderEntry, PartSpec

DEFAULT_CONTEXT = 131072          # config.json names no longest context; pools are sized by the engine's caller


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"config.json: {where} has no '{key}'")
    return d[key]


@dataclass(frozen=True)
class PetelixConfig:
    raw: dict

    # -- what the rest of the framework asks a configuration -----------------------------
    @property
    def vocab_size(self) -> int:
        return int(self.raw["vocab"])

    @property
    def hidden_size(self) -> int:
        return int(self.raw["width"])

    @property
    def num_hidden_layers(self) -> int:
        return len(self.raw["layers"])

    @property
    def max_position_embeddings(self) -> int:
        return int(self.raw.get("max_context") or DEFAULT_CONTEXT)

    @property
    def eos_token_ids(self) -> tuple:
        eos = self.raw.get("eos_token_id")
        return () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))

    @property
    def norm_eps(self) -> float:
        return float(self.raw["norm"]["eps"])

    @classmethod
    def from_dict(cls, cfg: dict, tensor_names: Optional[Iterable[str]] = None) -> "PetelixConfig":
        out = cls(copy.deepcopy(cfg))
        out.check()
        return out

    def check(self) -> None:
        c = self.raw
        for key in ("vocab", "width", "layers"):
            _need(c, key, "the model")
        _need(_need(c, "norm", "the model"), "eps", "norm")
        if not isinstance(c["layers"], list) or not c["layers"]:
            raise ConfigError("config.json: 'layers' is a non-empty list")
        for i, layer in enumerate(c["layers"]):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind != "attention":
                raise ConfigError(f"{where}: unknown mixer type '{kind}'; Petelix knows 'attention'")
            m = _need(layer, "mixer", where)
            for k in ("heads", "kv_heads", "dim", "vdim", "scale"):
                _need(m, k, where + ".mixer")
            if int(m["kv_heads"]) < 1 or int(m["heads"]) % int(m["kv_heads"]):
                raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
            rot = m.get("rot")
            if rot is not None:
                _need(rot, "base", where + ".mixer.rot"), _need(rot, "dims", where + ".mixer.rot")
                if int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= int(m["dim"]):
                    raise ConfigError(f"{where}: {rot['dims']} rotated dimensions must be even and at most dim {m['dim']}")
            src = m.get("kv_from")
            if src is not None:
                if not isinstance(src, int) or not 0 <= src < i:
                    raise ConfigError(f"{where}: kv_from {src!r} names no earlier layer")
                o = c["layers"][src]["mixer"]
                if o.get("kv_from") is not None:
                    raise ConfigError(f"{where}: kv_from {src} names a layer without keys and values of its own")
                for k in ("kv_heads", "dim", "vdim"):
                    if int(o[k]) != int(m[k]):
                        raise ConfigError(f"{where}: '{k}' differs from layer {src}'s, whose keys and values it reads")
            f = layer.get("mlp")
            if f is not None:
                fk = _need(f, "kind", where + ".mlp")
                if fk != "moe":
                    raise ConfigError(f"{where}: unknown mlp kind '{fk}'; Petelix knows 'moe'")
                r = _need(f, "router", where + ".mlp")
                _need(_need(f, "expert", where + ".mlp"), "ff", where + ".mlp.expert")
                _need(r, "experts", where + ".mlp.router"), _need(r, "top", where + ".mlp.router")
                n_out = int(r["experts"]) + int(r.get("identity") or 0)
                g = r.get("groups") or {}
                count = int(g.get("count") or 1)
                keep = int(g.get("keep") or count)
                if n_out % count or not 1 <= keep <= count:
                    raise ConfigError(f"{where}: {n_out} router outputs in {count} groups of which {keep} are kept")
                if not 1 <= int(r["top"]) <= (n_out // count) * keep:
                    raise ConfigError(f"{where}: top {r['top']} of {(n_out // count) * keep} router outputs that can be chosen")

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    def dump(self) -> dict:
        d = self.to_dict()
        d["kv sources (derived)"] = [layer["mixer"].get("kv_from") for layer in self.raw["layers"]]
        return d

    # -- plan ------------------------------------------------------------------------------
    def plan(self) -> ModelPlan:
        c = self.raw
        d, vocab, eps = self.hidden_size, self.vocab_size, self.norm_eps
        n_layers = len(c["layers"])

        def norm(tensor):
            return PartSpec("rmsnorm", {"dim": d, "eps": eps}, {"weight": tensor})

        def window(m):
            size = (m.get("mask") or {}).get("size")
            return int(size) if size else None

        # pages keep what the widest window among the layers that read them needs
        retain = {}
        for i, layer in enumerate(c["layers"]):
            m = layer["mixer"]
            owner = i if m.get("kv_from") is None else int(m["kv_from"])
            w = window(m)
            if owner not in retain:
                retain[owner] = w
            elif retain[owner] is not None:
                retain[owner] = None if w is None else max(retain[owner], w)

        layers, ignorable = [], []
        for i, layer in enumerate(c["layers"]):
            p, m = f"l{i}", layer["mixer"]
            shares = m.get("kv_from") is not None
            rot = m.get("rot") or {}
            names = ["q", "q.norm", "g", "o"] + ([] if shares else ["k", "v", "k.norm"])
            mixer = PartSpec("gated_attention", {
                "hidden": d, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
                "vdim": int(m["vdim"]), "scale": float(m["scale"]), "softcap": float(m.get("softcap") or 0.0),
                "window": window(m), "retain": retain[i] if not shares else retain[int(m["kv_from"])],
                "rot_base": float(rot.get("base", 1.0)), "rot_dims": int(rot.get("dims", 0)), "eps": eps,
                "qk_norm": "whole", "sink": True, "gate": True, "shares_kv": shares,
            }, {k: f"{p}.mix.{k}" for k in names})
            parts = [("mixer_norm", "norm", norm(f"{p}.norm1")), ("mixer", "mixer", mixer)]
            f = layer.get("mlp")
            if f is None:
                ignorable.append(f"{p}.norm2")
            else:
                r = f["router"]
                E, ident = int(r["experts"]), int(r.get("identity") or 0)
                groups = r.get("groups") or {}
                tensors = {"router": f"{p}.mlp.router", "correction": f"{p}.mlp.correction"}
                for e in range(E):
                    tensors.update({f"e{e}.{k}": f"{p}.mlp.e{e}.{k}" for k in ("gate", "up", "down")})
                ffn = PartSpec("routed_glu", {
                    "hidden": d, "experts": E, "top": int(r["top"]), "expert_inner": int(f["expert"]["ff"]),
                    "expert_limit": 0.0, "alpha": 1.0, "up_add": 0.0,            # silu(gate) * up, no clamp
                    "scores": "softmax", "correction": True, "identity": ident,
                    "groups": int(groups.get("count") or 1), "groups_keep": int(groups.get("keep") or groups.get("count") or 1),
                    "weight_on": "output",
                }, tensors)
                parts += [("ffn_norm", "norm", norm(f"{p}.norm2")), ("ffn", "feed_forward", ffn)]
            layers.append(LayerSpec("prenorm_residual", tuple(parts)))

        order = tuple(OrderEntry(i, None if layer["mixer"].get("kv_from") is None else int(layer["mixer"]["kv_from"]))
                      for i, layer in enumerate(c["layers"]))
        plan = ModelPlan(
            architecture="Petelix", vocab_size=vocab, hidden_size=d, max_context=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab": vocab, "dim": d,
                                                   "scale": float((c.get("embedding") or {}).get("scale", 1.0))},
                               {"weight": "embed"}),
            layers=tuple(layers), order=order, final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab": vocab, "dim": d}, {"weight": "head"}),
            ignorable=tuple(ignorable),
        )
        plan.validate()
        return plan
