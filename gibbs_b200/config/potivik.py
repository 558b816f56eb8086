"""Configuration of the Potivik design and its plan.

Potivik is a decoder-only model whose config.json lists its layers one by one
(``layers``): each entry names its mixer (``type``: ``latent_attention`` or
``mamba2``) with the mixer's sizes (``mixer``) and its feed-forward (``mlp``:
dense, routed among experts, or null for none).  Every layer has a layer norm
in front of and behind each sublayer, and (with ``token_side``) a gated input
looked up by token id after the feed-forward.  The model ends with its norm,
the head and a soft cap on the logits.

Tensor names: ``embed``, ``side.embed``, ``final.norm``, ``head``; layer i's
tensors start with ``l<i>.``: ``norm1``, ``norm1b``, ``norm2``, ``norm2b``,
``mix.*``, ``mlp.*`` (experts ``mlp.e<k>.*``, the shared expert ``mlp.shared.*``),
``side.gate``, ``side.proj``, ``side.norm``.

Constants the design fixes (they are not in config.json): the gated units use
g * sigmoid(1.702 g) * (u + 1); norms have a gain and no bias.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Iterable, Optional

from .lfm2 import ConfigError
from .plan import LayerSpec, ModelPlan, OrderEntry, PartSpec

GLU_ALPHA, GLU_UP_ADD = 1.702, 1.0
DEFAULT_CONTEXT = 131072          # config.json names no longest context; pools are sized by the engine's caller


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"config.json: {where} has no '{key}'")
    return d[key]


@dataclass(frozen=True)
class PotivikConfig:
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
    def from_dict(cls, cfg: dict, tensor_names: Optional[Iterable[str]] = None) -> "PotivikConfig":
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
            m = _need(layer, "mixer", where)
            if kind == "latent_attention":
                for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"):
                    _need(m, k, where + ".mixer")
                rot = _need(m, "rot", where + ".mixer")
                _need(rot, "base", where + ".mixer.rot")
                dims = int(rot.get("dims", m["rot_dim"]))
                if dims % 2 or dims > int(m["rot_dim"]):
                    raise ConfigError(f"{where}: {dims} rotated dimensions must be even and at most rot_dim {m['rot_dim']}")
            elif kind == "mamba2":
                for k in ("heads", "vdim", "state", "groups", "conv"):
                    _need(m, k, where + ".mixer")
                if int(m["heads"]) % int(m["groups"]):
                    raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['groups']} groups")
                if (int(m["heads"]) * int(m["vdim"])) % int(m.get("norm_groups", 1)):
                    raise ConfigError(f"{where}: heads * vdim is not a multiple of norm_groups")
            else:
                raise ConfigError(f"{where}: unknown mixer type '{kind}'; Potivik knows 'latent_attention' and 'mamba2'")
            f = layer.get("mlp")
            if f is not None:
                fk = _need(f, "kind", where + ".mlp")
                if fk == "dense":
                    _need(f, "ff", where + ".mlp"), _need(f, "limit", where + ".mlp")
                elif fk == "moe":
                    r = _need(f, "router", where + ".mlp")
                    ex = _need(f, "expert", where + ".mlp")
                    _need(r, "experts", where + ".mlp.router"), _need(r, "top", where + ".mlp.router")
                    _need(ex, "ff", where + ".mlp.expert"), _need(ex, "limit", where + ".mlp.expert")
                    if not 1 <= int(r["top"]) <= int(r["experts"]):
                        raise ConfigError(f"{where}: top {r['top']} of {r['experts']} experts")
                    if f.get("shared"):
                        _need(f["shared"], "ff", where + ".mlp.shared"), _need(f["shared"], "limit", where + ".mlp.shared")
                else:
                    raise ConfigError(f"{where}: unknown mlp kind '{fk}'; Potivik knows 'dense' and 'moe'")
        if c.get("token_side"):
            _need(c["token_side"], "dim", "token_side")

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    def dump(self) -> dict:
        d = self.to_dict()
        d["mixers (derived)"] = [layer["type"] for layer in self.raw["layers"]]
        return d

    # -- plan ------------------------------------------------------------------------------
    def plan(self) -> ModelPlan:
        c = self.raw
        d, vocab, eps = self.hidden_size, self.vocab_size, self.norm_eps
        n_layers = len(c["layers"])
        side = c.get("token_side") or None

        def norm(tensor):
            return PartSpec("layernorm", {"dim": d, "eps": eps}, {"weight": tensor})

        layers, ignorable = [], []
        if not side:
            ignorable += ["side.embed", "l*.side.*"]
        for i, layer in enumerate(c["layers"]):
            p, m = f"l{i}", layer["mixer"]
            if layer.get("mlp") is None:
                ignorable += [f"{p}.norm2", f"{p}.norm2b"]
            if layer["type"] == "latent_attention":
                mask, rot = m.get("mask") or {}, m["rot"]
                mixer = PartSpec("latent_attention", {
                    "hidden": d, "heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
                    "vdim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]), "scale": float(m["scale"]),
                    "window": int(mask["size"]) if mask.get("size") else None, "rot_base": float(rot["base"]),
                    "rot_dims": int(rot.get("dims", m["rot_dim"])), "eps": eps,
                }, {k: f"{p}.mix.{k}" for k in ("q", "dkv", "dkv.norm", "uk", "uv", "g", "o")})
            else:
                mixer = PartSpec("state_space", {
                    "hidden": d, "heads": int(m["heads"]), "vdim": int(m["vdim"]), "state": int(m["state"]),
                    "groups": int(m["groups"]), "conv": int(m["conv"]), "norm_groups": int(m.get("norm_groups", 1)),
                    "eps": eps,
                }, {k: f"{p}.mix.{k}" for k in ("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o")})
            parts = [("mixer_norm", "norm", norm(f"{p}.norm1")), ("mixer", "mixer", mixer),
                     ("mixer_post_norm", "norm", norm(f"{p}.norm1b"))]
            f = layer.get("mlp")
            if f is not None:
                if f["kind"] == "dense":
                    ffn = PartSpec("clamped_glu", {"hidden": d, "inner": int(f["ff"]), "limit": float(f["limit"]),
                                                   "alpha": GLU_ALPHA, "up_add": GLU_UP_ADD},
                                   {k: f"{p}.mlp.{k}" for k in ("gate", "up", "down")})
                else:
                    E = int(f["router"]["experts"])
                    shared = f.get("shared") or None
                    tensors = {"router": f"{p}.mlp.router"}
                    for e in range(E):
                        tensors.update({f"e{e}.{k}": f"{p}.mlp.e{e}.{k}" for k in ("gate", "up", "down")})
                    if shared:
                        tensors.update({f"shared.{k}": f"{p}.mlp.shared.{k}" for k in ("gate", "up", "down", "sg")})
                    ffn = PartSpec("routed_glu", {
                        "hidden": d, "experts": E, "top": int(f["router"]["top"]), "expert_inner": int(f["expert"]["ff"]),
                        "expert_limit": float(f["expert"]["limit"]), "shared_inner": int(shared["ff"]) if shared else 0,
                        "shared_limit": float(shared["limit"]) if shared else 0.0, "alpha": GLU_ALPHA, "up_add": GLU_UP_ADD,
                    }, tensors)
                parts += [("ffn_norm", "norm", norm(f"{p}.norm2")), ("ffn", "feed_forward", ffn),
                          ("ffn_post_norm", "norm", norm(f"{p}.norm2b"))]
            if side:
                sd = int(side["dim"])
                parts.append(("token_input", "token_input", PartSpec("gated_token_input", {
                    "hidden": d, "dim": sd, "offset": i * sd, "table_width": n_layers * sd, "vocab": vocab, "eps": eps,
                }, {"table": "side.embed", "gate": f"{p}.side.gate", "proj": f"{p}.side.proj", "norm": f"{p}.side.norm"})))
            layers.append(LayerSpec("sandwich_residual", tuple(parts)))

        plan = ModelPlan(
            architecture="Potivik", vocab_size=vocab, hidden_size=d, max_context=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab": vocab, "dim": d}, {"weight": "embed"}),
            layers=tuple(layers), order=tuple(OrderEntry(i) for i in range(n_layers)),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab": vocab, "dim": d, "softcap": float(c.get("logit_softcap") or 0.0)},
                          {"weight": "head"}),
            ignorable=tuple(ignorable),
        )
        plan.validate()
        return plan
