"""Potivik without a GPU: configuration, registry, plan, the loader's check of
a checkpoint against the plan, and the cache manager's bookkeeping for pages
of plain rows."""
from __future__ import annotations

import copy

import pytest
import torch

from gibbs_b200.cache import CacheManager, OutOfPages
from gibbs_b200.config import ConfigError, PotivikConfig, detect, parse_config
from gibbs_b200.parts.base import PagedRows, Runtime, SlotState
from gibbs_b200.weights import TensorDict
from gibbs_b200.weights.loader import WeightBinder, WeightError
from potivik_helpers import CFG_A, CFG_B, make_weights


def test_the_registry_finds_the_design_by_its_name():
    assert detect(CFG_A).name == "Potivik"
    assert detect({"model_type": "potivik"}).name == "Potivik"
    assert isinstance(parse_config(CFG_B), PotivikConfig)


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B])
def test_plan_reads_every_size_from_the_configuration(cfg):
    conf = parse_config(cfg)
    plan = conf.plan()
    assert (plan.vocab_size, plan.hidden_size, len(plan.layers)) == (cfg["vocab"], cfg["width"], len(cfg["layers"]))
    assert conf.to_dict() == cfg and parse_config(conf.to_dict()).plan() == plan
    for i, (layer, spec) in enumerate(zip(cfg["layers"], plan.layers)):
        assert spec.block == "sandwich_residual"
        roles = [r for r, _, _ in spec.parts]
        assert roles[:3] == ["mixer_norm", "mixer", "mixer_post_norm"]
        assert ("ffn" in roles) == (layer["mlp"] is not None)
        assert ("token_input" in roles) == bool(cfg.get("token_side"))
        m, p = layer["mixer"], spec.mixer.params
        if layer["type"] == "latent_attention":
            assert spec.mixer.kind == "latent_attention"
            assert (p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]) == \
                (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"])
            assert p["window"] == (m.get("mask") or {}).get("size") and p["scale"] == m["scale"]
            assert p["rot_base"] == m["rot"]["base"] and p["rot_dims"] == m["rot"]["dims"]
        else:
            assert spec.mixer.kind == "state_space"
            assert (p["heads"], p["vdim"], p["state"], p["groups"], p["conv"], p["norm_groups"]) == \
                (m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"])
        if layer["mlp"] and layer["mlp"]["kind"] == "moe":
            f, q = layer["mlp"], spec.ffn.params
            assert (q["experts"], q["top"], q["expert_inner"], q["expert_limit"]) == \
                (f["router"]["experts"], f["router"]["top"], f["expert"]["ff"], f["expert"]["limit"])
            assert q["shared_inner"] == (f["shared"]["ff"] if f.get("shared") else 0)
        if cfg.get("token_side"):
            t = spec.token_input.params
            assert (t["dim"], t["offset"]) == (cfg["token_side"]["dim"], i * cfg["token_side"]["dim"])
    assert plan.head.params["softcap"] == float(cfg.get("logit_softcap") or 0.0)


def test_configurations_that_are_refused():
    def broken(change):
        c = copy.deepcopy(CFG_A)
        change(c)
        with pytest.raises(ConfigError):
            parse_config(c)
    broken(lambda c: c.pop("vocab"))
    broken(lambda c: c["layers"][0].update(type="attention"))
    broken(lambda c: c["layers"][0]["mixer"].pop("kv_rank"))
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5))
    broken(lambda c: c["layers"][1]["mixer"].update(groups=3))
    broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=7))
    broken(lambda c: c["layers"][1]["mlp"].update(kind="swish"))
    broken(lambda c: c.update(layers=[]))


def _binder(cfg, W):
    return WeightBinder(parse_config(cfg).plan(), TensorDict(W), Runtime(torch.float32, torch.device("cpu")))


def test_the_loader_checks_a_checkpoint_against_the_plan():
    W = make_weights(CFG_A, 1)
    _binder(CFG_A, W).verify()
    missing = {k: v for k, v in W.items() if k != "l3.mlp.e4.down"}
    extra = dict(W, **{"l0.mix.extra": torch.zeros(3)})
    wrong = dict(W, **{"l1.mix.conv": torch.zeros(5, 4)})
    for bad, field, name in ((missing, "missing", "l3.mlp.e4.down"), (extra, "unexpected", "l0.mix.extra"),
                             (wrong, "wrong_shape", "l1.mix.conv")):
        with pytest.raises(WeightError) as e:
            _binder(CFG_A, bad).verify()
        assert name in [x[0] for x in getattr(e.value, field)]
    # a layer without a feed-forward may still carry that sublayer's norms; nothing reads them
    _binder(CFG_A, dict(W, **{"l2.norm2": torch.ones(64), "l2.norm2b": torch.ones(64)})).verify()
    # ... and a model without per-token input may carry the table
    _binder(CFG_B, dict(make_weights(CFG_B, 2), **{"side.embed": torch.zeros(257, 8)})).verify()
    # the table of the per-token input is ONE tensor for all layers
    b = _binder(CFG_A, W)
    assert b.uses["side.embed"] == len(CFG_A["layers"])


def test_pages_of_plain_rows_follow_their_window():
    needs = [([PagedRows(12, window=20)], None), ([SlotState((3, 5))], None), ([PagedRows(7, None)], None)]
    cm = CacheManager(needs, n_pages=6, page_size=8, n_slots=2, dtype=torch.float32, device="cpu", max_context=64)
    assert [g.window for g in cm.groups] == [20, None]
    views = cm.views([torch.zeros(1, 8, dtype=torch.int32)] * 2, torch.zeros(1, dtype=torch.int32), [0])
    assert tuple(views[0][0].pages.shape) == (6, 8, 12) and tuple(views[2][0].pages.shape) == (6, 8, 7)
    assert cm.kv_bytes_per_token() == (12 + 7) * 4
    a = cm.open("a")
    cm.reserve(a, 40)
    cm.advance(a, 40)
    assert cm.free_pages() == [1, 1]
    cm.reserve(a, 41)                      # the step starts at 40: positions before 21 are out of the window
    cm.advance(a, 41)
    assert a.block_tables[0][:2] == [-1, -1] and a.block_tables[0][2] >= 0
    assert cm.free_pages() == [2, 0]
    b = cm.open("b")
    with pytest.raises(OutOfPages):
        cm.reserve(b, 8)                   # the group that keeps everything is full
    cm.close("a")
    cm.reserve(b, 48)
    cm.check()
    cm.close("b")
    assert cm.free_pages() == [6, 6]
