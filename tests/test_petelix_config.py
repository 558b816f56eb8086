"""Petelix without a GPU: configuration, refusals, plan, tensor names, cache bookkeeping of
layers that read another layer's pages, and the plain implementation's own properties."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_petelix as plain
from petelix_helpers import CFG_A, CFG_B, CFG_C, make_weights, random_config


def test_detected_by_its_name_and_laid_out_as_a_plan():
    from gibbs_b200.config import PetelixConfig, parse_config
    conf = parse_config(CFG_A)
    assert isinstance(conf, PetelixConfig)
    plan = conf.plan()
    assert plan.architecture == "Petelix" and len(plan.layers) == 4
    assert [e.reads_cache_of for e in plan.order] == [None, 0, None, 2]
    assert plan.embedding.params["scale"] == 3.0
    m0, m1, m2, m3 = (layer.mixer.params for layer in plan.layers)
    # pages keep what the widest window among their readers needs; a reader keeps its own window
    assert (m0["window"], m0["retain"], m1["window"], m1["retain"]) == (19, 33, 33, 33)
    assert (m2["window"], m2["retain"], m3["window"]) == (None, None, 7)
    assert m1["shares_kv"] and "k" not in plan.layers[1].mixer.tensors and "k.norm" not in plan.layers[1].mixer.tensors
    assert [r for r, _, _ in plan.layers[1].parts] == ["mixer_norm", "mixer"]          # no feed-forward
    f = plan.layers[0].ffn.params
    assert (f["experts"], f["identity"], f["groups"], f["groups_keep"], f["top"]) == (6, 2, 4, 2, 3)
    assert f["scores"] == "softmax" and f["weight_on"] == "output" and f["alpha"] == 1.0 and f["up_add"] == 0.0
    # a reader without a window makes its source keep everything
    pc = parse_config(CFG_C).plan()
    assert pc.layers[1].mixer.params["window"] == 5 and pc.layers[1].mixer.params["retain"] is None


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B, CFG_C, random_config(4), random_config(9)])
def test_tensor_names_and_shapes(cfg):
    from gibbs_b200.config import parse_config
    from gibbs_b200.weights.loader import expected_tensors
    want = {k: tuple(v.shape) for k, v in make_weights(cfg, 1).items()}
    got = {k: d.shapes[0] for k, d in expected_tensors(parse_config(cfg).plan()).items()}
    assert got == want


def _broken(path, value):
    cfg = copy.deepcopy(CFG_A)
    d = cfg
    for k in path[:-1]:
        d = d[k]
    if value is KeyError:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value", [
    (("width",), KeyError), (("norm",), KeyError), (("layers",), []),
    (("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "dim"), KeyError),
    (("layers", 0, "mixer", "kv_heads"), 4),                       # 6 heads over 4
    (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "rot", "dims"), 18),
    (("layers", 1, "mixer", "kv_from"), 1), (("layers", 1, "mixer", "kv_from"), 3),
    (("layers", 3, "mixer", "kv_from"), 1),                        # a layer that has no keys of its own
    (("layers", 1, "mixer", "vdim"), 8),                           # differs from the source's
    (("layers", 0, "mlp", "kind"), "dense"), (("layers", 0, "mlp", "router", "top"), 5),      # only 4 outputs are open
    (("layers", 0, "mlp", "router", "groups", "count"), 3), (("layers", 0, "mlp", "router", "groups", "keep"), 5),
])
def test_refusals(path, value):
    from gibbs_b200.config import ConfigError, parse_config
    with pytest.raises(ConfigError):
        parse_config(_broken(path, value))


def test_cache_groups_follow_what_the_pages_keep():
    """Two sources with different retention make two groups; readers add none."""
    from gibbs_b200.config import parse_config
    from gibbs_b200.parts.base import PagedKV
    plan = parse_config(CFG_A).plan()
    needs = []
    for e in plan.order:
        p = plan.layers[e.layer].mixer.params
        needs.append(([] if p["shares_kv"] else [PagedKV(p["kv_heads"], p["dim"], p["retain"], p["vdim"])], e.reads_cache_of))
    from gibbs_b200.cache import CacheManager
    cm = CacheManager(needs, 8, 16, 2, torch.float32, "cpu", 128)
    assert [g.window for g in cm.groups] == [33, None]
    rc = cm.open("a")
    cm.reserve(rc, 100)
    cm.advance(rc, 100)
    cm.reserve(rc, 101)
    # the windowed group has given back what position 100 can no longer see (pages before (100 - 33 + 1) // 16 = 4)
    assert [p >= 0 for p in rc.block_tables[0]] == [False] * 4 + [True] * 3 and all(p >= 0 for p in rc.block_tables[1])
    views = cm.views([torch.zeros(1, 8, dtype=torch.int32)] * 2, torch.zeros(1, dtype=torch.int32), [0])
    assert views[1][0].k_pages is views[0][0].k_pages and not views[1][0].writable and views[0][0].writable
    assert tuple(views[0][0].v_pages.shape[1:]) == (2, 16, 24) and tuple(views[0][0].k_pages.shape[1:]) == (2, 16, 16)
    cm.close("a")
    cm.check()


def test_plain_implementation_prefix_property_and_sink():
    """Position t's logits do not depend on later tokens; with every score far below zero the sink
    takes the weight and the mixer's output vanishes."""
    W = make_weights(CFG_A, 3)
    ids = [int(v) for v in torch.randint(0, CFG_A["vocab"], (50,), generator=torch.Generator().manual_seed(1))]
    full = plain.forward(CFG_A, W, ids)
    part = plain.forward(CFG_A, W, ids[:31])
    assert torch.allclose(full[:31], part, atol=1e-9)
    q = torch.zeros(3, 1, 4, dtype=torch.float64)
    q[..., 0] = 1.0
    k = -40.0 * q.clone()
    v = torch.ones(3, 1, 2, dtype=torch.float64)
    out = plain.sink_softmax_attention(q, k, v, 1.0, 0.0, None)
    assert float(out.abs().max()) < 1e-15
    out = plain.sink_softmax_attention(q, -k, v, 1.0, 0.0, None)
    assert float((out - 1).abs().max()) < 1e-15
