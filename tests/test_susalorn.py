"""Susalorn without a GPU: reading the configuration, the order of runs, the tensors the model
asks for, the stretched rotation's tables, and the plain implementation against itself."""

import copy
import json
import math

import pytest
import torch

from enginekernel_b200 import registry
from enginekernel_b200.config.base import ConfigError
from enginekernel_b200.config.susalorn import SusalornConfig
from enginekernel_b200.engine.model import expected_tensors, ignorable_tensors
from enginekernel_b200.parts.spec import PartSpec
from tests.plain import susalorn_models as models
from tests.plain import susalorn_plain as plain


def test_registered_and_chosen_by_the_architecture_key(tmp_path):
    assert "Susalorn" in registry.architectures()
    folder = models.write_folder(str(tmp_path), models.MIXED, {})
    cfg = registry.config_from_folder(folder)
    assert isinstance(cfg, SusalornConfig)
    assert cfg.to_dict() == models.file_config(models.MIXED)
    assert SusalornConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg


@pytest.mark.parametrize("tag", list(models.SHAPES))
def test_runs_parts_and_tensors_follow_the_configuration(tag):
    raw = models.SHAPES[tag]
    cfg = SusalornConfig.from_dict(models.file_config(raw))
    spec = registry.model_spec_for(cfg)
    runs = plain.layer_runs(raw)
    assert [r.layer for r in spec.schedule] == runs
    assert [r.cache for r in spec.schedule] == list(range(len(runs)))        # every pass its own entry
    assert not any(r.add_embedding for r in spec.schedule)
    want = models.tensor_shapes(raw)
    got = expected_tensors(spec)
    assert set(got) == set(want)
    for name, shape in want.items():
        assert got[name].fits(shape), (name, got[name].shape, shape)
    free = sorted(n for n, ts in got.items() if -1 in ts.shape)              # sizes only the file knows
    assert all(n.rsplit(".", 1)[-1] in ("a1", "a2", "g1", "g2") for n in free)
    for i, layer in enumerate(raw["layers"]):
        ls = spec.layers[i]
        assert ls.block.kind == ("hyper_connections" if "streams" in raw else "pre_norm")
        assert ls.mixer.kind == layer["type"]
        assert (ls.feed_forward is None) == (layer["mlp"] is None)
        assert (f"l{i}.norm2" in ignorable_tensors(spec)) == (layer["mlp"] is None)
        if layer["mlp"] is not None:
            assert ls.feed_forward.kind == {"dense": "gated_mlp", "moe": "routed_experts"}[layer["mlp"]["kind"]]


def test_the_order_of_runs():
    f = lambda c: SusalornConfig.from_dict(models.file_config(c)).runs()
    assert f(models.MIXED) == [0, 1, 2, 1, 2]
    assert f(models.PLAIN) == [0, 1]
    assert f(models.ODD) == [0, 1, 0, 1, 2]
    assert f(models.WIDE) == [0, 1]


@pytest.mark.parametrize("change,match", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].pop("base"), "base"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0].update(type="window"), "not a Susalorn mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "not a Susalorn feed-forward"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c["loop"].update(stop=9), "loop"),
])
def test_bad_configurations_are_refused_by_name(change, match):
    raw = copy.deepcopy(models.file_config(models.MIXED))
    change(raw)
    with pytest.raises(ConfigError, match=match):
        SusalornConfig.from_dict(raw)


@pytest.mark.parametrize("dims,base,scaling", [(16, 10000.0, (8.0, 1024, 32.0, 1.0)), (8, 100.0, (4.0, 64, 8.0, 1.0)),
                                               (32, 50000.0, None), (4, 10.0, (2.0, 16, 2.0, 1.0))])
def test_stretched_rotation_tables(dims, base, scaling):
    """cos and sin of the part against the plain frequencies, factor on both included; without
    scaling the part is the plain rotation."""
    from enginekernel_b200.parts.rope import RopeStretched
    params = {"rotary_dim": dims, "theta": base}
    sc = None
    if scaling is not None:
        sc = dict(zip(("factor", "original", "fast", "slow"), scaling))
        params.update(sc)
    part = RopeStretched(PartSpec("rope_stretched", params), torch.float32, "cpu")
    part.prepare(300)
    f, mult = plain.rotary_frequencies(dims, base, sc)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    assert part.cos.shape == (300, dims // 2)
    assert (part.cos.double() - torch.cos(ang) * mult).abs().max() < 1e-6
    assert (part.sin.double() - torch.sin(ang) * mult).abs().max() < 1e-6
    if scaling is None:
        assert mult == 1.0
    else:
        assert abs(mult - (0.1 * math.log(scaling[0]) + 1.0)) < 1e-12
        plain_f, _ = plain.rotary_frequencies(dims, base, None)
        assert (f <= plain_f + 1e-15).all() and (f >= plain_f / scaling[0] - 1e-15).all()


def test_plain_model_is_causal_and_the_scan_matches_its_closed_form():
    cfg = models.MIXED
    w = models.make_tensors(cfg, 3)
    ids = models.random_prompts(cfg, [40], seed=1)[0]
    full = plain.logits(cfg, w, ids)
    assert (plain.logits(cfg, w, ids[:17]) - full[:17]).abs().max() < 1e-9
    # one token through the delta rule from a zero state: o = beta (k . q) v
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 2, 5, generator=g, dtype=torch.float64), torch.randn(1, 2, 5, generator=g, dtype=torch.float64)
    v, beta = torch.randn(1, 2, 3, generator=g, dtype=torch.float64), torch.rand(1, 2, generator=g, dtype=torch.float64)
    o = plain.delta_scan(q, k, v, beta, torch.rand(1, 2, 5, generator=g, dtype=torch.float64))
    assert (o - beta[..., None] * (q * k).sum(-1, keepdim=True) * v).abs().max() < 1e-12


def test_plain_router_keeps_to_the_best_groups():
    g = torch.Generator().manual_seed(2)
    h = torch.randn(50, 12, generator=g, dtype=torch.float64)
    wr = torch.randn(8, 12, generator=g)
    idx, wt = plain.route(h, wr, {"experts": 8, "top": 2, "scale": 1.7, "groups": {"count": 4, "keep": 1}})
    assert ((idx[:, 0] // 2) == (idx[:, 1] // 2)).all()           # both from one group of two neighbours
    assert (wt.sum(-1) - 1.7).abs().max() < 1e-9
    idx2, _ = plain.route(h, wr, {"experts": 8, "top": 2, "scale": 1.0})
    s = torch.softmax(h @ wr.double().T, -1)
    assert (idx2 == s.topk(2, -1).indices).all()
