"""Lopazen without a GPU: reading the configuration, the order of runs, and the plain
implementation against itself (a prompt's logits do not depend on what follows it)."""

import copy
import json

import pytest
import torch

from enginekernel_b200 import registry
from enginekernel_b200.config.base import ConfigError
from enginekernel_b200.config.lopazen import LopazenConfig
from enginekernel_b200.engine.model import expected_tensors, ignorable_tensors
from tests.plain import lopazen_models as models
from tests.plain import lopazen_plain as plain


def test_registered_and_chosen_by_the_architecture_key(tmp_path):
    assert "Lopazen" in registry.architectures()
    folder = models.write_folder(str(tmp_path), models.LOOPED, {})
    cfg = registry.config_from_folder(folder)
    assert isinstance(cfg, LopazenConfig)
    assert cfg.to_dict() == models.LOOPED
    assert LopazenConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg


@pytest.mark.parametrize("tag", list(models.SHAPES))
def test_runs_and_tensors_follow_the_configuration(tag):
    raw = models.SHAPES[tag]
    cfg = LopazenConfig.from_dict(raw)
    spec = registry.model_spec_for(cfg)
    runs = plain.layer_runs(raw)
    assert [(r.layer, r.add_embedding) for r in spec.schedule] == runs
    assert [r.cache for r in spec.schedule] == list(range(len(runs)))        # every pass its own entry
    want = models.tensor_shapes(raw)
    got = {name: tuple(ts.shape) for name, ts in expected_tensors(spec).items()}
    assert got == want
    assert spec.embedding_multiplier == raw["embedding"]["scale"]
    for i, layer in enumerate(raw["layers"]):
        assert (f"l{i}.norm2" in ignorable_tensors(spec)) == (layer["mlp"] is None)
        assert (spec.layers[i].feed_forward is None) == (layer["mlp"] is None)
        p = spec.layers[i].mixer.params
        assert (p["num_heads"], p["num_kv_heads"], p["head_dim"]) == (
            layer["mixer"]["heads"], layer["mixer"]["kv_heads"], layer["mixer"]["dim"])
        assert p["scale"] == layer["mixer"]["scale"] and p["sink"] == 0.0 and p["position"] is None


def test_the_order_of_runs():
    cfg = LopazenConfig.from_dict(models.LOOPED)
    assert cfg.runs() == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False),
                          (3, False)]
    assert LopazenConfig.from_dict(models.ODD).runs() == [(0, False), (0, True), (1, False)]
    assert LopazenConfig.from_dict(models.FLAT).runs() == [(0, False), (1, False)]
    assert LopazenConfig.from_dict(models.WIDE).runs() == [(0, False), (1, False)]


@pytest.mark.parametrize("change,match", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "type"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 4), "multiple"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("vdim", 16), "vdim"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"), "kind"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c["loop"].__setitem__("times", 0), "times"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 2.5), "integer"),
])
def test_bad_configurations_are_refused(change, match):
    raw = copy.deepcopy(models.LOOPED)
    change(raw)
    with pytest.raises(ConfigError, match=match):
        LopazenConfig.from_dict(raw)


def test_a_configuration_without_loop_or_temperature():
    raw = copy.deepcopy(models.FLAT)
    raw["layers"][0]["mixer"].pop("q_temp")
    cfg = LopazenConfig.from_dict(raw)
    assert cfg.loop is None and cfg.layers[0].mixer.q_temp_coef == 0.0
    assert registry.model_spec_for(cfg).layers[0].mixer.params["query_temperature"] is None


def test_plain_model_is_causal_and_the_sink_takes_weight():
    cfg = models.LOOPED
    w = models.make_tensors(cfg, 3)
    ids = models.random_prompts(cfg, [40], seed=1)[0]
    full = plain.logits(cfg, w, ids)
    assert torch.allclose(full[:25], plain.logits(cfg, w, ids[:25]), atol=1e-5)
    scores = torch.tensor([[0.0, 1.0, -1.0]], dtype=torch.float64)
    p = plain.sink_softmax(scores, torch.ones(1, 3, dtype=torch.bool))
    assert abs(float(p.sum()) - (1 - 1 / (1 + float(torch.exp(scores).sum())))) < 1e-12
    t = plain.query_temperature([0, 14, 15, 16, 31, 32], 0.5, 16)
    assert t[0] == 1 and t[1] == 1 and t[2] > 1 and t[2] == t[3] and t[4] > t[3] and t[5] == t[4]


def test_random_model_folder_reads_back(tmp_path):
    from enginekernel_b200.weights.checkpoint import CheckpointIndex, check_against
    from enginekernel_b200.weights.random_init import write_random_model
    cfg = LopazenConfig.from_dict(models.ODD)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=4)
    again = registry.config_from_folder(folder)
    assert again == cfg
    spec = registry.model_spec_for(again)
    check_against(CheckpointIndex(folder), expected_tensors(spec), ignorable_tensors(spec))
