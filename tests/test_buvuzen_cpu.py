"""Buvuzen without a GPU: the configuration reader and its faults, the plan (tensor names, running order of layers
that share tensors, cache needs), random-model folders, and the plain implementation's own mechanisms on cases worked
out by hand."""
import copy
import json

import numpy as np
import pytest

import plain_buvuzen as B
from buvuzen_helpers import CONFIGS, EVEN, ODD, lively_weights, tensor_shapes


def typed(cfg):
    from velox_b200.config import BuvuzenConfig
    return BuvuzenConfig.from_dict(cfg)


def test_the_registry_finds_the_design_by_its_name_and_reads_every_key():
    from velox_b200.config.registry import resolve_architecture
    arch = resolve_architecture(ODD)
    assert arch.name == "Buvuzen"
    cfg = arch.config_class.from_dict(ODD)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.embedding_scale, cfg.logit_scale) == (97, 140, 1e-5, 0.7, 1.0)
    assert typed(cfg.to_dict()) == cfg
    assert [cfg.weights_layer(i) for i in range(4)] == [0, 1, 0, 3]
    assert [typed(EVEN).weights_layer(i) for i in range(5)] == [0, 1, 2, 0, 0]   # (a chain ends at the layer that has tensors)


@pytest.mark.parametrize("change,says", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "multiple"),
    (lambda c: c["layers"][0].update(type="recurrent"), "type"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][2].update(weights_of=9), "weights_of"),
    (lambda c: c["layers"][0].update(weights_of=2), "circle"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),          # two kept groups of two outputs
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4), "groups"),
    (lambda c: c["layers"][3]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][3]["mlp"]["expert"].update(ff=0), "ff"),
])
def test_a_configuration_that_cannot_be_a_model_is_refused(change, says):
    from velox_b200.config import ConfigError
    cfg = copy.deepcopy(ODD)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        typed(cfg)
    assert says in str(e.value)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plan_names_the_tensors_of_the_layers_that_own_them(name):
    from velox_b200.models import DecoderModel
    from velox_b200.models.buvuzen import buvuzen_plan
    cfg = CONFIGS[name]
    plan = buvuzen_plan(typed(cfg))
    model = DecoderModel(plan)
    got = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert got == tensor_shapes(cfg)
    owners = [i for i, lay in enumerate(cfg["layers"]) if lay.get("weights_of") is None]
    assert [owners[k] for k in plan.order] == B.layer_sources(cfg)
    # every place of the running order has a cache of its own, with its layer's window and sizes
    specs = model.cache_specs()
    assert len(specs) == len(cfg["layers"])
    for spec, src in zip(specs, B.layer_sources(cfg)):
        m = cfg["layers"][src]["mixer"]
        assert (spec.num_kv_heads, spec.head_dim, spec.value_dim, spec.window) == \
            (m["kv_heads"], m["dim"], m["vdim"], (m.get("mask") or {}).get("size", 0))


def test_a_random_model_folder_has_the_plans_tensors(tmp_path):
    from velox_b200.weights import write_random_model
    from velox_b200.weights.safetensors_io import SafetensorsFile
    write_random_model(str(tmp_path), typed(ODD), seed=5)
    assert json.load(open(tmp_path / "config.json"))["architecture"] == "Buvuzen"
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    assert {k: tuple(f.info(k)[1]) for k in f.keys()} == tensor_shapes(ODD)


def test_the_sink_takes_its_share_of_every_row():
    scores = np.log(np.asarray([[1.0, 2.0, 5.0], [3.0, 1.0, 1.0]]))
    vis = np.asarray([[True, True, False], [True, True, True]])
    a = B.sink_softmax(scores, vis, np.log(3.0))
    assert np.allclose(a, [[1 / 6, 2 / 6, 0.0], [3 / 8, 1 / 8, 1 / 8]])
    # a sink far above every score leaves almost nothing; one far below changes nothing
    assert B.sink_softmax(scores, vis, 50.0).max() < 1e-18
    assert np.allclose(B.sink_softmax(scores, vis, -50.0).sum(axis=1), 1.0)


def test_the_window_counts_the_query_itself():
    v = B.window_visible(6, 3)
    assert [int(r.sum()) for r in v] == [1, 2, 3, 3, 3, 3] and v[5, 3] and not v[5, 2] and not v[2, 3]
    assert B.window_visible(4, 0).sum() == 10


def test_groups_hide_their_outputs_even_where_choice_scores_are_negative():
    # three groups of two; the middle group holds the single best value, the last group the next best
    choice = np.asarray([[-0.5, -0.4, 0.9, -0.9, 0.1, 0.05]])
    assert B.group_limited_choice(choice, 3, 2, 3).tolist() == [[2, 4, 5]]        # (-0.9 of a kept group never beats 0.05, but ...)
    assert B.group_limited_choice(choice, 3, 2, 4).tolist() == [[2, 4, 5, 3]]     # ... it is chosen before any output of a dropped group
    assert B.group_limited_choice(choice, 3, 1, 2).tolist() == [[2, 3]]
    assert B.group_limited_choice(choice, 1, 1, 2).tolist() == [[2, 4]]
    assert B.group_limited_choice(np.zeros((1, 4)), 2, 1, 2).tolist() == [[0, 1]]  # equal values: the lower index first


def test_routing_weights_are_scores_times_the_multiplier_and_identity_experts_return_the_token():
    rng = np.random.default_rng(3)
    K, T = 16, 5
    h = rng.normal(size=(T, K))
    w = {"router": rng.normal(size=(4, K)), "correction": np.asarray([0.0, 0.0, 5.0, 5.0])}
    cfg = {"router": {"experts": 2, "identity": 2, "top": 2, "scale": 3.0}, "expert": {"ff": 8}, "shared": None}
    chosen, weights, s, _ = B.route(h, w["router"], w["correction"], cfg["router"])
    assert (np.sort(chosen, axis=1) == [2, 3]).all()                  # the correction decides ...
    assert np.allclose(weights, 3.0 * np.take_along_axis(s, chosen, 1))   # ... and stays out of the weights
    out = B.routed_ff(h, w, "", cfg)
    assert np.allclose(out, h * weights.sum(axis=1, keepdims=True))


def test_layers_that_share_tensors_are_the_same_function_at_another_place():
    cfg = copy.deepcopy(ODD)
    w = lively_weights(cfg, 1)
    toks = [int(t) for t in np.random.default_rng(0).integers(0, cfg["vocab"], 12)]
    twin = copy.deepcopy(cfg)
    del twin["layers"][2]["weights_of"]
    w2 = dict(w)
    w2.update({k.replace("l0.", "l2.", 1): v for k, v in w.items() if k.startswith("l0.")})
    assert np.array_equal(B.forward(cfg, w, toks), B.forward(twin, w2, toks))
