"""Dobepel without a device: its configuration reader, its plan against the checkpoint's tensor names, the cache
needs of its parts in the cache manager's books (kept first pages, members of a parallel mixer, the embedding's
slot), and the plain implementation against itself."""
import copy
import json

import numpy as np
import pytest

import plain_dobepel as D
from dobepel_helpers import CONFIGS, lively_weights, tensor_shapes


def test_the_configuration_reads_every_size_from_the_file_and_writes_it_back():
    from velox_b200.config import ConfigError, DobepelConfig, resolve_architecture
    raw = copy.deepcopy(CONFIGS["odd"])
    assert resolve_architecture(raw).name == "Dobepel"
    cfg = DobepelConfig.from_dict(raw)
    assert (cfg.vocab, cfg.width, cfg.residual_mult, cfg.norm_eps) == (97, 140, 0.5, 1e-5)
    assert (cfg.bigram_buckets, cfg.bigram_mul_prev, cfg.bigram_mul_cur) == (53, 31, 7)
    assert DobepelConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    faults = copy.deepcopy(raw)
    faults["layers"][0]["mixer"]["left"]["kv_heads"] = 3
    faults["layers"][1]["type"] = "serial"
    faults["layers"][2]["mixer"]["right"]["decay"] = [0.5, 0.5]
    faults["layers"][3]["mlp"]["router"]["top"] = 9
    del faults["norm"]
    with pytest.raises(ConfigError) as e:
        DobepelConfig.from_dict(faults)
    assert "norm.eps" in str(e.value)
    faults["norm"] = {"eps": 1e-5}
    with pytest.raises(ConfigError) as e:
        DobepelConfig.from_dict(faults)
    for piece in ("not a multiple of kv_heads", "'serial'", "one number per head", "top (9) exceeds experts (4)"):
        assert piece in str(e.value)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plan_wants_exactly_the_checkpoints_tensors(name):
    from velox_b200.config import DobepelConfig, resolve_architecture
    from velox_b200.models import DecoderModel
    raw = CONFIGS[name]
    model = DecoderModel(resolve_architecture(raw).plan(DobepelConfig.from_dict(raw)))
    assert {s.name: tuple(s.shape) for s in model.tensor_specs()} == tensor_shapes(raw)
    roles = {s.name: s.role for s in model.tensor_specs()}
    assert all(roles[n] == "matrix_f32" for n in roles if n.endswith("mlp.router"))
    assert all(roles[n] == "norm" for n in roles if n.split(".")[-1] in ("norm1", "norm1b", "norm2", "norm2b", "out", "norm"))


def test_cache_needs_kept_first_pages_members_and_the_embeddings_slot():
    from velox_b200.cache import CacheManager
    from velox_b200.config import DobepelConfig, resolve_architecture
    from velox_b200.models import DecoderModel
    from velox_b200.parts import CacheParts, FixedState, PagedKV
    raw = CONFIGS["even"]
    model = DecoderModel(resolve_architecture(raw).plan(DobepelConfig.from_dict(raw)))
    specs = model.cache_specs()
    assert len(specs) == 4 and specs[3] == FixedState((1,), "int32")          # three layers and the embedding
    assert specs[1] == CacheParts((PagedKV(1, 128, 23, 64, 1), FixedState((4, 32, 32), "float32")))
    assert specs[0].parts[0] == PagedKV(2, 64, 40, 0, 4)                         # values of the keys' size: no size of their own
    cache = CacheManager(specs, model.cache_sources(), page_size=8, num_pages=40, max_requests=2, max_blocks=40)
    assert len(cache.groups) == 3 and [g.layers for g in cache.groups] == [[0], [1], [2]]
    assert cache.layer(0).parts[0].group == 0 and cache.layer(0).parts[1].group == -1 and cache.layer(3).parts is None
    cache.add_request("r")
    for n in (30, 1, 1, 100, 1):
        assert cache.reserve("r", n)
        cache.commit("r", n)
    cache.check()
    tables = cache.requests["r"].tables
    # the next query, at position 133, reads keys from 133 + 1 - window on, and the first keep_first ones
    for table, (window, keep) in zip(tables, ((40, 4), (23, 1), (70, 17))):
        first_seen = (133 + 1 - window) // 8
        kept = -(-keep // 8)
        assert all(p >= 0 for p in table[:kept]) and all(p >= 0 for p in table[first_seen:])
        assert all(p < 0 for p in table[kept:first_seen])
    cache.release("r")
    assert cache.free_pages() == [40, 40, 40] and cache.slots.num_free == 2


def test_the_plain_recurrence_carries_its_state_and_the_mask_is_what_it_says():
    rng = np.random.default_rng(0)
    q, k, v = rng.normal(size=(30, 2, 5)), rng.normal(size=(30, 2, 5)), rng.normal(size=(30, 2, 7))
    decay = np.asarray([0.9, 1.0])
    whole, _ = D.decayed_linear_attention(q, k, v, decay)
    a, s = D.decayed_linear_attention(q[:11], k[:11], v[:11], decay)
    b, _ = D.decayed_linear_attention(q[11:], k[11:], v[11:], decay, state=s)
    assert np.allclose(np.concatenate([a, b]), whole)
    # the closed form: o_i = sum_{j <= i} decay^(i - j) (q_i . k_j) v_j
    i, h = 17, 0
    want = sum(decay[h] ** (i - j) * (q[i, h] @ k[j, h]) * v[j, h] for j in range(i + 1))
    assert np.allclose(whole[i, h], want)
    m = D.visible(12, 4, 2)
    assert m[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert m[3].tolist() == [True] * 4 + [False] * 8
    assert D.bigram_rows([3, 4, 5], 7, 10, 1).tolist() == [7, (30 + 4) % 7, (40 + 5) % 7]


def test_the_plain_model_runs_and_the_first_token_takes_the_tables_last_row():
    cfg = CONFIGS["odd"]
    w = lively_weights(cfg, 1)
    ids = [5, 9, 5, 9, 1]
    logits = D.forward(cfg, w, ids)
    assert logits.shape == (5, 97) and np.isfinite(logits).all()
    assert np.allclose(D.forward(cfg, w, ids[:3]), logits[:3])          # causal: a prefix gives the same rows
    w2 = dict(w, bigram=w["bigram"].copy())
    w2["bigram"][cfg["embedding"]["bigram"]["buckets"]] += 1.0
    changed = D.forward(cfg, w2, ids)
    assert not np.allclose(changed[0], logits[0])
