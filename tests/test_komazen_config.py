"""The Komazen configuration on the CPU: what its config.json turns into, what is refused, what the cache manager is
asked for, and the tensors a model wants."""
import copy

import pytest

import komazen_models as km
from litellmengine_b200.cache import CacheManager, PagedNeed, StateNeed
from litellmengine_b200.config import ConfigError, KomazenConfig, config_from_dict
from litellmengine_b200.parts.model import Model, model_parameters


def test_plan_of_a_configuration():
    cfg = config_from_dict(km.KOMA_A)
    assert isinstance(cfg, KomazenConfig) and cfg.to_dict() == km.KOMA_A
    plan = cfg.plan()
    assert [b.arrangement for b in plan.blocks] == ["post_norm"] * 4
    assert all(b.residual_scale == 1.7 and b.input_conv == 3 for b in plan.blocks)
    assert [s.cache_from for s in plan.order] == [None, None, None, 1]
    a, l, _, r = (b.mixer for b in plan.blocks)
    assert a.kind == "gated_attention" and a.head_temperature and a.log_distance_bias and a.window is None
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.scale) == (4, 2, 16, 24, 0.3)
    assert l.kind == "latent_attention" and l.has_kv and l.window == 9 and dict(l.params)["keep_window"] == 21
    assert not r.has_kv and r.window == 21 and r.position.rotary_dim == 4 and r.position.theta == 500.0
    assert plan.blocks[2].feed_forward is None
    assert dict(plan.blocks[0].feed_forward.params)["activation"] == "gelu_tanh"
    assert plan.embedding_scale == 3.5 and plan.final_norm.kind == "rmsnorm"


def test_tensors_are_the_design_s_names():
    for cfg in (km.KOMA_A, km.KOMA_B, km.KOMA_C, km.KOMA_D, km.KOMA_E):
        want = km.tensor_shapes(cfg)
        got = model_parameters(config_from_dict(cfg).plan())
        assert {n: tuple(p.shape) for n, p in got.items()} == want


def test_cache_needs_pages_for_one_row_per_token_and_kept_rows_per_layer():
    model = Model(config_from_dict(km.KOMA_A).plan(), dtype="float32", device="meta")
    needs = model.stage_needs()
    rows = StateNeed((2, 2, 40), "float32", name="block")
    assert needs[0] == [PagedNeed(2, 16, None, 24), rows]
    assert needs[1] == [PagedNeed(1, 16, 21, 0), rows]                  # one row [latent | rotated key part], no values
    assert needs[2] == [PagedNeed(1, 8, None, None), StateNeed((1, 2, 40), "float32", name="block")]     # no feed-forward
    assert needs[3] == [("borrow", 1), rows]
    cache = CacheManager(needs, 16, 256, 3)
    assert cache.stage_group[3] == cache.stage_group[1] and set(cache.stage_state) == {(s, "block") for s in range(4)}
    # one tap keeps nothing
    assert all(not any(isinstance(n, StateNeed) for n in (ns if isinstance(ns, list) else [ns]))
               for ns in Model(config_from_dict(km.KOMA_B).plan(), dtype="float32", device="meta").stage_needs())
    # a window the reader widens; without a window anywhere among the readers everything stays
    b = Model(config_from_dict(km.KOMA_B).plan(), dtype="float32", device="meta").stage_needs()
    assert b[0] == PagedNeed(1, 32, None, 0)


def _broken(path, value, base=km.KOMA_A):
    d = copy.deepcopy(base)
    node = d
    for key in path[:-1]:
        node = node[key]
    if value is None:
        node.pop(path[-1])
    else:
        node[path[-1]] = value
    return d


@pytest.mark.parametrize("path,value", [
    (("postln_alpha",), None), (("canon",), None), (("canon", "taps"), 0), (("norm", "eps"), 0.0),
    (("layers", 0, "type"), "retention"), (("layers", 0, "mixer", "heads"), 3), (("layers", 1, "mixer", "rot", "dims"), 3),
    (("layers", 1, "mixer", "rot", "dims"), 6), (("layers", 3, "mixer", "kv_from"), 3), (("layers", 3, "mixer", "kv_from"), 0),
    (("layers", 3, "mixer", "kv_rank"), 10), (("layers", 3, "mixer", "rot", "base"), 100.0), (("layers", 1, "mixer", "q_rank"), None),
    (("layers", 0, "mlp", "kind"), "moe"), (("layers", 1, "mixer", "kv_from"), 3)])
def test_refused_configurations(path, value):
    with pytest.raises(ConfigError):
        config_from_dict(_broken(path, value))
