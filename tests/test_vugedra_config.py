"""The Vugedra configuration on the CPU: what its config.json turns into, what is refused, what the cache manager is
asked for, the tensors a model wants, and the pages of a window that keeps a request's first positions."""
import copy
import math

import pytest

import vugedra_models as vm
from litellmengine_b200.cache import CacheManager, PagedNeed, StateNeed
from litellmengine_b200.config import ConfigError, VugedraConfig, config_from_dict
from litellmengine_b200.config.specs import PositionSpec
from litellmengine_b200.parts.model import Model, model_parameters
from litellmengine_b200.parts.registry import lookup


def test_plan_of_a_configuration():
    cfg = config_from_dict(vm.VUG_A)
    assert isinstance(cfg, VugedraConfig) and cfg.to_dict() == vm.VUG_A
    plan = cfg.plan()
    assert [s.block for s in plan.order] == [0, 1, 2, 0, 3]          # the fourth layer runs the first one's tensors
    assert all(b.arrangement == "sandwich_norm" and b.mixer_norm.kind == "tanh" and b.mixer_post_norm.kind == "tanh" for b in plan.blocks)
    a, g, l, _ = (b.mixer for b in plan.blocks)
    assert a.kind == "gated_attention" and a.qk_norm_scope == "projection" and a.bias and a.output_gate_scope == "head"
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.scale) == (4, 2, 16, 24, 0.3)
    assert (a.window, a.keep_first, a.softmax_sink) == (9, 3, 0.0)
    assert a.position.kind == "rope_pairs" and a.position.rotary_dim == 8 and a.position.theta == 500.0
    assert dict(a.position.params)["scaling"] == (4.0, 16.0, 4.0, 0.5)
    assert abs(dict(a.position.params)["magnitude"] - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    assert g.kind == "gla" and dict(g.params)["tau"] == 4.0
    assert l.kind == "latent_attention" and l.window is None and l.output_gate_scope == "head" and l.position.kind == "rope_pairs"
    ff = dict(plan.blocks[1].feed_forward.params)
    assert (ff["experts"], ff["top"], ff["identity"], ff["shared"], ff["score"], ff["activation"]) == (5, 2, 1, 24, "softmax", "silu")
    assert plan.blocks[0].feed_forward.kind == "swiglu" and plan.blocks[3].feed_forward is None
    assert plan.final_norm.kind == "tanh"


def test_tensors_are_the_design_s_names():
    for cfg in (vm.VUG_A, vm.VUG_B, vm.VUG_C, vm.VUG_D, vm.VUG_E):
        want = vm.tensor_shapes(cfg)
        got = model_parameters(config_from_dict(cfg).plan())
        assert set(got) == set(want)
        for n, p in got.items():       # -1: the rank of the decay projection, which only the tensors know
            assert len(p.shape) == len(want[n]) and all(a in (-1, b) for a, b in zip(p.shape, want[n])), n


def test_a_layer_may_run_a_later_layer_s_tensors():
    plan = config_from_dict(vm.VUG_C).plan()
    assert [s.block for s in plan.order] == [2, 0, 1, 2] and plan.blocks[2].weight_prefix == "l3"


def test_what_is_refused():
    def broken(change):
        d = copy.deepcopy(vm.VUG_A)
        change(d)
        with pytest.raises(ConfigError):
            config_from_dict(d)
    broken(lambda d: d["layers"][0].update(type="conv"))
    broken(lambda d: d["layers"][0]["mixer"].update(kv_heads=3))
    broken(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7))
    broken(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=18))
    broken(lambda d: d["layers"][0]["mixer"]["mask"].update(keep_first=-1))
    broken(lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"))
    broken(lambda d: d["layers"][1]["mlp"]["router"].update(top=7))
    broken(lambda d: d["layers"][1]["mlp"].update(kind="sparse"))
    broken(lambda d: d["layers"][3].update(weights_of=9))
    broken(lambda d: d["layers"][0].update(weights_of=3))          # a circle
    broken(lambda d: d.pop("norm"))


def test_options_that_may_be_absent():
    d = copy.deepcopy(vm.VUG_A)
    m = d["layers"][0]["mixer"]
    del m["mask"], m["rot"]
    d["layers"][1]["mlp"]["router"].pop("identity")
    d["layers"][1]["mlp"].pop("shared")
    plan = config_from_dict(d).plan()
    a = plan.blocks[0].mixer
    assert a.window is None and a.keep_first == 0 and a.position.kind == "none" and a.softmax_sink == 0.0
    ff = dict(plan.blocks[1].feed_forward.params)
    assert ff["identity"] == 0 and ff["shared"] is None


def test_stretched_frequencies():
    """The table against the rule written out: pairs whose wavelength exceeds the original context are slowed by the
    factor, short ones stay, a ramp between."""
    dims, base, factor, original, fast, slow = 12, 300.0, 4.0, 16.0, 4.0, 0.5
    pos = lookup("position", "rope_pairs")(PositionSpec("rope_pairs", base, dims, (("scaling", (factor, original, fast, slow)),
                                                                                   ("magnitude", 1.3))), 16, "cpu")
    pair = lambda t: dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(base))
    lo, hi = max(math.floor(pair(fast)), 0), min(math.ceil(pair(slow)), dims - 1)
    for i, got in enumerate(pos.freq.tolist()):
        f = base ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert abs(got - (f / factor * ramp + f * (1 - ramp))) < 1e-7 * f
    assert pos.kernel_args()[1:] == (12, 1.3, True)
    plain = lookup("position", "rope_pairs")(PositionSpec("rope_pairs", base, dims), 16, "cpu")
    assert abs(plain.freq[3].item() - base ** (-0.5)) < 1e-8 and plain.magnitude == 1.0


def test_cache_needs():
    model = Model(config_from_dict(vm.VUG_A).plan(), dtype="float32", device="meta")
    needs = model.stage_needs()
    assert needs[0] == PagedNeed(2, 16, 9, 24, 3) == needs[3]          # two stages, one layer's tensors, a cache each
    assert needs[1] == StateNeed((3, 8 * 12), "float32") or isinstance(needs[1], StateNeed)
    assert needs[2] == PagedNeed(1, 12 + 4, None, 0)
    m = CacheManager(needs, page_size=16, max_total_tokens=128, max_slots=2)
    assert len(m.groups) == 2 and m.groups[0].stages == [0, 3]


@pytest.mark.parametrize("page,window,keep", [(4, 10, 3), (4, 10, 4), (4, 10, 9), (4, 3, 14), (8, 5, 0), (4, 6, 40)])
def test_window_with_kept_first_positions_gives_back_only_the_pages_between(page, window, keep):
    """As the window passes, pages behind it go back, but never the pages that hold the first `keep` positions; what a
    later query may read is always held; a released slot leaves nothing behind, and its pages serve the next request."""
    need = PagedNeed(1, 8, window, None, keep)
    m = CacheManager([need], page_size=page, max_total_tokens=64, max_slots=2)
    g = m.groups[0]
    head = -(-keep // page)
    for _ in range(2):                      # the second request runs in pages the first one gave back
        s = m.admit()
        for n in range(1, 49):
            m.ensure(s, n)
            m.commit(s, n)
            held = set(g.held_pages(s))
            assert len(held) == len(g.held_pages(s))
            # the next query sits at position n: it sees the kept positions and keys n - window + 1 .. n
            wanted = set(range(min(keep, n))) | set(range(max(0, n - window + 1), n))
            for pos in wanted:
                assert int(g.table[s, pos // page]) in held, (n, pos)
            first_needed = max(0, n - window + 1) // page
            expect = len(set(range(min(head, -(-n // page)))) | set(range(first_needed, -(-n // page))))
            assert len(held) == expect, (n, held)
            m.check_invariants()
        other = m.admit()
        m.ensure(other, 5)
        m.release(s)
        m.release(other)
        assert g.pool.free_count == g.pool.num_pages
        m.check_invariants()
