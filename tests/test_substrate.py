"""Serialization, pytree, wrapper types, RNG keys, schedules, loss scaler, profiling."""
import dataclasses
import math
from collections import namedtuple

import pytest
import torch

from opaque_b200 import pytree as pt
from opaque_b200.precision import all_finite, loss_scaler
from opaque_b200.profiling import PerfState, StepPerf, perf_tracker, step_perf
from opaque_b200.random import RngKey, fold_in, generator_from_key, key, split
from opaque_b200 import scheduling as S
from opaque_b200.serialization import from_state_dict, register_serializer, state_dict
from opaque_b200.types import ClippedPytree, NoisedPytree, PerGroup, clipped, noised


@dataclasses.dataclass(frozen=True)
class Inner:
    a: int
    b: float


@dataclasses.dataclass(frozen=True)
class Outer:
    inner: Inner
    items: tuple
    table: dict


def test_state_dict_round_trip_and_paths():
    obj = Outer(Inner(1, 2.5), (3, [4, 5]), {"x": 6, "y": None})
    sd = state_dict(obj)
    assert sd == {"inner.a": 1, "inner.b": 2.5, "items[0]": 3, "items[1][0]": 4, "items[1][1]": 5,
                  "table.x": 6, "table.y": None}
    template = Outer(Inner(0, 0.0), (0, [0, 0]), {"x": 0, "y": 1})
    assert from_state_dict(template, sd) == obj


def test_missing_leaves_keep_template_and_unknown_leaf_fails_closed():
    sd = {"inner.a": 9}
    out = from_state_dict(Outer(Inner(0, 1.5), (), {}), sd)
    assert out.inner == Inner(9, 1.5)

    class Opaque:
        pass
    with pytest.raises(TypeError):
        state_dict({"k": Opaque()})
    with pytest.raises(TypeError):
        from_state_dict({"k": Opaque()}, {})


def test_registered_serializer_and_mro():
    class Base:
        def __init__(self, v):
            self.v = v

    class Child(Base):
        pass
    register_serializer(Base, lambda o: {"v": o.v}, lambda t, sd: type(t)(sd["v"]))
    sd = state_dict({"c": Child(7)})
    assert sd == {"c.v": 7}
    assert from_state_dict({"c": Child(0)}, sd)["c"].v == 7


def test_rng_key_state_dict():
    k = fold_in(key(5), 3)
    assert from_state_dict(key(0), state_dict(k)) == k


def test_pytree_flatten_map_partition_merge():
    NT = namedtuple("NT", "p q")
    tree = {"b": [torch.ones(2), NT(torch.zeros(1), None)], "a": (torch.full((3,), 2.0),)}
    paths, leaves, td = pt.tree_flatten_with_paths(tree)
    assert paths == [("a", 0), ("b", 0), ("b", 1, "p")]
    rebuilt = pt.tree_unflatten(td, leaves)
    assert rebuilt["b"][1].q is None and torch.equal(rebuilt["a"][0], tree["a"][0])
    doubled = pt.tree_map(lambda x: x * 2, tree)
    assert float(doubled["a"][0][0]) == 4.0
    yes, no = pt.partition(lambda p, x: p[0] == "a", tree)
    merged = pt.merge(yes, no)
    assert torch.equal(merged["b"][0], tree["b"][0]) and torch.equal(merged["a"][0], tree["a"][0])
    assert math.isclose(float(pt.global_norm(tree)), math.sqrt(2 + 12), rel_tol=1e-6)


def test_global_norm_accumulates_wide():
    big = {"x": torch.full((1 << 16,), 1e-3, dtype=torch.bfloat16)}
    assert math.isclose(float(pt.global_norm(big)), float(torch.tensor(1e-3, dtype=torch.bfloat16)) * 256, rel_tol=1e-4)


def test_wrapper_type_algebra():
    c = clipped({"w": torch.ones(2)}, 2.0)
    d = c / 4
    assert isinstance(d, ClippedPytree) and d.max_norm == 0.5 and float(d.pytree["w"][0]) == 0.25
    n = noised({"w": torch.ones(2)}, 2.0, 3.0) * -2
    assert isinstance(n, NoisedPytree) and n.max_norm == 4.0 and n.noise_stddev == 6.0
    for bad in (lambda: c + c, lambda: c - 1, lambda: c ** 2, lambda: 1 / c):
        with pytest.raises(TypeError):
            bad()
    with pytest.raises(TypeError):
        c * torch.ones(2)
    assert c.noise_stddev_for(noise_multiplier=1.5) == 3.0


def test_per_group_and_optimal_allocation():
    pg = PerGroup({"a": "g1", ("b", "w"): "g2"}, {"g1": 3.0, "g2": 4.0})
    assert pg.effective == 5.0 and pg.for_path("a") == 3.0 and (2 * pg).values["g2"] == 8.0
    c = clipped({"a": torch.zeros(1), "b": {"w": torch.zeros(1)}}, pg)
    std = c.noise_stddev_for(noise_multiplier=2.0)
    assert math.isclose(std.values["g1"], 2.0 * math.sqrt(3.0 * 7.0))
    # Mahalanobis sensitivity equals 1/nm^2 exactly
    assert math.isclose(sum(pg.values[g] ** 2 / std.values[g] ** 2 for g in pg.values), 0.25)
    assert c.noise_stddev_for(noise_multiplier=2.0, allocation="isotropic") == 10.0


def test_fold_in_algebra_and_golden_values():
    k = key(42)
    assert key(-1).seed == 2 ** 64 - 1
    assert fold_in(k, 1, "a") == fold_in(fold_in(k, 1), "a")
    assert split(k, 3) == tuple(fold_in(k, i) for i in range(3))
    assert fold_in(k, 0) != fold_in(k, "0")
    # BLAKE2b-64 over (seed as 16-byte LE signed, '|', item, '|'), little-endian digest
    import hashlib
    h = hashlib.blake2b(digest_size=8)
    h.update((42).to_bytes(16, "little", signed=True) + b"|" + (7).to_bytes(16, "little", signed=True) + b"|")
    assert fold_in(k, 7).seed == int.from_bytes(h.digest(), "little")
    g1, g2 = generator_from_key(k), generator_from_key(k)
    assert torch.equal(torch.rand(4, generator=g1), torch.rand(4, generator=g2))
    with pytest.raises(TypeError):
        fold_in(k, 1.5)
    with pytest.raises(ValueError):
        fold_in(k)


def test_schedules_values():
    assert S.constant_schedule(0.3)(10) == 0.3
    lin = S.linear_schedule(1.0, 0.0, 10, transition_begin=5)
    assert lin(0) == 1.0 and lin(10) == 0.5 and lin(100) == 0.0
    cos = S.cosine_schedule(1.0, 0.0, 10)
    assert math.isclose(cos(5), 0.5) and math.isclose(cos(10), 0.0, abs_tol=1e-12)
    assert math.isclose(S.exponential_schedule(1.0, 0.5, transition_steps=2)(4), 0.25)
    assert S.exponential_schedule(1.0, 0.5, staircase=True, transition_steps=2)(3) == 0.5
    assert S.exponential_schedule(1.0, 0.5, end_value=0.3)(10) == 0.3
    assert math.isclose(S.inverse_sqrt_schedule(2.0, 4)(4), 2.0 / math.sqrt(2))
    assert math.isclose(S.one_minus_sqrt_schedule(1.0, 0.0, 4)(1), 0.5)
    assert math.isclose(S.polynomial_schedule(1.0, 0.0, 2.0, 10)(5), 0.25)
    wsd = S.warmup_stable_decay(1.0, 0.1, num_warmup_steps=2, num_stable_steps=2, num_decay_steps=4)
    assert [wsd(i) for i in (0, 1, 2, 3)] == [0.0, 0.5, 1.0, 1.0] and math.isclose(wsd(5), 0.1 + 0.9 * 0.5) and wsd(99) == 0.1
    ww = S.with_warmup(2.0, 4)
    assert ww(0) == 0.0 and ww(2) == 1.0 and ww(4) == 2.0
    wr = S.with_restarts(S.linear_schedule(1.0, 0.0, 5), 10, 2)
    assert wr(0) == 1.0 and math.isclose(wr(5), 1.0) and math.isclose(wr(7), 0.6) and wr(10) == 0.0
    with pytest.raises(ValueError):
        S.with_warmup(1.0, 0)
    with pytest.raises(ValueError):
        S.warmup_stable_decay(1.0, num_warmup_steps=1, num_stable_steps=0, num_decay_steps=1, decay_shape="nope")


def test_schedule_wire_round_trip():
    sch = S.with_warmup(S.cosine_schedule(1.0, 0.1, 100, transition_begin=10), 10, ramp="cosine")
    wire = S.schedule_to_wire(sch)
    assert wire["__opaque_recipe__"] == "WithWarmup" and wire["schedule"]["__opaque_recipe__"] == "CosineSchedule"
    assert S.schedule_from_wire(wire) == sch and hash(S.schedule_from_wire(wire)) == hash(sch)


def test_loss_scaler_state_machine():
    ls, st = loss_scaler(init_scale=8.0, growth_interval=2)
    assert float(ls.scale_loss(torch.tensor(2.0), st)) == 16.0
    g = ls.unscale_grads({"w": torch.full((2,), 8.0), "i": torch.tensor([1])}, st)
    assert float(g["w"][0]) == 1.0 and int(g["i"][0]) == 1
    st = ls.update(st, True)
    st = ls.update(st, True)
    assert st.scale == 16.0 and st.growth_tracker == 0
    st = ls.update(st, False)
    assert st.scale == 8.0
    off, s0 = loss_scaler(enabled=False)
    assert off.update(s0, False) == s0
    assert all_finite({"a": torch.ones(2)}) and not all_finite(clipped({"a": torch.tensor([float("nan")])}, 1.0))
    with pytest.raises(ValueError):
        loss_scaler(backoff_factor=1.5)


def test_step_perf_and_tracker():
    with step_perf("cpu", batch_size=4) as sp:
        sp.mark("clip")
        sp.mark("noise")
    assert sp.result.batch_size == 4 and set(sp.result.phases) == {"clip", "noise"}
    st = PerfState(warmup_steps=1).add(StepPerf(1.0, {}, 10)).add(StepPerf(2.0, {"clip": 0.5}, 10))
    assert st.steps == 2 and st.timed_steps == 1 and st.samples_per_second == 5.0
    tr = perf_tracker("cpu", warmup_steps=0)
    with tr.step("train", batch_size=3):
        pass
    assert tr.state("train").samples == 3


def test_trace_range_and_trace_collect_named_phases(tmp_path):
    """``trace_range`` names a phase for the PyTorch profiler (NVTX stays off without a GPU); ``trace`` writes a Chrome trace."""
    import json
    import torch
    from opaque_b200 import profiling
    profiling.enable_nvtx(True)                       # without CUDA this must stay a no-op
    out = tmp_path / "trace.json"
    with profiling.trace(str(out)) as prof:
        with profiling.trace_range("opaque::test/outer"):
            with profiling.trace_range("opaque::test/inner"):
                torch.ones(8).sum()
    profiling.enable_nvtx(False)
    names = {e.key for e in prof.key_averages()}
    assert {"opaque::test/outer", "opaque::test/inner"} <= names
    events = json.load(open(out))["traceEvents"]
    assert any(e.get("name") == "opaque::test/inner" for e in events)
