"""The Kugilix configuration, plan and cache needs (no GPU), and second readings of the plain implementation's
mechanisms: each is evaluated once more, element by element from its formula, at sizes where a slip shows."""

import math

import pytest
import torch

import kugilix_cases as cases
import plain_kugilix as plain

from ferrisinfer_b200.cache import CacheManager
from ferrisinfer_b200.config import KugilixConfig, resolve_config
from ferrisinfer_b200.errors import ConfigError, UnsupportedError
from ferrisinfer_b200.parts import CombinedNeed, FixedState, PagedKV, build_model

F64 = torch.float64


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_config_round_trip_and_tensor_names(name):
    d = cases.CASES[name]
    arch, cfg = resolve_config(d)
    assert arch.name == "Kugilix" and isinstance(cfg, KugilixConfig)
    again = KugilixConfig.from_dict(cfg.to_dict())
    assert again == cfg
    model = build_model(arch.plan(cfg))
    required = {s.name: tuple(s.shape) for s in model.tensor_specs() if s.required}
    assert required == cases.tensor_shapes(d)


def test_run_order_of_loops():
    _, a = resolve_config(cases.CASE_A)
    assert a.run_order() == [(0, False), (1, False), (2, False), (1, True), (2, False)]
    _, b = resolve_config(cases.CASE_B)
    assert b.run_order() == [(0, False), (1, False), (0, True), (1, False), (0, True), (1, False), (2, False)]
    _, c = resolve_config(cases.CASE_C)
    assert c.run_order() == [(0, False), (1, False)]
    assert [(i, again) for i, again in plain.run_order(cases.CASE_B)] == b.run_order()


def test_config_errors():
    bad = dict(cases.CASE_A, width=66)  # not divisible into four groups
    with pytest.raises(ConfigError):
        KugilixConfig.from_dict(bad)
    bad = dict(cases.CASE_A, loop={"start": 2, "stop": 1, "times": 2})
    with pytest.raises(ConfigError):
        KugilixConfig.from_dict(bad)
    layers = [dict(cases.CASE_A["layers"][0], type="convolution")]
    with pytest.raises(UnsupportedError):
        KugilixConfig.from_dict(dict(cases.CASE_A, layers=layers))
    lightning = cases.lightning_layer(2, 8, 8, 16, decay=[0.5])
    with pytest.raises(ConfigError):
        KugilixConfig.from_dict(dict(cases.CASE_A, layers=[lightning], loop={"start": 0, "stop": 0, "times": 1}))


def test_cache_needs_every_run_its_own_state_and_window_pages_return():
    arch, cfg = resolve_config(cases.CASE_A)
    model = build_model(arch.plan(cfg))
    needs = model.cache_needs()
    assert len(needs) == 5 and all(isinstance(n, CombinedNeed) for n in needs)
    assert needs[0].needs == (FixedState((3, 64), torch.float32), PagedKV(2, 32, 48, None))
    assert needs[1].needs[1] == FixedState((2, 32, 32), torch.float32)
    _, cfg_b = resolve_config(cases.CASE_B)
    needs_b = build_model(arch.plan(cfg_b)).cache_needs()
    assert PagedKV(1, 40, 21, 24) in needs_b[1].needs  # value heads of their own size
    cm = CacheManager(needs, page_size=16, num_pages=6, max_requests=2)
    assert len(cm.groups) == 1 and sorted(cm.groups[0].members) == [0, 2, 4]  # the three attention runs share page ids
    cm.admit("r")
    cm.extend("r", 80)
    cm.commit("r", 80)
    # a query at position 80 reads keys from 33 on: blocks 0 and 1 have gone back
    assert cm.block_table("r", 0)[:2] == [-1, -1] and cm.groups[0].pool.num_free == 3
    cm.check_invariants()
    cm.release("r")
    assert cm.groups[0].pool.num_free == 6 and cm.num_free_slots == 2


# ------------------------------------------------------------------------------- second readings of the plain functions
def test_plain_sinusoid_and_embedding():
    pe = plain.sinusoid([0, 3, 250], 6)
    assert torch.allclose(pe[0], torch.tensor([0.0, 1.0, 0.0, 1.0, 0.0, 1.0], dtype=F64))
    for i in range(3):
        a = 250 * 10000.0 ** (-2.0 * i / 6)
        assert abs(pe[2, 2 * i] - math.sin(a)) < 1e-12 and abs(pe[2, 2 * i + 1] - math.cos(a)) < 1e-12
    table = torch.arange(12, dtype=F64).reshape(3, 4)
    x = plain.embed(table, [2, 0], 1.5, start=7)
    assert abs(x[1, 1] - (table[0, 1] * 1.5 + math.cos(8.0))) < 1e-12


def test_plain_grouped_norm():
    x = torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=F64)
    w = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=F64)
    y = plain.grouped_rms_norm(x, w, 2, 0.0)
    r0, r1 = math.sqrt((9 + 16) / 2), math.sqrt(4 / 2)
    assert torch.allclose(y, torch.tensor([[3 / r0, 8 / r0, 0.0, 8 / r1]], dtype=F64))
    one = plain.grouped_rms_norm(x, w, 1, 0.5)
    assert abs(one[0, 0] - 3 / math.sqrt(29 / 4 + 0.5)) < 1e-12


def test_plain_convolution_is_causal_and_adds_to_its_input():
    y = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=F64)
    c = torch.tensor([[0.5, 0.25, 2.0]], dtype=F64)  # taps: t-2, t-1, t
    u = plain.input_convolution(y, c)
    assert u[:, 0].tolist() == [1 + 2 * 1, 10 + 0.25 * 1 + 2 * 10, 100 + 0.5 * 1 + 0.25 * 10 + 2 * 100,
                                1000 + 0.5 * 10 + 0.25 * 100 + 2 * 1000]


def test_plain_lightning_equals_the_unrolled_sum():
    torch.manual_seed(0)
    mixer = {"heads": 2, "dim": 3, "vdim": 2, "decay": [0.9, 0.5]}
    w = {"m.q": torch.randn(6, 4, dtype=F64), "m.k": torch.randn(6, 4, dtype=F64), "m.v": torch.randn(4, 4, dtype=F64)}
    u = torch.randn(5, 4, dtype=F64)
    o = plain.lightning(u, w, "m", mixer)
    q = plain.silu(u @ w["m.q"].T).reshape(5, 2, 3)
    k = plain.silu(u @ w["m.k"].T).reshape(5, 2, 3)
    v = plain.silu(u @ w["m.v"].T).reshape(5, 2, 2)
    for t in range(5):
        for h in range(2):
            want = sum(mixer["decay"][h] ** (t - s) * float(q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert torch.allclose(o[t, 2 * h:2 * h + 2], want)


def test_plain_attention_window_slopes_and_temperature():
    torch.manual_seed(1)
    mixer = {"heads": 2, "kv_heads": 1, "dim": 2, "vdim": 3, "scale": 0.7, "mask": {"size": 3},
             "q_temp": {"coef": 0.5, "every": 2}}
    w = {"m.q": torch.randn(4, 4, dtype=F64), "m.k": torch.randn(2, 4, dtype=F64), "m.v": torch.randn(3, 4, dtype=F64),
         "m.o": torch.eye(6, dtype=F64)}
    u = torch.randn(6, 4, dtype=F64)
    out = plain.attention_mixer(u, w, "m", mixer, 1e-6)
    t, h = 5, 1
    unit = lambda x: x / math.sqrt(float((x * x).mean()) + 1e-6)
    q = unit((u[t] @ w["m.q"].T)[2:4]) * (1 + 0.5 * math.log((t + 1) // 2 + 1))
    scores, values = [], []
    for j in (3, 4, 5):  # the window of three
        k = unit(u[j] @ w["m.k"].T)
        scores.append(float(q @ k) * 0.7 - 2.0 ** (-8 * 2 / 2) * (t - j))
        values.append(u[j] @ w["m.v"].T)
    p = torch.softmax(torch.tensor(scores, dtype=F64), 0)
    assert torch.allclose(out[t, 3:6], sum(pi * vi for pi, vi in zip(p, values)))


def test_plain_xielu():
    z = torch.tensor([-2.0, 0.0, 1.5], dtype=F64)
    y = plain.xielu(z, 0.3, -0.2)
    sp, sq = math.log(1 + math.exp(0.3)), math.log(1 + math.exp(-0.2))
    assert abs(y[0] - ((0.5 + sq) * (math.exp(-2) - 1 + 2) - 1)) < 1e-12
    assert y[1] == 0 and abs(y[2] - (sp * 2.25 + 0.75)) < 1e-12


def test_plain_forward_does_not_look_ahead():
    cfg = cases.CASE_B
    w = cases.make_weights(cfg, 3)
    ids = cases.random_ids(cfg["vocab"], 30, 1)
    full = plain.forward(cfg, w, ids)
    part = plain.forward(cfg, w, ids[:17])
    assert torch.allclose(full[:17], part, atol=1e-9)
