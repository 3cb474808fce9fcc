"""The Nusudra decoder without a GPU: its configuration (round trip, errors), the plan (kinds of parts, tensor names
and shapes, cache needs), and a second reading of the plain implementation's mechanisms, element by element with
``math`` alone, at sizes where a slip in the vectorised code shows."""

import math

import pytest
import torch

import nusudra_cases as cases
import plain_nusudra as plain

F64 = torch.float64


def build(cfg):
    from ferrisinfer_b200.config import resolve_config
    from ferrisinfer_b200.parts import build_model

    arch, c = resolve_config(cfg)
    return c, arch.plan(c), build_model(arch.plan(c))


@pytest.mark.parametrize("case", sorted(cases.CASES))
def test_configuration_round_trip_and_tensor_names(case):
    cfg = cases.CASES[case]
    c, plan, model = build(cfg)
    assert c.to_dict() == cfg
    assert {s.name: tuple(s.shape) for s in model.tensor_specs()} == cases.tensor_shapes(cfg)
    assert plan.residual_streams == (cfg.get("streams") or 1)
    assert [step.layer for step in plan.run_order] == list(range(len(cfg["layers"])))


def test_configuration_errors():
    from ferrisinfer_b200.config.nusudra import NusudraConfig
    from ferrisinfer_b200.errors import ConfigError, UnsupportedError
    import copy

    def broken(change):
        d = copy.deepcopy(cases.CASE_A)
        change(d)
        return d

    with pytest.raises(UnsupportedError):
        NusudraConfig.from_dict(broken(lambda d: d["layers"][0].update(type="lightning")))
    with pytest.raises(ConfigError):
        NusudraConfig.from_dict(broken(lambda d: d["layers"][0]["mixer"].update(kv_heads=3)))
    with pytest.raises(ConfigError):
        NusudraConfig.from_dict(broken(lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7)))
    with pytest.raises(ConfigError):
        NusudraConfig.from_dict(broken(lambda d: d["layers"][2]["mixer"]["right"].update(norm_groups=5)))
    with pytest.raises(ConfigError):
        NusudraConfig.from_dict(broken(lambda d: d.update(streams=0)))
    with pytest.raises(ConfigError):
        NusudraConfig.from_dict(broken(lambda d: d.pop("width")))
    with pytest.raises(UnsupportedError):
        NusudraConfig.from_dict(broken(lambda d: d["layers"][0]["mlp"].update(kind="experts")))


def test_cache_needs_of_the_three_mixers():
    from ferrisinfer_b200.parts.base import FixedState, PagedKV, leaf_needs

    _, _, model = build(cases.CASE_A)
    delta, latent, parallel = (leaf_needs(n) for n in model.cache_needs())
    W = cases.CASE_A["width"]
    assert delta == [FixedState((W,)), FixedState((3, 2 * 64 + 64)), FixedState((4, 16, 32))]
    assert latent == [FixedState((W,)), PagedKV(1, 48 + 16, None, 0)]  # one shared row a token, no value rows
    assert parallel == [FixedState((W,)), PagedKV(2, 32, None, None), FixedState((3, 64 + 2 * 32)), FixedState((4, 16, 16))]
    _, _, model = build(cases.CASE_C)  # one tap: the convolution keeps nothing
    assert leaf_needs(model.cache_needs()[2]) == [FixedState((72,)), FixedState((2, 64, 64))]
    assert model.graph_safe


def test_cache_manager_serves_the_needs_and_gives_slots_back():
    from ferrisinfer_b200.cache import CacheManager

    _, _, model = build(cases.CASE_A)
    cache = CacheManager(model.cache_needs(), page_size=16, num_pages=6, max_requests=2)
    assert len(cache.groups) == 2  # the latent rows and the attention's keys and values page apart
    a = cache.admit("a")
    cache.extend("a", 40)
    cache.commit("a", 40)
    b = cache.admit("b")
    assert {a.slot, b.slot} == {0, 1} and cache.num_free_slots == 0
    cache.release("a")
    assert cache.admit("c").slot == a.slot  # the slot comes back
    cache.check_invariants()


# ------------------------------------------------------------------------------- a second reading, element by element
def test_token_shift_element_by_element():
    h, shift = torch.randn(5, 3, dtype=F64), torch.rand(3, dtype=F64)
    got, last = plain.token_shift(h, shift)
    for t in range(5):
        for c in range(3):
            prev = 0.0 if t == 0 else float(h[t - 1, c])
            assert abs(float(got[t, c]) - (float(h[t, c]) + (prev - float(h[t, c])) * float(shift[c]))) < 1e-12
    again, _ = plain.token_shift(h[3:], shift, before=h[2])
    assert torch.allclose(again, got[3:]) and torch.equal(last, h[4])


def test_streams_element_by_element():
    S, T, W = 3, 2, 4
    xs, mix, out, inn, y = (torch.randn(*s, dtype=F64) for s in ((S, T, W), (S, S), (S,), (S,), (T, W)))
    u, new = plain.streams_read(xs, inn), plain.streams_write(xs, mix, out, y)
    for t in range(T):
        for c in range(W):
            assert abs(float(u[t, c]) - sum(float(inn[s]) * float(xs[s, t, c]) for s in range(S))) < 1e-12
            for r in range(S):
                want = sum(float(mix[s, r]) * float(xs[s, t, c]) for s in range(S)) + float(out[r]) * float(y[t, c])
                assert abs(float(new[r, t, c]) - want) < 1e-12


def test_convolution_and_rotation_element_by_element():
    x, w, b = torch.randn(6, 2, dtype=F64), torch.randn(2, 3, dtype=F64), torch.randn(2, dtype=F64)
    got, kept = plain.causal_conv(x, w, b)
    for t in range(6):
        for c in range(2):
            want = float(b[c]) + sum(float(w[c, j]) * (float(x[t - 2 + j, c]) if t - 2 + j >= 0 else 0.0) for j in range(3))
            assert abs(float(got[t, c]) - want) < 1e-12  # the last column is the current token's
    assert torch.equal(kept, x[4:])
    v = torch.randn(3, 1, 6, dtype=F64)
    rot = plain.rotate_half(v, [0, 5, 9], 100.0, 4)
    for t, p in enumerate([0, 5, 9]):
        for i in range(2):
            a = p * 100.0 ** (-2.0 * i / 4)
            u0, u1 = float(v[t, 0, i]), float(v[t, 0, i + 2])
            assert abs(float(rot[t, 0, i]) - (u0 * math.cos(a) - u1 * math.sin(a))) < 1e-12
            assert abs(float(rot[t, 0, i + 2]) - (u1 * math.cos(a) + u0 * math.sin(a))) < 1e-12
        assert torch.equal(rot[t, 0, 4:], v[t, 0, 4:])  # the rest passes unchanged


def test_recurrences_element_by_element():
    T, n, dv = 4, 3, 2
    q, k = torch.randn(T, 1, n, dtype=F64), torch.randn(T, 1, n, dtype=F64)
    v, g, beta = torch.randn(T, 1, dv, dtype=F64), torch.rand(T, 1, dtype=F64), torch.rand(T, 1, dtype=F64)
    o1, _ = plain.delta_rule_scan(q, k, v, g, beta, torch.zeros(1, n, dv, dtype=F64))
    o2, _ = plain.decayed_scan(q, k, v, g, torch.zeros(1, n, dv, dtype=F64))
    S1 = [[0.0] * dv for _ in range(n)]
    S2 = [[0.0] * dv for _ in range(n)]
    for t in range(T):
        gt, bt = float(g[t, 0]), float(beta[t, 0])
        kt, qt, vt = [float(x) for x in k[t, 0]], [float(x) for x in q[t, 0]], [float(x) for x in v[t, 0]]
        S1 = [[gt * S1[i][j] for j in range(dv)] for i in range(n)]
        u = [bt * (vt[j] - sum(S1[i][j] * kt[i] for i in range(n))) for j in range(dv)]
        S1 = [[S1[i][j] + kt[i] * u[j] for j in range(dv)] for i in range(n)]
        S2 = [[gt * S2[i][j] + kt[i] * vt[j] for j in range(dv)] for i in range(n)]
        for j in range(dv):
            assert abs(float(o1[t, 0, j]) - sum(S1[i][j] * qt[i] for i in range(n))) < 1e-12
            assert abs(float(o2[t, 0, j]) - sum(S2[i][j] * qt[i] for i in range(n))) < 1e-12


def test_sink_attention_element_by_element():
    torch.manual_seed(1)
    T, W = 4, 3
    m = {"heads": 2, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 0.7}
    w = {"a.q": torch.randn(4, W, dtype=F64), "a.k": torch.randn(2, W, dtype=F64), "a.v": torch.randn(2, W, dtype=F64),
         "a.q.b": torch.randn(4, dtype=F64), "a.k.b": torch.randn(2, dtype=F64), "a.v.b": torch.randn(2, dtype=F64),
         "a.r1": torch.rand(2, dtype=F64), "a.r2": torch.rand(2, dtype=F64), "a.sink": torch.randn(2, dtype=F64),
         "a.o": torch.eye(4, dtype=F64)}
    h = torch.randn(T, W, dtype=F64)
    got = plain.sink_attention(h, w, "a", m)[0]
    q, k, v = h @ w["a.q"].T + w["a.q.b"], h @ w["a.k"].T + w["a.k.b"], h @ w["a.v"].T + w["a.v.b"]
    for i in range(T):
        for head in range(2):
            s = [0.7 * float(q[i, 2 * head:2 * head + 2] @ k[j]) - float(w["a.r1"][head]) * math.log(1 + float(w["a.r2"][head]) * (i - j))
                 for j in range(i + 1)]
            z = sum(math.exp(x) for x in s) + math.exp(float(w["a.sink"][head]))  # the sink: once, unscaled, no value
            for c in range(2):
                want = sum(math.exp(s[j]) / z * float(v[j, c]) for j in range(i + 1))
                assert abs(float(got[i, 2 * head + c]) - want) < 1e-12


def test_prompt_cut_anywhere_gives_the_same_logits_plainly():
    for name, cfg in cases.CASES.items():
        w = cases.make_weights(cfg, 1)
        ids = cases.random_ids(cfg["vocab"], 30, 2)
        full, _ = plain.forward(cfg, w, ids)
        a, st = plain.forward(cfg, w, ids[:11])
        b, st = plain.forward(cfg, w, ids[11:12], st)
        c, _ = plain.forward(cfg, w, ids[12:], st)
        assert torch.allclose(torch.cat([a, b, c]), full, atol=1e-10), name
