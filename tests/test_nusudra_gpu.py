"""The Nusudra decoder on the GPU against the plain implementation (``plain_nusudra``, float64): each kernel of its
mechanisms alone, then whole models of several small configurations driven through the step function the ways a
server drives it (whole prompts, token by token, portions down to two tokens, mixed batches over pages and state
slots that come back), and greedy generation through the engine."""

import functools
import json
import math
import os
from types import SimpleNamespace

import pytest
import torch

import helpers
import nusudra_cases as cases
import plain_nusudra as plain

pytestmark = pytest.mark.gpu
F32, F64, BF16 = torch.float32, torch.float64, torch.bfloat16
DTYPES = {"float32": F32, "bfloat16": BF16}


def _ops():
    from ferrisinfer_b200.kernels import ops
    return ops


def make_runner(cfg, weights, dtype, device, num_pages=24, max_requests=4, graphs=True, page_size=16):
    from ferrisinfer_b200.config import resolve_config
    from ferrisinfer_b200.engine.runner import ModelRunner
    from ferrisinfer_b200.parts import build_model
    from ferrisinfer_b200.weights.loader import bind_tensors

    arch, c = resolve_config(cfg)
    model = build_model(arch.plan(c))
    bind_tensors(model, weights, DTYPES[dtype], device)
    return ModelRunner(model, DTYPES[dtype], device, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                       cuda_graphs=graphs)


@functools.lru_cache(maxsize=None)
def weights_of(case: str):
    return cases.make_weights(cases.CASES[case], seed=sum(map(ord, case)))


@functools.lru_cache(maxsize=None)
def wanted(case: str, n: int, seed: int):
    """(ids, float64 logits of every position) of a random sequence."""
    cfg = cases.CASES[case]
    ids = cases.random_ids(cfg["vocab"], n, seed)
    return ids, plain.forward(cfg, weights_of(case), ids)[0]


def check_replay(got: dict, requests: dict, case: str, dtype: str, what: str):
    """Every (request, position) of ``requests`` (id -> (n, seed)) is there and within tolerance.  In bfloat16 a few
    positions amplify rounding several times over the typical error (the same ones whatever the schedule; the 32-bit
    run is exact there too): at most one position in fifty may exceed the tolerance, none four times it."""
    worst, where, over, count = 0.0, None, 0, 0
    tol = cases.TOLERANCE[dtype]
    for rid, (n, seed) in requests.items():
        _, want = wanted(case, n, seed)
        rows = torch.stack([got[(rid, p)] for p in range(n)])
        assert torch.isfinite(rows).all(), f"{what}: request {rid} has logits that are not finite"
        err = cases.row_errors(rows, want)
        over, count = over + int((err > tol).sum()), count + n
        if float(err.max()) > worst:
            worst, where = float(err.max()), (rid, int(err.argmax()))
    if dtype == "float32":
        assert worst <= tol, f"{what} ({case}, {dtype}): error {worst:.3g} at {where}"
    else:
        assert worst <= 4 * tol and over <= max(1, count // 50), \
            f"{what} ({case}, {dtype}): error {worst:.3g} at {where}, {over} of {count} positions over {tol}"


def fake_ctx(device, q_lens, start_pos, slots, workspace=None):
    """The device arrays of a step, as the step function lays them out."""
    S = len(q_lens)
    q_start = [0]
    for n in q_lens:
        q_start.append(q_start[-1] + n)
    token_seq = [s for s in range(S) for _ in range(q_lens[s])]
    positions = [start_pos[s] + i for s in range(S) for i in range(q_lens[s])]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return SimpleNamespace(num_tokens=q_start[-1], num_seqs=S, max_q_len=max(q_lens), workspace=workspace,
                           max_kv_len=max(a + b for a, b in zip(q_lens, start_pos)),
                           token_seq=i32(token_seq), positions=i32(positions),
                           seq_q_start=i32(q_start), seq_start_pos=i32(start_pos), seq_state_slot=i32(slots))


def tol_of(dtype, loose=1.0):
    return dict(atol=2e-5 * loose, rtol=1e-4 * loose) if dtype == F32 else dict(atol=3e-2 * loose, rtol=3e-2 * loose)


# =========================================================================================== each mechanism alone
@pytest.mark.parametrize("streams,width", [(1, 40), (2, 64), (4, 96), (5, 2048), (8, 24)])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_residual_streams_write_and_read(device, streams, width, dtype):
    """The write of one sublayer and the normed read of the next in one pass, each half alone, expand and sum."""
    ops = _ops()
    torch.manual_seed(streams * width)
    T, S, W = 7, streams, width
    row = torch.randn(T, W)
    xs = torch.empty(T, S * W, device=device)
    ops.streams_expand(row.to(device), xs, S)
    assert torch.equal(xs.cpu().view(T, S, W), row[:, None, :].expand(T, S, W))
    old = torch.randn(S, T, W, dtype=F64)
    y, mix, out_w, in_w, norm_w = torch.randn(T, W), torch.eye(S) + 0.3 * torch.randn(S, S), torch.randn(S), torch.randn(S), 1 + 0.1 * torch.randn(W)
    new = plain.streams_write(old, mix.double(), out_w.double(), y.double())
    want = plain.rms_norm(plain.streams_read(new, in_w.double()), norm_w.double(), 1e-5)
    dev = lambda t: t.to(device)
    layout = lambda t: t.permute(1, 0, 2).reshape(T, S * W).float().contiguous()
    for halves in ("both", "apart"):
        xs = dev(layout(old))
        out = torch.empty(T, W, dtype=dtype, device=device)
        if halves == "both":
            ops.streams_step(xs, S, write=(dev(y), dev(mix), dev(out_w)), read=(dev(in_w), dev(norm_w), 1e-5, out))
        else:
            ops.streams_step(xs, S, write=(dev(y), dev(mix), dev(out_w)))
            ops.streams_step(xs, S, read=(dev(in_w), dev(norm_w), 1e-5, out))
        assert torch.allclose(xs.cpu().double(), layout(new).double(), atol=1e-5, rtol=1e-5)
        assert torch.allclose(out.cpu().double(), want, **tol_of(dtype))
    total = torch.empty(T, W, device=device)
    ops.streams_sum(xs, total, S)
    assert torch.allclose(total.cpu().double(), new.sum(0), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_token_shift_carries_the_last_row_across_steps(device, dtype):
    """Three requests over slots out of order, cut into unequal steps (portions, single tokens, a request that sits a
    step out): every row is shifted towards the request's row before, across steps from the state."""
    ops = _ops()
    torch.manual_seed(3)
    W, lens = 72, [23, 9, 14]
    shift = torch.rand(W)
    xs = [torch.randn(n, W).to(dtype) for n in lens]
    want = [plain.token_shift(x.double(), shift.double())[0] for x in xs]
    state = torch.randn(5, W, device=device)  # slots hold what their last request left
    slots = [3, 0, 4]
    state[slots] = 0.0  # ... until a request is admitted
    schedule = [[5, 1, 2], [1, 0, 1], [10, 8, 1], [1, 0, 10], [6, 0, 0]]
    done = [0, 0, 0]
    for step in schedule:
        live = [i for i in range(3) if step[i] > 0]
        ctx = fake_ctx(device, [step[i] for i in live], [done[i] for i in live], [slots[i] for i in live])
        rows = torch.cat([xs[i][done[i]:done[i] + step[i]] for i in live]).to(device)
        out = torch.empty_like(rows)
        ops.token_shift(rows, out, shift.to(device), state, ctx)
        at = 0
        for i in live:
            assert torch.allclose(out[at:at + step[i]].cpu().double(), want[i][done[i]:done[i] + step[i]], **tol_of(dtype)), (step, i)
            at += step[i]
            done[i] += step[i]
    assert done == lens
    for i in range(3):
        assert torch.equal(state[slots[i]].cpu(), xs[i][-1].float())


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_convolution_with_bias_and_silu_on_a_slice_of_the_rows(device, taps, dtype):
    ops = _ops()
    torch.manual_seed(taps)
    C, n, before = 40, 19, 8
    wide = torch.randn(n, before + C + 5).to(dtype)  # the channels are columns before .. before + C of wider rows
    w, b = 0.5 * torch.randn(C, taps), 0.3 * torch.randn(C)
    x = wide[:, before:before + C].double()
    want = plain.silu(plain.causal_conv(x, w.double(), b.double())[0])
    state = torch.zeros(2, max(taps - 1, 1), C, device=device)
    wide_d = wide.to(device)
    pos = 0
    for cut in (6, 1, 1, 9, 2):
        ctx = fake_ctx(device, [cut], [pos], [1])
        out = torch.empty(cut, C, dtype=dtype, device=device)
        ops.short_conv(wide_d[pos:pos + cut, before:before + C], out, w.to(device), state if taps > 1 else None, ctx,
                       bias=b.to(device), residual=False, silu=True)
        assert torch.allclose(out.cpu().double(), want[pos:pos + cut], **tol_of(dtype)), (taps, pos)
        pos += cut


def recurrence_inputs(T, heads, qk_heads, dim, vdim, dtype, seed, long_memory=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, qk_heads * dim, generator=g).to(dtype)
    k = (torch.randn(T, qk_heads * dim, generator=g) / math.sqrt(dim)).to(dtype)  # about unit length: the delta rule is stable
    v = torch.randn(T, heads * vdim, generator=g).to(dtype)
    decay = torch.rand(T, heads, generator=g) * (0.02 if long_memory else 0.5) + (0.98 if long_memory else 0.5)
    beta = torch.rand(T, heads, generator=g)
    return q, k, v, decay, beta


@pytest.mark.parametrize("heads,qk_heads,dim,vdim", [(4, 2, 32, 16), (3, 1, 24, 40), (2, 2, 64, 64), (1, 1, 128, 130), (2, 1, 200, 8)])
@pytest.mark.parametrize("delta", [True, False])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_recurrence_whole_in_portions_and_token_by_token(device, heads, qk_heads, dim, vdim, delta, dtype):
    """One request's tokens in one go, in portions of unequal size and one by one, from the state its slot holds:
    unit-norm factors, the skip weight, grouped q/k heads, head sizes that fill no lane evenly."""
    ops = _ops()
    T = 45
    q, k, v, decay, beta = recurrence_inputs(T, heads, qk_heads, dim, vdim, dtype, seed=dim + vdim)
    qs, ks = torch.rand(T, qk_heads) + 0.5, 0.7 * torch.rand(T, qk_heads) + 0.5
    skip = torch.randn(heads)
    of = torch.arange(heads) // (heads // qk_heads)
    qh = (q.double().view(T, qk_heads, dim) * qs.double()[..., None])[:, of]
    kh = (k.double().view(T, qk_heads, dim) * ks.double()[..., None])[:, of]
    vh = v.double().view(T, heads, vdim)
    zero = torch.zeros(heads, dim, vdim, dtype=F64)
    if delta:
        want, last = plain.delta_rule_scan(qh, kh, vh, decay.double(), beta.double(), zero)
    else:
        want, last = plain.decayed_scan(qh, kh, beta.double()[..., None] * vh, decay.double(), zero)
        want = want + skip.double()[None, :, None] * vh
    want = want.reshape(T, heads * vdim)
    dev = lambda t: t.to(device)
    for cuts in ([T], [7, 1, 20, 2, 15], [1] * T):
        state = torch.randn(3, heads, vdim, dim, device=device)
        state[2] = 0.0
        pos = 0
        for n in cuts:
            ctx = fake_ctx(device, [n], [pos], [2])
            sl = slice(pos, pos + n)
            out = torch.empty(n, heads * vdim, device=device)
            ops.gated_recurrence(dev(q[sl]), dev(k[sl]), dev(v[sl]), dev(decay[sl]), dev(beta[sl]), out, state, ctx, heads,
                                 qk_heads, dim, vdim, delta_rule=delta, qscale=dev(qs[sl]), kscale=dev(ks[sl]),
                                 skip=None if delta else dev(skip))
            assert torch.allclose(out.cpu().double(), want[sl], atol=2e-4, rtol=2e-4), (cuts[:3], pos)
            pos += n
        assert torch.allclose(state[2].cpu().double().transpose(1, 2), last, atol=2e-4, rtol=2e-4)  # S lies transposed


def test_recurrence_of_several_requests_keeps_their_states_apart(device):
    """A portion, two single tokens and a longer portion in one step, over slots out of order; a later step continues
    two of them; a write that is switched off leaves the state as it was."""
    ops = _ops()
    heads, qk_heads, dim, vdim = 4, 2, 32, 48
    lens = [30, 12, 9, 50]
    data = [recurrence_inputs(n, heads, qk_heads, dim, vdim, F32, seed=n) for n in lens]
    of = torch.arange(heads) // (heads // qk_heads)
    want = []
    for (q, k, v, decay, beta), n in zip(data, lens):
        o, _ = plain.delta_rule_scan(q.double().view(n, qk_heads, dim)[:, of], k.double().view(n, qk_heads, dim)[:, of],
                                     v.double().view(n, heads, vdim), decay.double(), beta.double(),
                                     torch.zeros(heads, dim, vdim, dtype=F64))
        want.append(o.reshape(n, heads * vdim))
    state = torch.zeros(6, heads, vdim, dim, device=device)
    slots = [4, 1, 5, 0]
    done = [0, 0, 0, 0]
    for step in ([17, 1, 1, 33], [13, 1, 0, 17], [0, 10, 8, 0]):
        live = [i for i in range(4) if step[i]]
        ctx = fake_ctx(device, [step[i] for i in live], [done[i] for i in live], [slots[i] for i in live])
        cat = lambda j: torch.cat([data[i][j][done[i]:done[i] + step[i]] for i in live]).to(device)
        out = torch.empty(sum(step), heads * vdim, device=device)
        before = state.clone()
        ops.gated_recurrence(cat(0), cat(1), cat(2), cat(3), cat(4), out, state, ctx, heads, qk_heads, dim, vdim,
                             delta_rule=True, write_state=False)
        assert torch.equal(state, before)
        ops.gated_recurrence(cat(0), cat(1), cat(2), cat(3), cat(4), out, state, ctx, heads, qk_heads, dim, vdim,
                             delta_rule=True)
        at = 0
        for i in live:
            assert torch.allclose(out[at:at + step[i]].cpu().double(), want[i][done[i]:done[i] + step[i]], atol=1e-4, rtol=1e-4)
            at += step[i]
            done[i] += step[i]
    assert done == lens


def test_recurrence_keeps_a_write_from_hundreds_of_tokens_ago(device):
    """Decays near one: what token 3 wrote is read out 700 tokens later, the rest of the keys being orthogonal to the
    query; portions of 64 and single tokens in between."""
    ops = _ops()
    heads, dim, vdim, T = 1, 64, 32, 704
    k = torch.zeros(T, dim)
    k[:, 1:] = torch.randn(T, dim - 1) / math.sqrt(dim)
    k[3] = 0.0
    k[3, 0] = 1.0  # the only key along the first axis
    v = torch.randn(T, vdim)
    q = torch.zeros(T, dim)
    q[:, 0] = 1.0  # every query asks along that axis
    decay = torch.full((T, heads), 0.999)
    beta = torch.ones(T, heads)
    want, _ = plain.decayed_scan(q.double().view(T, 1, dim), k.double().view(T, 1, dim), v.double().view(T, 1, vdim),
                                 decay.double(), torch.zeros(1, dim, vdim, dtype=F64))
    assert torch.allclose(want[T - 1, 0], 0.999 ** (T - 4) * v[3].double(), atol=1e-9)
    state = torch.zeros(1, heads, vdim, dim, device=device)
    pos, outs = 0, []
    dev = lambda t: t.to(device)
    for n in [64] * 10 + [1] * 64:
        ctx = fake_ctx(device, [n], [pos], [0])
        sl = slice(pos, pos + n)
        out = torch.empty(n, vdim, device=device)
        ops.gated_recurrence(dev(q[sl]), dev(k[sl]), dev(v[sl]), dev(decay[sl]), dev(beta[sl]), out, state, ctx, heads, 1, dim,
                             vdim, delta_rule=False)
        outs.append(out.cpu())
        pos += n
    got = torch.cat(outs)
    assert torch.allclose(got.double(), want.reshape(T, vdim), atol=1e-4, rtol=1e-4)
    assert float((got[T - 1].double() - 0.999 ** (T - 4) * v[3].double()).abs().max()) < 1e-4


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_recurrence_gates_and_unit_norms(device, dtype):
    ops = _ops()
    torch.manual_seed(11)
    T, heads, g, dim = 9, 6, 3, 24
    proj = torch.randn(T, 2 * heads + 5).to(dtype)
    rows = (3 * torch.randn(T, 2 * g * dim + 7)).to(dtype)
    A_log, dt_bias = torch.randn(heads), torch.randn(heads)
    dt = plain.softplus(proj[:, 3:3 + heads].double() + dt_bias.double())
    want_decay = torch.exp(-torch.exp(A_log.double()) * dt)
    want_beta = torch.sigmoid(proj[:, 3 + heads:3 + 2 * heads].double())
    qd, kd = rows[:, 2:2 + g * dim].double().view(T, g, dim), rows[:, 5 + g * dim:5 + 2 * g * dim].double().view(T, g, dim)
    decay, beta = torch.empty(T, heads, device=device), torch.empty(T, heads, device=device)
    qs, ks = torch.empty(T, g, device=device), torch.empty(T, g, device=device)
    dev = lambda t: t.to(device)
    ops.recurrence_gates(dev(proj), 3, 3 + heads, dev(A_log), dev(dt_bias), decay, beta, heads,
                         unit_norm=(dev(rows), 2, 5 + g * dim, g, dim, 1e-6, dim ** -0.5, qs, ks))
    assert torch.allclose(decay.cpu().double(), want_decay, atol=1e-6, rtol=1e-5)
    assert torch.allclose(beta.cpu().double(), want_beta, atol=1e-6, rtol=1e-5)
    assert torch.allclose(qs.cpu().double(), dim ** -0.5 / torch.sqrt((qd * qd).sum(-1) + 1e-6), rtol=1e-5)
    assert torch.allclose(ks.cpu().double(), 1 / torch.sqrt((kd * kd).sum(-1) + 1e-6), rtol=1e-5)
    ops.recurrence_gates(dev(proj), 3, None, dev(A_log), dev(dt_bias), decay, beta, heads)  # the step size itself
    assert torch.allclose(beta.cpu().double(), dt, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("n,group,wlen", [(96, 24, 24), (128, 64, 128), (40, 40, 40), (2048, 512, 2048)])
@pytest.mark.parametrize("gate_first", [False, True])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_gated_norm_in_groups(device, n, group, wlen, gate_first, dtype):
    ops = _ops()
    torch.manual_seed(n + group)
    T = 5
    o, gate, w = torch.randn(T, n), torch.randn(T, n + 3).to(dtype), 1 + 0.2 * torch.randn(wlen)
    act = plain.silu(gate[:, 3:].double())
    x = o.double() * act if gate_first else o.double()
    want = plain.rms_div(x.view(T, n // group, group), 1e-5).reshape(T, n) * w.double().repeat(n // wlen)
    if not gate_first:
        want = want * act
    out = torch.empty(T, n, dtype=dtype, device=device)
    ops.gated_group_norm(o.to(device), gate.to(device)[:, 3:], w.to(device), 1e-5, out, group=group, gate_kind="silu",
                         gate_first=gate_first)
    assert torch.allclose(out.cpu().double(), want, **tol_of(dtype))


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_results_of_mixers_side_by_side_are_normed_and_averaged(device, dtype):
    ops = _ops()
    torch.manual_seed(5)
    T, W = 6, 200
    h, a, b = torch.randn(T, W), 3 * torch.randn(T, W), 0.1 * torch.randn(T, W)
    wa, wb = 1 + 0.1 * torch.randn(W), 1 + 0.1 * torch.randn(W)
    want = h.double() + 0.5 * (plain.rms_norm(a.double(), wa.double(), 1e-6) + plain.rms_norm(b.double(), wb.double(), 1e-6))
    hd = h.to(device)
    ops.branch_norm_sum(hd, [(a.to(device), wa.to(device)), (b.to(device), wb.to(device))], 0.5, 1e-6)
    assert torch.allclose(hd.cpu().double(), want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("T,H,K,N", [(1, 3, 24, 32), (9, 4, 16, 48), (17, 2, 96, 130)])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_product_per_head_with_a_gate(device, T, H, K, N, dtype):
    ops = _ops()
    torch.manual_seed(T + K)
    x = torch.randn(T, H * (K + 5) + 2).to(dtype)  # a head's inputs lie K + 5 apart
    w = (torch.randn(H, K, N) / math.sqrt(K)).to(dtype)
    gate = torch.randn(T, H).to(dtype)
    xin = torch.stack([x[:, h * (K + 5):h * (K + 5) + K] for h in range(H)], dim=1).double()
    want = torch.einsum("thk,hkn->thn", xin, w.double())
    out = torch.zeros(T, H * (N + 3), dtype=dtype, device=device)
    ops.head_gemm(x.to(device), K + 5, w.to(device), out, N + 3)
    got = out.cpu().double().view(T, H, N + 3)
    assert torch.allclose(got[..., :N], want, **tol_of(dtype, 3.0)) and float(got[..., N:].abs().max()) == 0.0
    ops.head_gemm(x.to(device), K + 5, w.to(device), out, N + 3, gate=gate.to(device))
    got = out.cpu().double().view(T, H, N + 3)
    assert torch.allclose(got[..., :N], want * torch.sigmoid(gate.double())[..., None], **tol_of(dtype, 3.0))


@pytest.mark.parametrize("T", [3, 16, 40, 130, 700])  # weight-stationary, tcgen05 short, token-major, CTA pairs
def test_up_product_with_the_squared_relu_in_its_epilogue(device, T):
    ops = _ops()
    torch.manual_seed(T)
    K, N = 256, 384
    x, w = torch.randn(T, K).to(BF16), (torch.randn(N, K) / 16).to(BF16)
    want = torch.relu(x.double() @ w.double().T) ** 2
    out = torch.empty(T, N, dtype=BF16, device=device)
    ops.gemm_activation(x.to(device), w.to(device), out, "relu2")
    assert torch.allclose(out.cpu().double(), want, atol=2e-2, rtol=2e-2)
    out32 = torch.empty(T, N, device=device)
    ops.gemm_activation(x.float().to(device), w.float().to(device), out32, "relu2")
    assert torch.allclose(out32.cpu().double(), want, atol=1e-4, rtol=1e-4)


def paged(device, dtype, T, nkv, d, dv, page_size, order, extra_pages=1):
    """Empty caches, the block table of one request whose pages lie in ``order``, and its tokens' cache slots."""
    blocks = -(-T // page_size)
    assert len(order) >= blocks
    k = torch.zeros(len(order) + extra_pages, nkv, page_size, d, dtype=dtype, device=device)
    v = torch.zeros(len(order) + extra_pages, nkv, page_size, dv, dtype=dtype, device=device) if dv else None
    table = torch.tensor([order[:blocks]], dtype=torch.int32, device=device)
    slots = torch.tensor([order[p // page_size] * page_size + p % page_size for p in range(T)], dtype=torch.int32, device=device)
    return k, v, table, slots


@pytest.mark.parametrize("form", ["single", "tiled", "shares"])
@pytest.mark.parametrize("back", [0, 1, 15, 16, 17, 63, 64, 255, 256, 599])
def test_attention_with_a_sink_and_a_distance_penalty_one_key_stands_out(device, back, form):
    """The key ``back`` positions before the last query (page borders, near and hundreds of keys away) points the query's
    way, every other key the opposite way: the output is that key's value times its weight against the sink,
    exp(s) / (exp(s) + exp(sink)) with s = q . k * scale - r1 ln(1 + r2 * back), for every head with its own numbers."""
    ops = _ops()
    from ferrisinfer_b200.engine.workspace import Workspace

    torch.manual_seed(back)
    nh, nkv, d, dv, ps, T = 4, 2, 32, 24, 16, 620
    direction = torch.randn(d)
    direction /= direction.norm()
    keys = -30.0 * direction.repeat(T, nkv, 1)
    keys[T - 1 - back] = 2.0 * direction
    values = torch.randn(T, nkv, dv)
    r1, r2, sink = torch.rand(nh) + 0.2, torch.rand(nh) + 0.1, torch.randn(nh) + 1.0
    order = torch.randperm(40).tolist()
    k, v, table, slots = paged(device, F32, T, nkv, d, dv, ps, order)
    page, off = (slots // ps).long(), (slots % ps).long()
    k[page, :, off] = keys.to(device)
    v[page, :, off] = values.to(device)
    q = torch.zeros(T, nh * d)
    q[T - 1] = (3.0 * direction).repeat(nh)
    ctx = fake_ctx(device, [1], [T - 1], [0]) if form != "tiled" else fake_ctx(device, [T], [0], [0])
    rows = q[T - 1:].to(device) if form != "tiled" else q.to(device)
    out = torch.empty(rows.shape[0], nh * dv, device=device)
    terms = ops.ScoreTerms(log_r1=r1.to(device), log_r2=r2.to(device), sink=sink.to(device))
    extra = dict(max_kv_len=T, workspace=Workspace(device)) if form == "shares" else {}
    ops.paged_attention_simt(rows, out, k, v, table, ctx.token_seq, ctx.positions, nh, nkv, d, 0, 0.5, score_slopes=terms,
                             v_head_dim=dv, max_q_len=T if form == "tiled" else 1, **extra)
    s = 3.0 * 2.0 * 0.5 - r1.double() * torch.log1p(r2.double() * back)  # the others score -45 or less
    share = torch.exp(s) / (torch.exp(s) + torch.exp(sink.double()))
    got = out[-1].cpu().double().view(nh, dv)
    want = share[:, None] * values[T - 1 - back].double()[torch.arange(nh) // (nh // nkv)]
    assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), (got[0, :4], want[0, :4])


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nh,nkv,d,dv", [(4, 2, 32, 32), (3, 1, 24, 40), (8, 2, 16, 16), (6, 6, 64, 64)])
def test_attention_with_a_sink_against_the_plain_mixer(device, nh, nkv, d, dv, dtype):
    """Random rows through the cache write and every form of the general attention (whole, a portion behind a cached
    prefix, single tokens alone and in shares) against the plain mixer, which reads the same rounded projections."""
    ops = _ops()
    from ferrisinfer_b200.engine.workspace import Workspace

    torch.manual_seed(nh * d + dv)
    T, ps = 90, 16
    m = {"heads": nh, "kv_heads": nkv, "dim": d, "vdim": dv, "scale": 2.0 / math.sqrt(d)}
    qkv = torch.randn(T, nh * d + nkv * d + nkv * dv).to(dtype)
    a, b = nh * d, nh * d + nkv * d
    wi = {"m.o": torch.eye(nh * dv, dtype=F64), "m.r1": torch.rand(nh, dtype=F64) + 0.3, "m.r2": torch.rand(nh, dtype=F64) + 0.1,
          "m.sink": torch.randn(nh, dtype=F64)}
    for part, lo, hi in (("m.q", 0, a), ("m.k", a, b), ("m.v", b, qkv.shape[1])):
        wi[part] = torch.zeros(hi - lo, qkv.shape[1], dtype=F64)
        wi[part][:, lo:hi] = torch.eye(hi - lo, dtype=F64)
        wi[part + ".b"] = torch.zeros(hi - lo, dtype=F64)
    want = plain.sink_attention(qkv.double(), wi, "m", m)[0]
    terms = ops.ScoreTerms(log_r1=wi["m.r1"].float().to(device), log_r2=wi["m.r2"].float().to(device),
                           sink=wi["m.sink"].float().to(device))
    for cuts, ws in (([T], None), ([40, 17] + [1] * 33, None), ([50] + [1] * 40, Workspace(device))):
        k, v, table, slots = paged(device, dtype, T, nkv, d, dv, ps, [4, 0, 3, 1, 5, 2])
        pos = 0
        for n in cuts:
            ctx = fake_ctx(device, [n], [pos], [0])
            rows = qkv[pos:pos + n].to(device).contiguous()
            ops.qk_prepare_cache_write(rows, ctx.positions, slots[pos:pos + n].contiguous(), k, v, nh, nkv, d, dv, None, None)
            out = torch.empty(n, nh * dv, dtype=dtype, device=device)
            extra = dict(max_kv_len=pos + n, workspace=ws) if ws is not None and n == 1 else {}
            ops.paged_attention_simt(rows, out, k, v, table, ctx.token_seq, ctx.positions, nh, nkv, d, 0, m["scale"],
                                     score_slopes=terms, v_head_dim=dv, max_q_len=n, **extra)
            assert torch.allclose(out.cpu().double(), want[pos:pos + n], **tol_of(dtype, 2.0)), (cuts[:2], pos)
            pos += n


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nh,d,r,dv,rank,dims", [(4, 16, 16, 24, 48, 16), (3, 24, 8, 40, 32, 4), (8, 8, 8, 8, 16, 8), (2, 64, 32, 64, 96, 32),
                                                 (2, 32, 32, 32, 320, 32)])  # a row of 352: beyond what the wide-load forms take
def test_attention_over_a_shared_latent_against_the_plain_mixer(device, nh, d, r, dv, rank, dims, dtype):
    """Norm of the latent, rotation of the shared key part and of the heads' query parts, the cache row, the plain
    queries through the key up-projection, attention whose keys carry the values, the value up-projection with the
    output gate: whole, a portion behind a cached prefix and single tokens (alone and in shares, 330 keys deep), over
    pages out of order, against the plain mixer reading the same rounded projections."""
    ops = _ops()
    from ferrisinfer_b200.engine.workspace import Workspace

    torch.manual_seed(nh * d + rank)
    T, ps, row = 330, 16, rank + r
    m = {"heads": nh, "dim": d, "rot_dim": r, "vdim": dv, "kv_rank": rank, "scale": 2.0 / math.sqrt(d + r),
         "rot": {"base": 300.0, "dims": dims}}
    Q = nh * (d + r)
    proj = torch.randn(T, Q + row + nh).to(dtype)
    uk, uv = (torch.randn(nh * d, rank) / math.sqrt(rank)).to(dtype), (torch.randn(nh * dv, rank) / math.sqrt(rank)).to(dtype)
    norm_w = 1 + 0.1 * torch.randn(rank)
    wi = {"m.uk": uk.double(), "m.uv": uv.double(), "m.dkv.norm": norm_w.double(), "m.o": torch.eye(nh * dv, dtype=F64)}
    for part, lo, hi in (("m.q", 0, Q), ("m.dkv", Q, Q + row), ("m.g", Q + row, Q + row + nh)):
        wi[part] = torch.zeros(hi - lo, proj.shape[1], dtype=F64)
        wi[part][:, lo:hi] = torch.eye(hi - lo, dtype=F64)
    want = plain.latent_attention(proj.double(), wi, "m", m, 1e-5, list(range(T)))[0]
    freq = torch.tensor([300.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64).float().to(device)
    uk_d = uk.view(nh, d, rank).contiguous().to(device)
    uv_d = uv.view(nh, dv, rank).transpose(1, 2).contiguous().to(device)
    for cuts, ws in (([T], None), ([200, 90] + [1] * 40, None), ([290] + [1] * 40, Workspace(device))):
        k, _, table, slots = paged(device, dtype, T, 1, row, 0, ps, torch.randperm(22).tolist())
        pos = 0
        for n in cuts:
            ctx = fake_ctx(device, [n], [pos], [0])
            rows = proj[pos:pos + n].to(device).contiguous()
            q_att = torch.empty(n, nh * row, dtype=dtype, device=device)
            ops.latent_prepare(rows, 0, Q, norm_w.to(device), 1e-5, ctx.positions, freq, dims, slots[pos:pos + n].contiguous(), k,
                               q_att, nh, d, r, rank)
            ops.head_gemm(rows, d + r, uk_d, q_att, row)
            mixed = torch.empty(n, nh * rank, dtype=dtype, device=device)
            extra = dict(max_kv_len=pos + n, workspace=ws) if ws is not None and n == 1 else {}
            ops.paged_attention_simt(q_att, mixed, k, None, table, ctx.token_seq, ctx.positions, nh, 1, row, 0, m["scale"],
                                     v_head_dim=rank, max_q_len=n, values_in_keys=True, **extra)
            out = torch.empty(n, nh * dv, dtype=dtype, device=device)
            ops.head_gemm(mixed, rank, uv_d, out, dv, gate=rows[:, Q + row:])
            assert torch.allclose(out.cpu().double(), want[pos:pos + n], **tol_of(dtype, 3.0)), (cuts[:2], pos)
            pos += n


# ================================================================================================ whole models
MODEL_CASES = sorted(cases.CASES)
LENGTHS = {"long": (150, 11), "mid": (67, 12), "short": (23, 13), "one": (1, 14), "edge": (49, 15)}


def requests_of(case, names):
    return {n: wanted(case, *LENGTHS[n])[0] for n in names}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
def test_whole_prompts(device, case, dtype):
    """Also the first tokens of a sequence: every position's logits are compared, from position 0 on."""
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device)
    names = ["long", "one", "short", "edge"]
    got = helpers.replay(runner, helpers.trace_whole(requests_of(case, names)))
    check_replay(got, {n: LENGTHS[n] for n in names}, case, dtype, "whole prompts")
    runner.cache.check_invariants()
    assert runner.cache.num_free_slots == 4 and all(g.pool.num_used == 0 for g in runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
def test_every_layer_against_the_plain_layers(device, case, dtype):
    """The residual stream (the sum of the streams) after every layer, not only the logits."""
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device, graphs=False)
    ids = cases.random_ids(cases.CASES[case]["vocab"], 37, 3)
    want = []
    plain.forward(cases.CASES[case], weights_of(case), ids, layer_outputs=want)
    got = []
    runner.model.after_run = lambda i, h: got.append(h.detach().clone().cpu())
    helpers.replay(runner, helpers.trace_whole({"a": ids}))
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        scale = float(w.abs().max())
        assert float((g.double() - w).abs().max()) <= (1e-4 if dtype == "float32" else 6e-2) * scale, (case, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
def test_token_by_token_from_the_first_token(device, case, dtype):
    """A long decode: 150 single tokens through recorded steps, over page borders."""
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device)
    got = helpers.replay(runner, helpers.trace_tail_decoded(requests_of(case, ["long"]), tail=149))
    check_replay(got, {"long": LENGTHS["long"]}, case, dtype, "token by token")
    assert runner.graph_replays > 100  # the decode steps were replayed from graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
def test_prompt_then_decoded_tail(device, case, dtype):
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device, graphs=False)
    names = ["long", "mid", "edge"]
    got = helpers.replay(runner, helpers.trace_tail_decoded(requests_of(case, names), tail=40))
    check_replay(got, {n: LENGTHS[n] for n in names}, case, dtype, "prompt then single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
@pytest.mark.parametrize("sizes", [(2,), (7, 2, 13, 3, 5, 2, 16, 4, 9, 2, 31, 6), (64, 1, 2, 17)])
def test_portions(device, case, dtype, sizes):
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device)
    names = ["long", "short"] if sizes != (2,) else ["mid"]
    got = helpers.replay(runner, helpers.trace_portions(requests_of(case, names), sizes=sizes))
    check_replay(got, {n: LENGTHS[n] for n in names}, case, dtype, f"portions of {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
def test_mixed_batches_over_few_pages_and_slots(device, case, dtype):
    """Seven requests, at most three live, in a pool of three state slots and just enough pages: portions of some beside
    single tokens of others, requests that sit a step out, slots and pages that are used again by the next request."""
    names = ["mid", "short", "long", "one", "edge", "mid2", "short2"]
    lengths = dict(LENGTHS, mid2=(80, 21), short2=(30, 22))
    reqs = {n: wanted(case, *lengths[n])[0] for n in names}
    steps = helpers.trace_mixed(reqs, seed=5, max_live=3)
    pages = helpers.tokens_held(steps, round_to=16) // 16
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device, num_pages=pages, max_requests=3)
    got = helpers.replay(runner, steps)
    check_replay(got, {n: lengths[n] for n in names}, case, dtype, "mixed batches")
    runner.cache.check_invariants()
    assert runner.cache.num_free_slots == 3 and all(g.pool.num_used == 0 for g in runner.cache.groups)


def test_a_slot_that_is_used_again_starts_from_zero(device):
    """One state slot: the second request takes the slot (last shifted row, convolution inputs, recurrent states) and
    the pages the first one left, and computes what it computes alone."""
    case = "A"
    runner = make_runner(cases.CASES[case], weights_of(case), "float32", device, num_pages=10, max_requests=1)
    reqs = requests_of(case, ["long", "mid"])
    got = helpers.replay(runner, helpers.trace_portions(reqs, sizes=(40, 3, 1)))
    check_replay(got, {n: LENGTHS[n] for n in reqs}, case, "float32", "a slot used again")


def test_a_far_token_among_hundreds_in_a_long_prompt_and_decode(device):
    """640 tokens, the last 40 one by one, in 32-bit: every position against the plain implementation, so that keys
    and writes from hundreds of tokens ago are in every logit that is compared."""
    case = "C"
    ids, want = wanted(case, 640, 77)
    runner = make_runner(cases.CASES[case], weights_of(case), "float32", device, num_pages=48)
    got = helpers.replay(runner, helpers.trace_tail_decoded({"far": ids}, tail=40))
    check_replay(got, {"far": (640, 77)}, case, "float32", "a long prompt and its tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(device, tmp_path, dtype):
    """A folder of the design through ``Engine.generate`` (scheduler, portions, sampling on the device): every token
    is the plain implementation's greedy choice for the same prefix."""
    from ferrisinfer_b200 import SamplingParams
    from ferrisinfer_b200.engine.engine import Engine
    from ferrisinfer_b200.engine.scheduler import SchedulerConfig
    from ferrisinfer_b200.weights.safetensors_io import write_safetensors

    case = "A"
    cfg, weights = cases.CASES[case], weights_of(case)
    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    engine = Engine(folder, dtype=dtype, page_size=16, num_pages=40,
                    scheduler=SchedulerConfig(max_batch_size=4, max_prefill_chunk_tokens=32, max_prefill_batch_tokens=48,
                                              max_sequence_length=256))
    prompts = [cases.random_ids(cfg["vocab"], n, n) for n in (5, 70, 33, 1, 90, 12)]
    new = 20
    outs = engine.generate(prompts, SamplingParams.greedy(max_new_tokens=new))
    slack = 1e-4 if dtype == "float32" else 0.15
    for prompt, out in zip(prompts, outs):
        ids = out.generated_token_ids()
        assert len(ids) == new
        logits = plain.forward(cfg, weights, prompt + ids)[0]
        for i, tok in enumerate(ids):
            row = logits[len(prompt) + i - 1]
            assert row[tok] >= row.max() - slack * float(row.std()), (dtype, len(prompt), i, tok, int(row.argmax()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_trace_runner(device, tmp_path, dtype):
    """``bin/trace_run`` as a user runs it (a subprocess fed JSON lines, four state slots, just enough pages): a folder
    of the design is chosen by its config.json, and a mixed schedule over six requests gives the plain logits."""
    from test_trace_run_gpu import run_trace
    from ferrisinfer_b200.weights.safetensors_io import write_safetensors

    case = "B"
    cfg, weights = cases.CASES[case], weights_of(case)
    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    lengths = {"a": (70, 31), "b": (33, 32), "c": (101, 33), "d": (48, 34), "e": (64, 35), "f": (90, 36)}
    reqs = {n: wanted(case, *lengths[n])[0] for n in lengths}
    steps = helpers.trace_mixed(reqs, seed=2)
    got = run_trace(folder, dtype, steps, tmp_path / "out", helpers.tokens_held(steps), cfg["vocab"])
    check_replay(got, lengths, case, dtype, "the trace runner")


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_random_configuration_in_every_way_of_cutting(device, seed):
    """Configurations drawn at random (sizes, head counts and groupings, taps, streams, the order and number of the
    layers, pages of 4 to 32), replayed whole, with a decoded tail, in portions and in mixed batches, in 32-bit
    against the plain implementation and in bfloat16 against the 32-bit run's tolerance class."""
    import random

    rng = random.Random(seed)
    cfg = cases.random_config(rng)
    weights = cases.make_weights(cfg, seed)
    page = rng.choice([4, 8, 16, 16, 32])
    lengths = [rng.randint(1, 40), rng.randint(20, 140), rng.randint(2, 70), rng.randint(60, 200), rng.randint(1, 20)]
    reqs = {f"r{i}": cases.random_ids(cfg["vocab"], n, seed * 10 + i) for i, n in enumerate(lengths)}
    want = {rid: plain.forward(cfg, weights, ids)[0] for rid, ids in reqs.items()}
    traces = {"whole": helpers.trace_whole(reqs), "tail": helpers.trace_tail_decoded(reqs),
              "portions": helpers.trace_portions(reqs), "mixed": helpers.trace_mixed(reqs, seed)}
    for dtype in ("float32", "bfloat16"):
        for kind, steps in traces.items():
            pages = helpers.tokens_held(steps, round_to=page) // page
            runner = make_runner(cfg, weights, dtype, device, num_pages=pages, max_requests=8, page_size=page)
            got = helpers.replay(runner, steps)
            runner.cache.check_invariants()
            assert all(g.pool.num_used == 0 for g in runner.cache.groups)
            worst, over, count = 0.0, 0, 0
            for rid, ids in reqs.items():
                rows = torch.stack([got[(rid, p)] for p in range(len(ids))])
                assert torch.isfinite(rows).all(), (cfg, dtype, kind, rid)
                err = cases.row_errors(rows, want[rid])
                worst, over, count = max(worst, float(err.max())), over + int((err > cases.TOLERANCE[dtype]).sum()), count + len(ids)
            if dtype == "float32":
                assert worst <= cases.TOLERANCE[dtype], f"{cfg} page {page} {dtype} {kind}: {worst:.3g}"
            else:
                assert worst <= 4 * cases.TOLERANCE[dtype] and over <= max(1, count // 50), \
                    f"{cfg} page {page} {dtype} {kind}: {worst:.3g}, {over} of {count} over"


def test_a_model_without_any_pages(device):
    """Delta-rule layers only: no page group at all, state slots alone; portions and a decoded tail in 32-bit."""
    cfg = cases.config([cases.delta_layer(2, 1, 16, 24, 3, 64), cases.delta_layer(3, 3, 8, 8, 2, None)], width=40, vocab=61,
                       streams=2)
    weights = cases.make_weights(cfg, 9)
    ids = cases.random_ids(cfg["vocab"], 90, 4)
    want = plain.forward(cfg, weights, ids)[0]
    runner = make_runner(cfg, weights, "float32", device, num_pages=1, max_requests=2)
    assert not runner.cache.groups
    for steps in (helpers.trace_portions({"a": ids}), helpers.trace_tail_decoded({"a": ids}, tail=30)):
        got = helpers.replay(runner, steps)
        rows = torch.stack([got[("a", p)] for p in range(len(ids))])
        assert float(cases.row_errors(rows, want).max()) <= cases.TOLERANCE["float32"]
