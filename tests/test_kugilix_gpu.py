"""The Kugilix decoder on the GPU against the plain implementation (``plain_kugilix``, float64): each kernel of
its mechanisms alone, then whole models of several small configurations driven through the step function the ways a
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
import kugilix_cases as cases
import plain_kugilix as plain

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
    return ids, plain.forward(cfg, weights_of(case), ids)


def check_replay(got: dict, requests: dict, case: str, dtype: str, what: str):
    """Every (request, position) of ``requests`` (id -> (n, seed)) is there and within tolerance."""
    worst, where = 0.0, None
    for rid, (n, seed) in requests.items():
        _, want = wanted(case, n, seed)
        rows = torch.stack([got[(rid, p)] for p in range(n)])
        assert torch.isfinite(rows).all(), f"{what}: request {rid} has logits that are not finite"
        err = cases.row_errors(rows, want)
        if float(err.max()) > worst:
            worst, where = float(err.max()), (rid, int(err.argmax()))
    assert worst <= cases.TOLERANCE[dtype], f"{what} ({case}, {dtype}): error {worst:.3g} at {where}"


def fake_ctx(device, q_lens, start_pos, slots):
    """The device arrays of a step, as the step function lays them out."""
    S = len(q_lens)
    q_start = [0]
    for n in q_lens:
        q_start.append(q_start[-1] + n)
    token_seq = [s for s in range(S) for _ in range(q_lens[s])]
    positions = [start_pos[s] + i for s in range(S) for i in range(q_lens[s])]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return SimpleNamespace(num_tokens=q_start[-1], num_seqs=S, max_q_len=max(q_lens), workspace=None,
                           token_seq=i32(token_seq), positions=i32(positions),
                           seq_q_start=i32(q_start), seq_start_pos=i32(start_pos), seq_state_slot=i32(slots))


# =========================================================================================== each mechanism alone
@pytest.mark.parametrize("hidden,groups", [(64, 4), (72, 3), (40, 1), (30, 5), (2048, 8)])
def test_grouped_rmsnorm(device, hidden, groups):
    ops = _ops()
    torch.manual_seed(hidden)
    x = torch.randn(9, hidden, device=device) * 3
    w = 1 + 0.2 * torch.randn(hidden, device=device)
    want = plain.grouped_rms_norm(x.double().cpu(), w.double().cpu(), groups, 1e-5)
    out = torch.empty(9, hidden, device=device)
    ops.grouped_rmsnorm(x, w, 1e-5, groups, out)
    assert torch.allclose(out.cpu().double(), want, atol=1e-5, rtol=1e-5)
    w2 = 1 + 0.2 * torch.randn(hidden, device=device)
    one, two = torch.empty_like(out), torch.empty_like(out)
    ops.grouped_rmsnorm_pair(x, w, w2, 1e-5, groups, one, two)  # both branches' norms in one launch
    assert torch.allclose(one, out, atol=1e-6, rtol=1e-6)  # (one group: the plain kernel sums in another order)
    assert torch.allclose(two.cpu().double(), plain.grouped_rms_norm(x.double().cpu(), w2.double().cpu(), groups, 1e-5),
                          atol=1e-5, rtol=1e-5)
    index = torch.tensor([7, 0, 7, 3], dtype=torch.int32, device=device)
    some = torch.empty(4, hidden, dtype=BF16, device=device)
    ops.grouped_rmsnorm(x, w, 1e-5, groups, some, index)
    assert torch.allclose(some.cpu().double(), want[index.cpu().long()], atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_embedding_with_scale_and_positions(device, dtype):
    from ferrisinfer_b200.parts.embedding import ScaledSinusoidalEmbedding

    torch.manual_seed(0)
    table = torch.randn(50, 36).to(dtype)
    part = ScaledSinusoidalEmbedding(50, 36, scale=6.0, weight_name="")
    part.bind({"e": table.to(device)}, "e")
    ids = [3, 49, 0, 17, 17]
    positions = [0, 1, 127, 4095, 20000]
    out = torch.empty(5, 36, device=device)
    part.forward(torch.tensor(ids, dtype=torch.int32, device=device), out,
                 torch.tensor(positions, dtype=torch.int32, device=device))
    want = table.double()[ids] * 6.0 + plain.sinusoid(positions, 36)
    # an fp32 angle of 20000 radians is good to a few thousandths
    assert torch.allclose(out.cpu().double()[:4], want[:4], atol=5e-4)
    assert torch.allclose(out.cpu().double()[4], want[4], atol=5e-3)


@pytest.mark.parametrize("taps", [1, 2, 4, 5])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_short_convolution_carries_its_inputs_across_steps(device, taps, dtype):
    """Three requests cut into steps of unequal sizes (one token, fewer tokens than taps, many), in slots that are not
    in order: every step's output equals the whole sequence's convolution."""
    ops = _ops()
    torch.manual_seed(taps)
    C = 40
    w = (0.5 * torch.randn(C, taps)).to(device)
    lens = [23, 9, 14]
    ys = [torch.randn(n, C).to(dtype) for n in lens]
    want = [plain.input_convolution(y.double(), w.double().cpu()) for y in ys]
    state = torch.zeros(5, max(taps - 1, 1), C, device=device)[:, :taps - 1]
    state = state.contiguous()
    slots = [3, 0, 2]
    cuts = [[1, 2, 1, 10, 3, 6], [2, 1, 1, 5], [14]]
    done = [0, 0, 0]
    k = 0
    while any(done[i] < lens[i] for i in range(3)):
        live = [i for i in range(3) if done[i] < lens[i] and k < len(cuts[i])]
        q_lens = [cuts[i][k] for i in live]
        ctx = fake_ctx(device, q_lens, [done[i] for i in live], [slots[i] for i in live])
        y = torch.cat([ys[i][done[i]:done[i] + n] for i, n in zip(live, q_lens)]).to(device)
        out = torch.empty_like(y)
        ops.short_conv(y, out, w, state if taps > 1 else None, ctx)
        row = 0
        for i, n in zip(live, q_lens):
            tol = 1e-5 if dtype == F32 else 3e-2
            assert torch.allclose(out[row:row + n].cpu().double(), want[i][done[i]:done[i] + n], atol=tol, rtol=tol), (i, k)
            row += n
            done[i] += n
        k += 1


@pytest.mark.parametrize("heads,dim,vdim", [(2, 64, 64), (3, 24, 40), (1, 100, 9), (2, 16, 130)])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_linear_attention_whole_portions_and_single_tokens(device, heads, dim, vdim, dtype):
    ops = _ops()
    torch.manual_seed(dim)
    T, W = 70, 12
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": [1.0, 0.97, 0.6][:heads]}
    w = {"m.q": torch.randn(heads * dim, W), "m.k": torch.randn(heads * dim, W) / 4, "m.v": torch.randn(heads * vdim, W)}
    u = torch.randn(T, W)
    proj = torch.cat([u @ w["m.q"].T, u @ w["m.k"].T, u @ w["m.v"].T], dim=1).to(dtype)
    # the oracle starts from the rounded projections, as the kernel does
    qn, kn = heads * dim, heads * dim

    def oracle(rows):
        p = rows.double()
        q, k, v = plain.silu(p[:, :qn]), plain.silu(p[:, qn:qn + kn]), plain.silu(p[:, qn + kn:])
        o = torch.zeros(len(rows), heads, vdim, dtype=F64)
        for h in range(heads):
            S = torch.zeros(dim, vdim, dtype=F64)
            for t in range(len(rows)):
                S = mixer["decay"][h] * S + torch.outer(k[t, h * dim:(h + 1) * dim], v[t, h * vdim:(h + 1) * vdim])
                o[t, h] = S.T @ q[t, h * dim:(h + 1) * dim]
        return o.reshape(len(rows), heads * vdim)

    want = oracle(proj.cpu())
    decay = torch.tensor(mixer["decay"], device=device)
    offsets = (0, qn, qn + kn)
    dev = proj.to(device)
    tol = dict(atol=2e-4 * float(want.abs().max()), rtol=1e-4)
    # the last two: portions longer than a segment (of 16 and of 7 tokens here) run as segments side by side
    for cuts, segment in (([T], None), ([1] * 20 + [2, 30, 3, 15], None), ([33, 1, 1, 35], None), ([T], 16),
                          ([9, 40, 1, 20], 7)):
        state = torch.full((3, heads, vdim, dim), 7.0, device=device)
        state[1].zero_()  # the request's slot; the others must stay as they are
        pos = 0
        for n in cuts:
            ctx = fake_ctx(device, [n], [pos], [1])
            out = torch.empty(n, heads * vdim, device=device)
            ops.linear_attention(dev[pos:pos + n], offsets, out, state, decay, ctx, heads, dim, vdim, silu=True,
                                 segment=segment)
            assert torch.allclose(out.cpu().double(), want[pos:pos + n], **tol), (cuts, segment, pos)
            pos += n
        assert bool((state[0] == 7).all()) and bool((state[2] == 7).all())


def test_linear_attention_segments_of_several_requests(device):
    """Three requests of unequal length in one step, two of them longer than a segment, one a single token, each from
    a state of its own: every request's outputs and final state equal those of the request run alone, unsegmented."""
    ops = _ops()
    torch.manual_seed(3)
    heads, dim, vdim = 2, 48, 24
    lens, slots = [50, 1, 37], [2, 0, 3]
    width = 2 * heads * dim + heads * vdim
    proj = torch.randn(sum(lens), width, device=device) * 0.7
    decay = torch.tensor([0.98, 0.8], device=device)
    start = torch.randn(4, heads, vdim, dim, device=device)
    offsets = (0, heads * dim, 2 * heads * dim)
    together = start.clone()
    out = torch.empty(sum(lens), heads * vdim, device=device)
    ops.linear_attention(proj, offsets, out, together, decay, fake_ctx(device, lens, [5, 9, 0], slots), heads, dim, vdim,
                         silu=True, segment=16)
    alone = start.clone()
    row = 0
    for n, slot in zip(lens, slots):
        one = torch.empty(n, heads * vdim, device=device)
        ops.linear_attention(proj[row:row + n], offsets, one, alone, decay, fake_ctx(device, [n], [0], [slot]), heads, dim,
                             vdim, silu=True, segment=1000)
        assert torch.allclose(out[row:row + n], one, atol=1e-4, rtol=1e-4), slot
        row += n
    assert torch.allclose(together, alone, atol=1e-4, rtol=1e-4)
    assert torch.equal(together[1], start[1])  # a slot that no request of the step holds


def test_linear_attention_keeps_a_key_from_hundreds_of_tokens_ago(device):
    """With a decay of one, a key that matches the last query, 600 tokens back among keys that do not, comes through
    with its value: one wrong state row or a lost update shows at full size."""
    ops = _ops()
    dim = vdim = 32
    T = 640
    q = torch.zeros(T, dim)
    k = torch.zeros(T, dim)
    v = torch.randn(T, vdim)
    k[:, 1:] = 0.01 * torch.randn(T, dim - 1)
    k[37, 0] = 5.0
    q[T - 1, 0] = 2.0
    proj = torch.cat([q, k, v], dim=1).to(device)
    state = torch.zeros(1, 1, vdim, dim, device=device)
    out = torch.empty(T, vdim, device=device)
    pos = 0
    for n in (300, 1, 1, 200, 138):
        ctx = fake_ctx(device, [n], [pos], [0])
        ops.linear_attention(proj[pos:pos + n], (0, dim, 2 * dim), out[pos:pos + n], state, torch.ones(1, device=device), ctx,
                             1, dim, vdim, silu=False)
        pos += n
    want = (q[T - 1].double() @ k.double().T) @ v.double()
    assert torch.allclose(out[T - 1].cpu().double(), want, atol=1e-4)
    assert float((out[T - 1].cpu() - 10.0 * v[37]).abs().max()) < 1e-3  # nothing but that one key counts


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_gated_rmsnorm(device, dtype):
    ops = _ops()
    torch.manual_seed(5)
    o = torch.randn(6, 88, device=device) * 4
    g = torch.randn(6, 200, device=device).to(dtype)
    w = 1 + 0.3 * torch.randn(88, device=device)
    out = torch.empty(6, 88, dtype=dtype, device=device)
    ops.gated_rmsnorm(o, g[:, 100:188], w, 1e-6, out)
    want = plain.rms_unit(o.double(), 1e-6) * w.double() * torch.sigmoid(g[:, 100:188].double())
    tol = 1e-5 if dtype == F32 else 2e-2
    assert torch.allclose(out.double(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("n", [1001, 4096])  # one value a thread; sixteen bytes a thread
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_xielu_activation(device, dtype, n):
    ops = _ops()
    z = torch.linspace(-9, 9, n, device=device).to(dtype)
    params = torch.tensor([0.4, -1.1], device=device)
    out = torch.empty_like(z)
    ops.activation(z, out, "xielu", params)
    want = plain.xielu(z.double(), 0.4, -1.1)
    tol = 1e-5 if dtype == F32 else 1e-2
    assert torch.allclose(out.double(), want, atol=tol, rtol=tol)
    ops.activation(z, z, "silu")
    assert torch.isfinite(z).all()


@pytest.mark.parametrize("T", [3, 16, 40, 130, 700])  # weight-stationary, tcgen05 short, token-major, CTA pairs
@pytest.mark.parametrize("kind", ["xielu", "silu"])
def test_up_product_with_the_activation_in_its_epilogue(device, T, kind):
    ops = _ops()
    torch.manual_seed(T)
    K, N = 192, 520
    x = torch.randn(T, K, device=device).to(BF16)
    w = (torch.randn(N, K, device=device) / math.sqrt(K)).to(BF16)
    params = torch.tensor([0.4, -1.1], device=device)
    coefficients = (math.log1p(math.exp(0.4)), 0.5 + math.log1p(math.exp(-1.1)))
    fused = torch.empty(T, N, dtype=BF16, device=device)
    ops.gemm_activation(x, w, fused, kind, coefficients, params)
    z = x.double() @ w.double().T
    want = plain.xielu(z, 0.4, -1.1) if kind == "xielu" else plain.silu(z)
    assert torch.allclose(fused.double(), want, atol=2e-2, rtol=2e-2)
    # nothing is left behind for the next product
    y = torch.empty(T, N, dtype=BF16, device=device)
    ops.gemm(x, w, None, y)
    assert torch.allclose(y.double(), z, atol=2e-2, rtol=2e-2)
    # 32-bit: the product, then the activation kernel
    out32 = torch.empty(T, N, device=device)
    ops.gemm_activation(x.float(), w.float(), out32, kind, coefficients, params)
    assert torch.allclose(out32.double(), want, atol=1e-4, rtol=1e-4)


def paged(device, dtype, T, nkv, d, dv, page_size, order):
    """Empty caches and the block table of one request whose pages are ``order``."""
    pages = max(order) + 1
    k = torch.zeros(pages, nkv, page_size, d, dtype=dtype, device=device)
    v = torch.zeros(pages, nkv, page_size, dv, dtype=dtype, device=device)
    table = torch.tensor([order], dtype=torch.int32, device=device)
    slots = torch.tensor([order[p // page_size] * page_size + p % page_size for p in range(T)], dtype=torch.int32, device=device)
    return k, v, table, slots


@pytest.mark.parametrize("nh,nkv,d,dv,window", [(4, 2, 32, 32, 21), (3, 1, 40, 24, 16), (2, 2, 16, 72, 50), (6, 3, 96, 96, 33),
                                                (5, 1, 8, 8, 64), (12, 2, 64, 32, 40)])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_unit_norm_temperature_slopes_window_attention(device, nh, nkv, d, dv, window, dtype):
    """q/k preparation + cache write + attention against the plain attention mixer (identity output matrix), over
    pages that are not in order, whole and then token by token from the cache."""
    ops = _ops()
    from ferrisinfer_b200.parts.position import DistanceSlopes

    torch.manual_seed(d + dv)
    T, W, ps = 75, 20, 16
    mixer = {"heads": nh, "kv_heads": nkv, "dim": d, "vdim": dv, "scale": 3.0 / math.sqrt(d), "mask": {"size": window},
             "q_temp": {"coef": 0.4, "every": 5}}
    w = {"m.q": torch.randn(nh * d, W), "m.k": torch.randn(nkv * d, W), "m.v": torch.randn(nkv * dv, W)}
    u = torch.randn(T, W)
    qkv = torch.cat([u @ w["m.q"].T, u @ w["m.k"].T, u @ w["m.v"].T], dim=1).to(dtype)
    # the oracle reads the rounded projections: its matrices only pick q, k and v out of the row
    wi = {"m.o": torch.eye(nh * dv, dtype=F64)}
    a, b = nh * d, nh * d + nkv * d
    for part, lo, hi in (("m.q", 0, a), ("m.k", a, b), ("m.v", b, qkv.shape[1])):
        wi[part] = torch.zeros(hi - lo, qkv.shape[1], dtype=F64)
        wi[part][:, lo:hi] = torch.eye(hi - lo, dtype=F64)
    want = plain.attention_mixer(qkv.double(), wi, "m", mixer, 1e-6)
    slopes = DistanceSlopes(8.0).score_slopes(nh, device)
    # bf16: the unit-normed queries and keys are rounded to 8 bits before scores of several units are formed from them
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == F32 else dict(atol=0.15, rtol=5e-2)
    for cuts in ([T], [40] + [1] * 35):
        k, v, table, slots = paged(device, dtype, T, nkv, d, dv, ps, [4, 0, 3, 1, 2])
        pos = 0
        for n in cuts:
            ctx = fake_ctx(device, [n], [pos], [0])
            rows = qkv[pos:pos + n].to(device).contiguous()
            ops.qk_prepare_cache_write(rows, ctx.positions, slots[pos:pos + n].contiguous(), k, v, nh, nkv, d, dv, 1e-6, (0.4, 5))
            out = torch.empty(n, nh * dv, dtype=dtype, device=device)
            ops.paged_attention_simt(rows, out, k, v, table, ctx.token_seq, ctx.positions, nh, nkv, d, window,
                                     mixer["scale"], score_slopes=slopes, v_head_dim=dv, max_q_len=n)
            assert torch.allclose(out.cpu().double(), want[pos:pos + n], **tol), (cuts, pos)
            if n > 1:  # the kernel of single tokens serves portions too, and agrees
                again = torch.empty_like(out)
                ops.paged_attention_simt(rows, again, k, v, table, ctx.token_seq, ctx.positions, nh, nkv, d, window,
                                         mixer["scale"], score_slopes=slopes, v_head_dim=dv, max_q_len=1)
                assert torch.allclose(again.cpu().double(), want[pos:pos + n], **tol), (cuts, pos)
            pos += n


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nh,nkv,d,dv", [(8, 2, 64, 64), (4, 2, 96, 32), (6, 1, 16, 16)])
def test_attention_of_single_tokens_in_shares_of_keys(device, nh, nkv, d, dv, dtype):
    """Single tokens of three requests, hundreds of keys deep: with scratch from a workspace the keys of a token are
    cut into shares that run side by side and query heads of a kv head share its keys; the result is that of the
    kernel that takes a token's keys in one go."""
    ops = _ops()
    from ferrisinfer_b200.engine.workspace import Workspace
    from ferrisinfer_b200.parts.position import DistanceSlopes

    torch.manual_seed(nh + d)
    ps, window = 16, 260
    held = [401, 77, 300]  # keys each request holds, its own token included
    blocks = [-(-n // ps) for n in held]
    pages = sum(blocks)
    k = torch.randn(pages + 1, nkv, ps, d, device=device).to(dtype)
    v = torch.randn(pages + 1, nkv, ps, dv, device=device).to(dtype)
    tables = torch.full((3, max(blocks)), -1, dtype=torch.int32)
    order, at = torch.randperm(pages).tolist(), 0
    for i, n in enumerate(blocks):
        tables[i, :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
        at += n
    tables = tables.to(device)
    ctx = fake_ctx(device, [1, 1, 1], [n - 1 for n in held], [0, 1, 2])
    qkv = torch.randn(3, nh * d + nkv * (d + dv), device=device).to(dtype)
    slopes = DistanceSlopes(8.0).score_slopes(nh, device)
    whole, shares = torch.empty(3, nh * dv, dtype=dtype, device=device), torch.empty(3, nh * dv, dtype=dtype, device=device)
    ops.paged_attention_simt(qkv, whole, k, v, tables, ctx.token_seq, ctx.positions, nh, nkv, d, window, 0.2,
                             score_slopes=slopes, v_head_dim=dv)
    ops.paged_attention_simt(qkv, shares, k, v, tables, ctx.token_seq, ctx.positions, nh, nkv, d, window, 0.2,
                             score_slopes=slopes, v_head_dim=dv, max_kv_len=max(held), workspace=Workspace(device))
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == F32 else dict(atol=2e-2, rtol=2e-2)
    assert torch.isfinite(shares.float()).all()
    assert torch.allclose(shares.float(), whole.float(), **tol)


def test_attention_tiles_that_hold_tokens_of_several_requests(device):
    """One step of four requests (a portion of 37, a single token deep in its sequence, a portion of two, one of 30
    from position 0), each over pages of its own: the tiled kernel's rows of one tile belong to several requests, and
    every row equals the kernel of single tokens, which takes rows one by one."""
    ops = _ops()
    from ferrisinfer_b200.parts.position import DistanceSlopes

    torch.manual_seed(9)
    nh, nkv, d, dv, ps, window = 4, 2, 32, 24, 16, 29
    q_lens, start = [37, 1, 2, 30], [20, 90, 7, 0]
    total = [a + b for a, b in zip(q_lens, start)]
    blocks = [-(-n // ps) for n in total]
    pages = sum(blocks)
    k = torch.randn(pages + 1, nkv, ps, d, device=device)
    v = torch.randn(pages + 1, nkv, ps, dv, device=device)
    order = torch.randperm(pages).tolist()
    tables = torch.full((4, max(blocks)), -1, dtype=torch.int32)
    at = 0
    for i, n in enumerate(blocks):
        tables[i, :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
        at += n
    tables = tables.to(device)
    S = len(q_lens)
    ctx = fake_ctx(device, q_lens, start, list(range(S)))
    T = sum(q_lens)
    qkv = torch.randn(T, nh * d + nkv * (d + dv), device=device)
    slopes = DistanceSlopes(8.0).score_slopes(nh, device)
    tiled, single = torch.empty(T, nh * dv, device=device), torch.empty(T, nh * dv, device=device)
    for out, longest in ((tiled, max(q_lens)), (single, 1)):
        ops.paged_attention_simt(qkv, out, k, v, tables, ctx.token_seq, ctx.positions, nh, nkv, d, window, 0.3,
                                 score_slopes=slopes, v_head_dim=dv, max_q_len=longest)
    assert torch.isfinite(tiled).all()
    assert torch.allclose(tiled, single, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("back,seen", [(0, True), (15, True), (16, True), (31, True), (32, True), (36, True), (37, False),
                                       (48, False)])
def test_attention_window_edge_one_key_stands_out(device, back, seen, tiled):
    """A window of 37 over pages of 16.  The key ``back`` positions before the last query points the query's way and every
    other key the opposite way, so the output is that key's value if (and only if) the window holds it."""
    ops = _ops()
    d, window, ps, T = 32, 37, 16, 70
    direction = torch.randn(d)
    direction /= direction.norm()
    keys = -direction.repeat(T, 1) + 0.01 * torch.randn(T, d)
    keys[T - 1 - back] = direction
    values = torch.randn(T, d)
    q = torch.zeros(T, d)
    q[T - 1] = direction
    qkv = torch.cat([q, keys, values], dim=1).to(device)
    k, v, table, slots = paged(device, F32, T, 1, d, d, ps, [2, 4, 1, 0, 3])
    ctx = fake_ctx(device, [T], [0], [0])
    ops.qk_prepare_cache_write(qkv, ctx.positions, slots, k, v, 1, 1, d, d, 1e-6, None)
    out = torch.empty(T, d, device=device)
    ops.paged_attention_simt(qkv, out, k, v, table, ctx.token_seq, ctx.positions, 1, 1, d, window, 1.0,
                             max_q_len=T if tiled else 1)
    # unit norm makes |q| = |k| = sqrt(d): the matching key scores +32, the others -32
    hit = float((out[T - 1].cpu() - values[T - 1 - back]).abs().max()) < 1e-3
    assert hit == seen


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
def test_token_by_token_from_the_first_token(device, case, dtype):
    """A long decode: 150 single tokens through recorded steps, over page borders and past every window."""
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
    """Six requests, at most three live, in a pool of three state slots and just enough pages: portions of some beside
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
    """One state slot: the second request takes the slot (convolution inputs, recurrent state) and the pages the
    first one left, and computes what it computes alone."""
    case = "A"
    runner = make_runner(cases.CASES[case], weights_of(case), "float32", device, num_pages=10, max_requests=1)
    reqs = requests_of(case, ["long", "mid"])
    got = helpers.replay(runner, helpers.trace_portions(reqs, sizes=(40, 3, 1)))
    check_replay(got, {n: LENGTHS[n] for n in reqs}, case, "float32", "a slot used again")


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
        logits = plain.forward(cfg, weights, prompt + ids)
        for i, tok in enumerate(ids):
            row = logits[len(prompt) + i - 1]
            assert row[tok] >= row.max() - slack * float(row.std()), (dtype, len(prompt), i, tok, int(row.argmax()))
