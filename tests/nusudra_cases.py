"""Small Nusudra configurations and weights for the tests, and how logits are compared with the plain
implementation (``plain_nusudra``).

The weights are not N(0, 0.02): projections are drawn with a standard deviation of 1 / sqrt(inputs), norm weights
around one, stream weights around a plain residual sum (in ~ 1 / S, mix ~ identity, out ~ 1) with enough noise that
every entry matters, shifts spread over 0 .. 0.6, taps of a few tenths, decays spread widely, distance penalties and
sinks of order one: every mechanism moves the logits by far more than a tolerance.
"""

from __future__ import annotations

import math
import random

import torch


def mlp(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def latent_layer(heads, dim, rot_dim, vdim, kv_rank, ff, base=10000.0, dims=None, scale=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
             "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim),
             "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp(ff)}


def delta_layer(heads, kv_heads, dim, vdim, conv, ff):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp(ff)}


def parallel_layer(left, right, ff):
    heads, kv_heads, dim, vdim = left
    rh, rv, state, groups, norm_groups, conv = right
    return {"type": "parallel", "mlp": mlp(ff), "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 1.0 / math.sqrt(dim)},
        "right": {"heads": rh, "vdim": rv, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}}}


def config(layers, width=64, vocab=97, streams=3, eps=1e-6, scale=None):
    d = {"architecture": "Nusudra", "vocab": vocab, "width": width,
         "embedding": {"scale": scale if scale is not None else math.sqrt(width)}, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        d["streams"] = streams
    return d


# A: all three mixers; grouped q/k heads in the delta rule and grouped kv heads in the attention (two value heads a
# q/k head), two groups of the state-space layer normed in four parts
CASE_A = config([delta_layer(4, 2, 32, 16, 4, 96),
                 latent_layer(4, 16, 16, 24, 48, 96),
                 parallel_layer((4, 2, 32, 32), (4, 16, 16, 2, 4, 4), 96)], width=64, streams=3)
# B: sizes that a usual model makes equal or one: one q/k head for all, one kv head, one group and one norm part, value
# heads larger than keys, only a part of the rotated dimensions rotating, head sizes that are no multiple of 32, two
# taps and three, one residual stream, a layer without a feed-forward, another base and eps
CASE_B = config([parallel_layer((3, 1, 24, 40), (3, 8, 24, 1, 1, 2), None),
                 delta_layer(3, 1, 24, 40, 3, 72),
                 latent_layer(3, 24, 8, 40, 32, 56, base=500.0, dims=4, scale=0.3)],
                width=48, vocab=131, streams=1, eps=1e-5, scale=5.0)
# C: no streams at all (plain residual layers), one tap (no convolution state), as many q/k heads as heads, two
# streams of attention in a row, eight heads sharing two
CASE_C = config([latent_layer(2, 32, 32, 32, 64, 80),
                 latent_layer(8, 8, 8, 8, 16, None),
                 delta_layer(2, 2, 64, 64, 1, 80),
                 parallel_layer((8, 2, 16, 16), (2, 32, 32, 2, 2, 1), 64)], width=72, vocab=64, streams=None)
# D: five streams, five taps, a state-space layer alone in front, heads of 128
CASE_D = config([parallel_layer((2, 2, 64, 64), (1, 128, 64, 1, 2, 5), 64),
                 delta_layer(1, 1, 128, 128, 5, None)], width=32, vocab=50, streams=5)
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D}


def tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor of a folder of this configuration."""
    W, V, S = cfg["width"], cfg["vocab"], cfg.get("streams")
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        out[p + ".norm1"] = (W,)
        out[p + ".shift"] = (W,)
        subs = ["hc1"]
        if layer["mlp"] is not None:
            out[p + ".norm2"] = (W,)
            out[p + ".mlp.up"] = (layer["mlp"]["ff"], W)
            out[p + ".mlp.down"] = (W, layer["mlp"]["ff"])
            subs.append("hc2")
        if S is not None:
            for hc in subs:
                out[f"{p}.{hc}.in"] = out[f"{p}.{hc}.out"] = (S,)
                out[f"{p}.{hc}.mix"] = (S, S)
        q = p + ".mix"
        if layer["type"] == "latent_attention":
            H = m["heads"]
            out[q + ".q"] = (H * (m["dim"] + m["rot_dim"]), W)
            out[q + ".dkv"] = (m["kv_rank"] + m["rot_dim"], W)
            out[q + ".dkv.norm"] = (m["kv_rank"],)
            out[q + ".uk"] = (H * m["dim"], m["kv_rank"])
            out[q + ".uv"] = (H * m["vdim"], m["kv_rank"])
            out[q + ".g"] = (H, W)
            out[q + ".o"] = (W, H * m["vdim"])
        elif layer["type"] == "delta":
            H, G = m["heads"], m["kv_heads"]
            for n, rows in (("q", G * m["dim"]), ("k", G * m["dim"]), ("v", H * m["vdim"])):
                out[f"{q}.{n}"] = (rows, W)
                out[f"{q}.{n}.conv"] = (rows, m["conv"])
            out[q + ".b"] = out[q + ".a"] = (H, W)
            out[q + ".A_log"] = out[q + ".dt_bias"] = (H,)
            out[q + ".norm"] = (m["vdim"],)
            out[q + ".g"] = (H * m["vdim"], W)
            out[q + ".o"] = (W, H * m["vdim"])
        else:
            l, r = m["left"], m["right"]
            for n, rows in (("q", l["heads"] * l["dim"]), ("k", l["kv_heads"] * l["dim"]), ("v", l["kv_heads"] * l["vdim"])):
                out[f"{q}.left.{n}"] = (rows, W)
                out[f"{q}.left.{n}.b"] = (rows,)
            out[q + ".left.r1"] = out[q + ".left.r2"] = out[q + ".left.sink"] = (l["heads"],)
            out[q + ".left.o"] = (W, l["heads"] * l["vdim"])
            inner, bc = r["heads"] * r["vdim"], r["groups"] * r["state"]
            out[q + ".right.in"] = (2 * inner + 2 * bc + r["heads"], W)
            out[q + ".right.conv"] = (inner + 2 * bc, r["conv"])
            out[q + ".right.conv.b"] = (inner + 2 * bc,)
            out[q + ".right.dt_bias"] = out[q + ".right.A_log"] = out[q + ".right.D"] = (r["heads"],)
            out[q + ".right.norm"] = (inner,)
            out[q + ".right.o"] = (W, inner)
            out[q + ".left.out"] = out[q + ".right.out"] = (W,)
    return out


def make_weights(cfg: dict, seed: int) -> dict:
    """bfloat16 tensors (as a folder stores them) for ``cfg``."""
    g = torch.Generator().manual_seed(seed)
    randn = lambda shape: torch.randn(shape, generator=g)
    S = cfg.get("streams")
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm", "out") and len(shape) == 1 and ".hc" not in name:
            t = 1.0 + 0.1 * randn(shape)
        elif ".hc" in name and last == "in":
            t = 1.0 / S + 0.3 * randn(shape)
        elif ".hc" in name and last == "out":
            t = 1.0 + 0.3 * randn(shape)
        elif ".hc" in name and last == "mix":
            t = torch.eye(S) + 0.2 * randn(shape)
        elif last == "shift":
            t = 0.6 * torch.rand(shape, generator=g)
        elif last == "conv":
            t = 0.5 * randn(shape)
        elif last == "b" and len(shape) == 1:
            t = 0.2 * randn(shape)
        elif last == "A_log":
            t = -1.0 + 1.5 * randn(shape)
        elif last == "dt_bias":
            t = randn(shape)
        elif last == "D":
            t = 1.0 + 0.3 * randn(shape)
        elif last == "r1":
            t = 0.5 + 0.5 * torch.rand(shape, generator=g)
        elif last == "r2":
            t = 0.1 + torch.rand(shape, generator=g)
        elif last == "sink":
            t = randn(shape)
        elif name == "embed":
            t = randn(shape) / math.sqrt(shape[1])
        else:
            t = randn(shape) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out


def random_ids(vocab: int, n: int, seed: int) -> list:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: root mean square of the difference (its mean taken off) over the standard deviation of the wanted row."""
    d = got.double() - want.double()
    d = d - d.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / want.double().std(dim=-1)


TOLERANCE = {"float32": 3e-5, "bfloat16": 5e-2}


def random_config(rng: random.Random) -> dict:
    """A configuration drawn at random: sizes, head counts, groupings, taps, streams, the order of the layers."""
    divisor = lambda n: rng.choice([d for d in range(1, n + 1) if n % d == 0])
    size = lambda: rng.choice([8, 16, 24, 32, 40, 64])
    width = rng.choice([40, 48, 64, 72, 96])
    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["delta", "latent", "parallel"])
        ff = None if rng.random() < 0.2 else rng.choice([56, 64, 96, 128])
        if kind == "delta":
            heads = rng.choice([1, 2, 3, 4, 6])
            layers.append(delta_layer(heads, divisor(heads), size(), size(), rng.randint(1, 4), ff))
        elif kind == "latent":
            rot = rng.choice([8, 16, 32])
            layers.append(latent_layer(rng.randint(1, 6), size(), rot, size(), rng.choice([16, 24, 32, 64, 136]), ff,
                                       base=rng.choice([100.0, 10000.0, 500000.0])))
        else:
            heads, rh, rv = rng.choice([1, 2, 4, 6]), rng.choice([1, 2, 3, 4, 8]), rng.choice([8, 16, 32])
            layers.append(parallel_layer((heads, divisor(heads), size(), size()),
                                         (rh, rv, rng.choice([8, 16, 24, 32, 64]), divisor(rh), divisor(rh) * rng.choice([1, 2]),
                                          rng.randint(1, 4)), ff))
    return config(layers, width=width, vocab=rng.randint(40, 200), streams=rng.choice([None, 1, 2, 3, 4, 6]),
                  eps=rng.choice([1e-6, 1e-5]), scale=rng.choice([None, 3.0, 12.0]))
