"""Small Kugilix configurations and weights for the tests, and how a step function's logits are compared with the
plain implementation (``plain_kugilix``).

The weights are not N(0, 0.02): projections are drawn with a standard deviation of 1 / sqrt(inputs), norm weights
around one, convolution taps of a few tenths and decays spread between 0.5 and 1, so that every mechanism moves the
logits by far more than a tolerance (queries and keys are unit-normed by the design, so attention scores spread
over several units whatever the projections' scale).
"""

from __future__ import annotations

import math
import random

import torch


def attention_layer(heads, kv_heads, dim, vdim, window, ff, coef=0.3, every=7, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
             "scale": scale if scale is not None else 1.0 / math.sqrt(dim), "mask": {"size": window},
             "q_temp": {"coef": coef, "every": every}}
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def lightning_layer(heads, dim, vdim, ff, decay=None, seed=0):
    rng = random.Random(seed)
    decay = decay or [round(rng.uniform(0.5, 0.999), 4) for _ in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, width=64, vocab=97, groups=4, taps=4, loop=(0, 0, 1), eps=1e-6, scale=None):
    d = {"architecture": "Kugilix", "vocab": vocab, "width": width,
         "embedding": {"scale": scale if scale is not None else math.sqrt(width)},
         "norm": {"eps": eps, "groups": groups}, "layers": layers,
         "loop": {"start": loop[0], "stop": loop[1], "times": loop[2]}}
    if taps is not None:
        d["canon"] = {"taps": taps}
    return d


# A: both mixers, a looped span, value heads of the keys' size, window of three pages
CASE_A = config([attention_layer(4, 2, 32, 32, 48, 96), lightning_layer(2, 32, 32, 96, seed=1),
                 attention_layer(4, 2, 32, 32, 48, 96)], width=64, groups=4, taps=4, loop=(1, 3, 2))
# B: sizes that the usual model makes equal or one: value heads of another size, one kv head, as many kv heads as heads,
# one norm group, two taps, a loop from layer 0 that runs three times, a layer without a feed-forward, a window that is
# no multiple of a page, head sizes that are no multiple of 32
CASE_B = config([lightning_layer(3, 24, 40, None, seed=2), attention_layer(3, 1, 40, 24, 21, 72, coef=0.5, every=3),
                 attention_layer(2, 2, 16, 48, 37, 56, coef=0.1, every=16, scale=0.4)],
                width=48, vocab=131, groups=1, taps=2, loop=(0, 2, 3), eps=1e-5, scale=5.0)
# C: no loop at all, five taps, three norm groups, a window of one page exactly
CASE_C = config([attention_layer(6, 3, 16, 16, 16, 80, every=1), lightning_layer(4, 16, 16, 80, decay=[1.0, 0.9, 0.5, 0.0])],
                width=72, vocab=64, groups=3, taps=5, loop=(0, 0, 1))
# D: one tap (no state of the convolution), no convolution key at all in E
CASE_D = config([lightning_layer(2, 64, 64, 64, seed=4), attention_layer(2, 1, 64, 64, 30, 64)], width=64, taps=1,
                loop=(1, 2, 2))
CASE_E = config([attention_layer(2, 2, 32, 32, 25, 64), lightning_layer(1, 32, 32, None, seed=5)], width=32, groups=2,
                taps=None, loop=(0, 2, 2))
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D, "E": CASE_E}


def tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor of a folder of this configuration."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    taps = (cfg.get("canon") or {}).get("taps")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        out[p + ".norm1"] = (W,)
        if taps is not None:
            out[p + ".canon1"] = (W, taps)
        if layer["type"] == "attention":
            out[p + ".mix.q"] = (m["heads"] * m["dim"], W)
            out[p + ".mix.k"] = (m["kv_heads"] * m["dim"], W)
            out[p + ".mix.v"] = (m["kv_heads"] * m["vdim"], W)
            out[p + ".mix.o"] = (W, m["heads"] * m["vdim"])
        else:
            out[p + ".mix.q"] = out[p + ".mix.k"] = (m["heads"] * m["dim"], W)
            out[p + ".mix.v"] = out[p + ".mix.g"] = (m["heads"] * m["vdim"], W)
            out[p + ".mix.o"] = (W, m["heads"] * m["vdim"])
            out[p + ".mix.norm"] = (m["heads"] * m["vdim"],)
        if layer["mlp"] is not None:
            out[p + ".norm2"] = (W,)
            out[p + ".mlp.up"] = (layer["mlp"]["ff"], W)
            out[p + ".mlp.down"] = (W, layer["mlp"]["ff"])
            out[p + ".mlp.act"] = (2,)
    return out


def make_weights(cfg: dict, seed: int) -> dict:
    """bfloat16 tensors (as a folder stores them) for ``cfg``."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last == "canon1":
            t = 0.3 * torch.randn(shape, generator=g)
        elif last == "act":
            t = torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
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


TOLERANCE = {"float32": 2e-5, "bfloat16": 4e-2}
