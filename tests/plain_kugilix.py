"""A plain, slow restatement of the Kugilix decoder, one function per mechanism, in one precision throughout
(float64 by default).  It shares no code with the package: it takes the dict of config.json and a dict of
tensors by name and loops over tokens where that is the clearest way to say what is computed.

Notation: W is the model width, t a position counted from 0 in its sequence.

  embedding          x_t = E[id_t] * scale + pe(t);  pe(t)[2i] = sin(t * 10000^(-2i / W)), pe(t)[2i+1] = cos(same)
  grouped RMS norm   the vector in `groups` equal consecutive parts; part / sqrt(mean(part^2) + eps); times w
  input convolution  u_t = y_t + sum_j c[:, j] * y_(t - taps + 1 + j), y before the sequence's start = 0
  lightning mixer    q, k, v = silu(Wq u), silu(Wk u), silu(Wv u), head by head;
                     S_t = decay_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;
                     out = Wo (rms(concat o) * n * sigmoid(Wg u))
  attention mixer    q, k per head divided by sqrt(mean(.^2) + eps);
                     q_t *= 1 + coef * ln(floor((t + 1) / every) + 1);
                     s_tj = (q_t . k_j) * scale - slope_h (t - j),  slope_h = 2^(-8 (h + 1) / H),
                     for 0 <= t - j < window; softmax; sum of values; Wo
  feed-forward       Wdown a(Wup y);  a(z) = softplus(p) z^2 + z / 2 for z > 0,
                     (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise
  layer              x <- x + (mixer(conv(norm1(x))) + ff(norm2(x)))
  loop               layers start .. stop-1 are run `times` times in a row; before each repeat the embedding
                     output is added to x
  output             logits = head . norm(x)
"""

from __future__ import annotations

import math

import torch


def sinusoid(positions, width, dtype=torch.float64):
    out = torch.zeros(len(positions), width, dtype=dtype)
    for n, p in enumerate(positions):
        for i in range(width // 2):
            a = p * 10000.0 ** (-2.0 * i / width)
            out[n, 2 * i] = math.sin(a)
            out[n, 2 * i + 1] = math.cos(a)
    return out


def embed(table, ids, scale, start=0):
    x = table[torch.as_tensor(ids, dtype=torch.long)] * scale
    return x + sinusoid(range(start, start + len(ids)), table.shape[1], x.dtype)


def grouped_rms_norm(x, w, groups, eps):
    T, n = x.shape
    parts = x.reshape(T, groups, n // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(T, n) * w


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def input_convolution(y, c):
    """y [T, W], c [W, taps]."""
    T, _ = y.shape
    taps = c.shape[1]
    out = y.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += c[:, j] * y[s]
    return out


def silu(z):
    return z * torch.sigmoid(z)


def lightning(u, w, prefix, mixer):
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    decay = mixer["decay"]
    T = u.shape[0]
    q = silu(u @ w[prefix + ".q"].T).reshape(T, heads, dim)
    k = silu(u @ w[prefix + ".k"].T).reshape(T, heads, dim)
    v = silu(u @ w[prefix + ".v"].T).reshape(T, heads, vdim)
    o = torch.zeros(T, heads, vdim, dtype=u.dtype)
    for h in range(heads):
        S = torch.zeros(dim, vdim, dtype=u.dtype)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ q[t, h]
    return o.reshape(T, heads * vdim)


def lightning_mixer(u, w, prefix, mixer, eps):
    o = lightning(u, w, prefix, mixer)
    o = rms_unit(o, eps) * w[prefix + ".norm"]
    o = o * torch.sigmoid(u @ w[prefix + ".g"].T)
    return o @ w[prefix + ".o"].T


def attention_mixer(u, w, prefix, mixer, eps):
    H, G, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    window = mixer["mask"]["size"]
    coef, every = mixer["q_temp"]["coef"], mixer["q_temp"]["every"]
    T = u.shape[0]
    q = rms_unit((u @ w[prefix + ".q"].T).reshape(T, H, dim), eps)
    k = rms_unit((u @ w[prefix + ".k"].T).reshape(T, G, dim), eps)
    v = (u @ w[prefix + ".v"].T).reshape(T, G, vdim)
    out = torch.zeros(T, H, vdim, dtype=u.dtype)
    for t in range(T):
        temp = 1.0 + coef * math.log((t + 1) // every + 1)
        lo = max(0, t - window + 1)
        for h in range(H):
            g = h // (H // G)
            slope = 2.0 ** (-8.0 * (h + 1) / H)
            dist = torch.arange(t - lo, -1, -1, dtype=u.dtype)  # t - j for j = lo .. t
            s = (k[lo:t + 1, g] @ (q[t, h] * temp)) * mixer["scale"] - slope * dist
            p = torch.softmax(s, dim=0)
            out[t, h] = p @ v[lo:t + 1, g]
    return out.reshape(T, H * vdim) @ w[prefix + ".o"].T


def xielu(z, p, q):
    sp = math.log1p(math.exp(p))
    sq = math.log1p(math.exp(q))
    pos = sp * z * z + z / 2
    neg = (0.5 + sq) * (torch.exp(torch.clamp(z, max=0.0)) - 1 - z) + z / 2
    return torch.where(z > 0, pos, neg)


def feed_forward(y, w, prefix):
    a = w[prefix + ".act"]
    return xielu(y @ w[prefix + ".up"].T, float(a[0]), float(a[1])) @ w[prefix + ".down"].T


def run_order(config):
    """Layer indices in the order in which they run, and whether the embedding output is added before each."""
    n = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for r in range(times if stop > start else 0):
        order += [(i, r > 0 and i == start) for i in range(start, stop)]
    order += [(i, False) for i in range(stop, n)]
    return order


def forward(config, weights, ids, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence from its start.  ``layers_out``: a list that receives the residual stream
    after every layer run."""
    w = {n: t.to(dtype) for n, t in weights.items()}
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    x0 = embed(w["embed"], ids, config["embedding"]["scale"])
    x = x0.clone()
    for i, again in run_order(config):
        layer = config["layers"][i]
        p = f"l{i}"
        if again:
            x = x + x0
        y = grouped_rms_norm(x, w[p + ".norm1"], groups, eps)
        u = input_convolution(y, w[p + ".canon1"]) if p + ".canon1" in w else y
        if layer["type"] == "lightning":
            m = lightning_mixer(u, w, p + ".mix", layer["mixer"], eps)
        elif layer["type"] == "attention":
            m = attention_mixer(u, w, p + ".mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            m = m + feed_forward(grouped_rms_norm(x, w[p + ".norm2"], groups, eps), w, p + ".mlp")
        x = x + m
        if layers_out is not None:
            layers_out.append(x.clone())
    y = grouped_rms_norm(x, w["final.norm"], groups, eps)
    return y @ w["head"].T
