"""The Nusudra decoder once more, plainly: one function per mechanism, float64 torch on the CPU, a whole sequence at
a time (or token by token through explicit states), sharing no code with the package.

Notation: a sequence of T tokens is a [T, ...] tensor; weights are a dict name -> tensor as the folder names them;
``cfg`` is the dict of config.json.  Every function takes what it needs explicitly.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms_div(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_div(x, eps) * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0.0)


def embedding(tokens, table, scale):
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


# --------------------------------------------------------------------------------------------- the layer's frame
def token_shift(h, shift, before=None):
    """h_t + (h_(t-1) - h_t) * shift with the unshifted h of the token before; ``before``: the row that precedes
    h[0] (None: zeros, the sequence starts here).  Returns the shifted rows and the last unshifted row."""
    prev = torch.zeros_like(h)
    prev[1:] = h[:-1]
    if before is not None:
        prev[0] = before
    return h + (prev - h) * shift, h[-1].clone()


def streams_read(xs, w_in):
    """xs [S, T, W] -> sum_s w_in[s] xs[s]."""
    return torch.einsum("s,stw->tw", w_in, xs)


def streams_write(xs, w_mix, w_out, y):
    """new[t] = sum_s mix[s, t] old[s] + out[t] y, all streams from the old ones."""
    return torch.einsum("sr,stw->rtw", w_mix, xs) + w_out[:, None, None] * y[None]


def causal_conv(x, w, bias=None, before=None):
    """Per channel: out_t = sum_j w[:, j] x_(t - taps + 1 + j) (+ bias).  x [T, C], w [C, taps]; ``before`` [taps - 1, C]:
    the inputs that precede x[0] (None: zeros).  Returns the outputs and the last taps - 1 inputs."""
    T, C = x.shape
    taps = w.shape[1]
    pad = torch.zeros(taps - 1, C, dtype=x.dtype) if before is None else before
    full = torch.cat([pad, x], dim=0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + full[j:j + T] * w[:, j]
    if bias is not None:
        out = out + bias
    return out, full[full.shape[0] - (taps - 1):].clone()


def rotate_half(x, positions, base, dims):
    """x [T, n, d]: the first ``dims`` of each vector rotated, dimension i paired with i + dims / 2, angle
    p * base^(-2 i / dims)."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = torch.as_tensor(positions, dtype=F)[:, None] * f[None]  # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def decayed_scan(q, k, v, g, S):
    """Per head: S_t = g_t S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, n]; v [T, H, dv]; g [T, H]; S [H, n, dv]."""
    S = S.clone()
    o = torch.zeros(v.shape, dtype=F)
    for t in range(q.shape[0]):
        S = g[t][:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hnv,hn->hv", S, q[t])
    return o, S


def delta_rule_scan(q, k, v, g, beta, S):
    """Per head: S <- g_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t (after the write)."""
    S = S.clone()
    o = torch.zeros(v.shape, dtype=F)
    for t in range(q.shape[0]):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hnv,hn->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hnv,hn->hv", S, q[t])
    return o, S


# --------------------------------------------------------------------------------------------- mixers
def latent_attention(h, w, p, m, eps, positions, past=None):
    """``past``: (latents [P, kv_rank], rotated key parts [P, rot_dim]) of the tokens before h[0], or None.
    Returns the mixer's output and the (latents, rotated parts) including this call's tokens."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + ".q"].T).reshape(T, H, d + r)
    q_plain, q_rot = q[..., :d], q[..., d:]
    dkv = h @ w[p + ".dkv"].T
    c = rms_norm(dkv[:, :rank], w[p + ".dkv.norm"], eps)
    k_rot = dkv[:, rank:].reshape(T, 1, r)
    rot = m["rot"]
    q_rot = rotate_half(q_rot, positions, rot["base"], rot["dims"])
    k_rot = rotate_half(k_rot, positions, rot["base"], rot["dims"])[:, 0]
    if past is not None:
        c = torch.cat([past[0], c], dim=0)
        k_rot = torch.cat([past[1], k_rot], dim=0)
    S = c.shape[0]
    k_plain = (c @ w[p + ".uk"].T).reshape(S, H, d)
    v = (c @ w[p + ".uv"].T).reshape(S, H, dv)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thr,sr->hts", q_rot, k_rot)) * m["scale"]
    first = S - T  # absolute position of h[0] within the keys
    i = torch.arange(T)[:, None] + first
    j = torch.arange(S)[None, :]
    scores = scores.masked_fill((j > i)[None], float("-inf"))
    o = torch.einsum("hts,shv->thv", torch.softmax(scores, dim=-1), v)
    gate = torch.sigmoid(h @ w[p + ".g"].T)  # [T, H]
    o = o * gate[..., None]
    return o.reshape(T, H * dv) @ w[p + ".o"].T, (c, k_rot)


def sink_attention(h, w, p, m, past=None):
    """Grouped-query attention without rotation: scores lose r1 ln(1 + r2 (i - j)); the softmax's denominator also
    holds exp(sink).  ``past``: (keys [P, G, d], values [P, G, dv]) before h[0]."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + ".q"].T + w[p + ".q.b"]).reshape(T, H, d)
    k = (h @ w[p + ".k"].T + w[p + ".k.b"]).reshape(T, G, d)
    v = (h @ w[p + ".v"].T + w[p + ".v.b"]).reshape(T, G, dv)
    if past is not None:
        k = torch.cat([past[0], k], dim=0)
        v = torch.cat([past[1], v], dim=0)
    S = k.shape[0]
    kv_of = torch.arange(H) // (H // G)
    scores = torch.einsum("thd,shd->hts", q, k[:, kv_of]) * m["scale"]
    i = torch.arange(T)[:, None] + (S - T)
    j = torch.arange(S)[None, :]
    dist = (i - j).clamp(min=0).to(F)
    scores = scores - w[p + ".r1"][:, None, None] * torch.log1p(w[p + ".r2"][:, None, None] * dist[None])
    scores = scores.masked_fill((j > i)[None], float("-inf"))
    sink = w[p + ".sink"][:, None, None].expand(H, T, 1)
    weights = torch.softmax(torch.cat([scores, sink], dim=-1), dim=-1)[..., :S]
    o = torch.einsum("hts,shv->thv", weights, v[:, kv_of])
    return o.reshape(T, H * dv) @ w[p + ".o"].T, (k, v)


def state_space(h, w, p, m, eps, past=None):
    """Mamba-2.  ``past``: (state [heads, N, vdim], last taps - 1 convolution inputs) or None."""
    T = h.shape[0]
    nh, dv, N, G, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = nh * dv
    proj = h @ w[p + ".in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc, conv_state = causal_conv(xbc, w[p + ".conv"], w[p + ".conv.b"], None if past is None else past[1])
    xbc = silu(xbc)
    x = xbc[:, :inner].reshape(T, nh, dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + ".dt_bias"])  # [T, nh]
    decay = torch.exp(-torch.exp(w[p + ".A_log"]) * dt)
    S = torch.zeros(nh, N, dv, dtype=F) if past is None else past[0]
    group_of = torch.arange(nh) // (nh // G)
    y, S = decayed_scan(C[:, group_of], B[:, group_of], dt[..., None] * x, decay, S)
    y = y + w[p + ".D"][:, None] * x
    y = y.reshape(T, inner) * silu(z)
    y = rms_div(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * w[p + ".norm"]
    return y @ w[p + ".o"].T, (S, conv_state)


def parallel_mixer(h, w, p, m, eps, past=None):
    left, lp = sink_attention(h, w, p + ".left", m["left"], None if past is None else past[0])
    right, rp = state_space(h, w, p + ".right", m["right"], eps, None if past is None else past[1])
    out = 0.5 * (rms_norm(left, w[p + ".left.out"], eps) + rms_norm(right, w[p + ".right.out"], eps))
    return out, (lp, rp)


def gated_delta(h, w, p, m, eps, past=None):
    """``past``: (state [heads, dim, vdim], last taps - 1 inputs of the q, k and v convolutions) or None."""
    T = h.shape[0]
    nh, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    conv_past = (None, None, None) if past is None else past[1]
    q, cq = causal_conv(h @ w[p + ".q"].T, w[p + ".q.conv"], None, conv_past[0])
    k, ck = causal_conv(h @ w[p + ".k"].T, w[p + ".k.conv"], None, conv_past[1])
    v, cv = causal_conv(h @ w[p + ".v"].T, w[p + ".v.conv"], None, conv_past[2])
    q, k, v = silu(q).reshape(T, G, d), silu(k).reshape(T, G, d), silu(v).reshape(T, nh, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + ".b"].T)  # [T, nh]
    g = torch.exp(-torch.exp(w[p + ".A_log"]) * softplus(h @ w[p + ".a"].T + w[p + ".dt_bias"]))
    S = torch.zeros(nh, d, dv, dtype=F) if past is None else past[0]
    qk_of = torch.arange(nh) // (nh // G)
    o, S = delta_rule_scan(q[:, qk_of], k[:, qk_of], v, g, beta, S)
    o = rms_div(o, eps) * w[p + ".norm"]
    o = o * silu(h @ w[p + ".g"].T).reshape(T, nh, dv)
    return o.reshape(T, nh * dv) @ w[p + ".o"].T, (S, (cq, ck, cv))


def feed_forward(h, w, p):
    z = torch.relu(h @ w[p + ".up"].T)
    return (z * z) @ w[p + ".down"].T


# --------------------------------------------------------------------------------------------- the model
def mixer(kind, h, w, p, m, eps, positions, past):
    if kind == "latent_attention":
        return latent_attention(h, w, p, m, eps, positions, past)
    if kind == "parallel":
        return parallel_mixer(h, w, p, m, eps, past)
    if kind == "delta":
        return gated_delta(h, w, p, m, eps, past)
    raise ValueError(kind)


def forward(cfg, w, tokens, state=None, layer_outputs=None):
    """Logits [T, vocab] of ``tokens`` continuing ``state`` (None: a new sequence); returns (logits, state).  The
    state is whatever the next call needs: the count of tokens so far and, per layer, the unshifted mixer input of the
    last token and the mixer's own past.  ``layer_outputs``: a list that receives the residual stream (the sum of
    the streams) after every layer."""
    w = {k: v.to(F) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    start = 0 if state is None else state["count"]
    T = len(tokens)
    positions = list(range(start, start + T))
    x = embedding(tokens, w["embed"], cfg.get("embedding", {}).get("scale", 1.0))
    streams = cfg.get("streams")
    xs = x[None].repeat(streams, 1, 1) if streams else None
    new_state = {"count": start + T, "layers": []}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        past = None if state is None else state["layers"][i]
        u = streams_read(xs, w[p + ".hc1.in"]) if streams else x
        h = rms_norm(u, w[p + ".norm1"], eps)
        h, last = token_shift(h, w[p + ".shift"], None if past is None else past[0])
        y, mixer_past = mixer(layer["type"], h, w, p + ".mix", layer["mixer"], eps, positions,
                              None if past is None else past[1])
        if streams:
            xs = streams_write(xs, w[p + ".hc1.mix"], w[p + ".hc1.out"], y)
        else:
            x = x + y
        if layer.get("mlp") is not None:
            u = streams_read(xs, w[p + ".hc2.in"]) if streams else x
            y = feed_forward(rms_norm(u, w[p + ".norm2"], eps), w, p + ".mlp")
            if streams:
                xs = streams_write(xs, w[p + ".hc2.mix"], w[p + ".hc2.out"], y)
            else:
                x = x + y
        new_state["layers"].append((last, mixer_past))
        if layer_outputs is not None:
            layer_outputs.append(xs.sum(0) if streams else x.clone())
    if streams:
        x = xs.sum(0)
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T, new_state


def softplus_scalar(x: float) -> float:
    return math.log1p(math.exp(-abs(x))) + max(x, 0.0)
