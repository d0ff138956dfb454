"""A plain, slow Loduzen: float64, whole sequences, one function per mechanism, written from the design's
equations and sharing no code with the package.  It reads config.json's dictionary itself.

Notation: T tokens, x the stream [T, width], W stored [out, in] and applied as x @ W.T.
    rms(x)        = x / sqrt(mean(x^2) + eps)
    gelu(z)       = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
    layer         x += mixer(rms(x) w1);  x += ff(rms(x) w2) (if any);  x += rms(P (gelu(G x) * e_token)) ws (if any)
    mixer parallel  a_l * window_attention + a_r * gated_linear_attention, both on the same input
    mixer mamba2    a state-space layer
    output        logits = E rms(x) wf, E the embedding table
"""
import math

import torch

D = torch.float64


def rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ---------------------------------------------------------------------------------------------- rotation
def rotation_table(rot):
    """(frequency of every pair [dims / 2], amplitude) of a rotation description {base, dims, scaling?}."""
    n, base = rot["dims"], rot["base"]
    i = torch.arange(n // 2, dtype=D)
    f = base ** (-2.0 * i / n) if n else i
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def pair_with_turns(t):
        return n * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))

    lo = max(math.floor(pair_with_turns(sc["fast"])), 0)
    hi = min(math.ceil(pair_with_turns(sc["slow"])), n - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_pairs(x, positions, rot):
    """x [T, heads, dim]: the neighbours (2i, 2i+1) of the first rot.dims numbers turn by positions * f_i."""
    n = rot["dims"]
    if n == 0:
        return x
    f, amp = rotation_table(rot)
    ang = positions.to(D)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * amp)[:, None, :], (torch.sin(ang) * amp)[:, None, :]
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = a * c - b * s
    out[..., 1:n:2] = b * c + a * s
    return out


# ---------------------------------------------------------------------------------------------- mixers
def sink_softmax(scores, visible):
    """p_j = exp(s_j) / (1 + sum over visible i of exp(s_i)); invisible places get 0."""
    m = torch.clamp(torch.where(visible, scores, torch.full_like(scores, -1e300)).max(-1, keepdim=True).values, min=0.0)
    e = torch.where(visible, torch.exp(scores - m), torch.zeros_like(scores))
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def window_attention(h, w, p, m, eps):
    """Grouped-query attention; the value of a token is its projected key before norm and rotation."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = k.clone()
    pos = torch.arange(T)
    q = rotate_pairs(rms(q, eps, w[p + "q.norm"]), pos, m["rot"])
    k = rotate_pairs(rms(k, eps, w[p + "k.norm"]), pos, m["rot"])
    i, j = pos[:, None], pos[None, :]
    visible = (j <= i)
    size = (m.get("mask") or {}).get("size")
    if size:
        visible = visible & (i - j < size)
    out = torch.zeros(T, H, d, dtype=D)
    for hh in range(H):
        g = hh // (H // G)
        out[:, hh] = sink_softmax((q[:, hh] @ k[:, g].T) * m["scale"], visible) @ v[:, g]
    return out.reshape(T, H * d) @ w[p + "o"].T


def gated_linear_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    decay = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=D)
    o = torch.zeros(T, H, dv, dtype=D)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = (S * q[t][:, :, None]).sum(1)
    o = rms(o, eps, w[p + "norm"]).reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def causal_conv(x, weight, bias):
    """x [T, C], weight [C, taps] (last column: the current token), zeros before the start."""
    T, taps = x.shape[0], weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=D), x])
    y = bias[None, :].expand(T, -1).clone()
    for j in range(taps):
        y = y + padded[j:j + T] * weight[:, j][None, :]
    return y


def mamba2(h, w, p, m, eps):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, parts = H * P, m["norm_groups"]
    proj = h @ w[p + "in"].T
    z, ubc, d = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    ubc = silu(causal_conv(ubc, w[p + "conv"], w[p + "conv.b"]))
    u = ubc[:, :inner].view(T, H, P)
    B = ubc[:, inner:inner + G * N].view(T, G, N)
    C = ubc[:, inner + G * N:].view(T, G, N)
    dt = softplus(d + w[p + "dt_bias"])
    rate = torch.exp(w[p + "A_log"])
    group_of = torch.arange(H) // (H // G)
    S = torch.zeros(H, N, P, dtype=D)
    y = torch.zeros(T, H, P, dtype=D)
    for t in range(T):
        S = torch.exp(-rate * dt[t])[:, None, None] * S + dt[t][:, None, None] * B[t][group_of][:, :, None] * u[t][:, None, :]
        y[t] = (S * C[t][group_of][:, :, None]).sum(1) + w[p + "D"][:, None] * u[t]
    y = y.reshape(T, inner) * silu(z)
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


# ---------------------------------------------------------------------------------------------- the model
def feed_forward(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def token_side(x, tokens, w, p, layer, dim, eps):
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms(y, eps, w[p + "norm"])


def forward(w, cfg, tokens, streams=None):
    """Logits [T, vocab] of one whole sequence; `streams` (a list) collects the stream after the embedding and
    after every layer."""
    w = {k: v.to(D) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens]
    if streams is not None:
        streams.append(x.clone())
    side = (cfg.get("token_side") or {}).get("dim")
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms(x, eps, w[p + "norm1"])
        m = L["mixer"]
        if L["type"] == "parallel":
            x = x + m.get("left_scale", 1.0) * window_attention(h, w, p + "mix.left.", m["left"], eps) \
                + m.get("right_scale", 1.0) * gated_linear_attention(h, w, p + "mix.right.", m["right"], eps)
        elif L["type"] == "mamba2":
            x = x + mamba2(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            x = x + feed_forward(rms(x, eps, w[p + "norm2"]), w, p + "mlp.")
        if side:
            x = x + token_side(x, tokens, w, p + "side.", i, side, eps)
        if streams is not None:
            streams.append(x.clone())
    return rms(x, eps, w["final.norm"]) @ w["embed"].T


def argmax_lowest(row):
    return int((row == row.max()).nonzero()[0])
