"""A plain, slow implementation of the Bidinex decoder, whole sequences at once, float64.

One function per mechanism, written from the equations and sharing nothing with the package: it reads
config.json's dictionary itself and takes weights as a dict of float64 tensors by their stored names.
Keys and values are expanded per head here (the package never does that), attention is a loop over
heads with a full score matrix, experts are run on every token and masked.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


def dynamic_tanh(x, w, b, alpha):
    """tanh(alpha * x) * w + b, element by element."""
    return torch.tanh(alpha * x) * w + b


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w along the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotate(x, positions, base: float, dims: int):
    """Rotary positions on the first `dims` numbers of the last dimension of x [T, ..., n]: number i is
    paired with i + dims/2; (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims)."""
    if dims == 0:
        return x.clone()
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = positions.to(F64)[:, None] * f[None, :]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * torch.cos(a) - v * torch.sin(a), v * torch.cos(a) + u * torch.sin(a), x[..., dims:]], -1)


def latent_attention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, positions=None,
                     window: Optional[int] = None, probe: Optional[dict] = None):
    """The mixer of one layer on h [T, width]; p is the tensor prefix ('l0.mix.'), m the mixer's sizes."""
    T = h.shape[0]
    H, d, r, vd, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T).view(T, H, d + r)
    dkv = h @ w[p + "dkv"].T
    c = rms_norm(dkv[:, :R], w[p + "dkv.norm"], eps)
    k_rot = rotate(dkv[:, R:], pos, m["rot"]["base"], m["rot"]["dims"])            # [T, r], shared by all heads
    q_rot = rotate(q[:, :, d:], pos, m["rot"]["base"], m["rot"]["dims"])           # [T, H, r]
    k_un = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, vd)
    gate = torch.sigmoid(h @ w[p + "g"].T)                                          # [T, H]
    out = torch.zeros(T, H, vd, dtype=F64)
    for hd in range(H):
        s = (q[:, hd, :d] @ k_un[:, hd, :].T + q_rot[:, hd, :] @ k_rot.T) * m["scale"]
        i = pos[:, None]
        j = pos[None, :]
        visible = j <= i
        if window:
            visible = visible & (i - j < window)
        s = s.masked_fill(~visible, -math.inf)
        pr = torch.softmax(s, -1)
        if probe is not None:
            probe.setdefault("probs", []).append(pr)
        out[:, hd, :] = (pr @ v[:, hd, :]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * vd) @ w[p + "o"].T


def route(z, top: int, groups: int, keep: int):
    """Router logits z [T, E] -> (chosen experts [T, top] by falling score, their weights [T, top])."""
    T, E = z.shape
    s = torch.softmax(z, -1)
    per = E // groups
    idx_out, w_out = [], []
    for t in range(T):
        st = s[t]
        gscore = [max(st[g * per:(g + 1) * per].tolist()) for g in range(groups)]
        kept = sorted(range(groups), key=lambda g: (-gscore[g], g))[:keep]
        allowed = [e for e in range(E) if e // per in kept]
        chosen = sorted(allowed, key=lambda e: (-st[e].item(), e))[:top]
        tot = sum(st[e].item() for e in chosen) + 1e-20
        idx_out.append(chosen)
        w_out.append([st[e].item() / tot for e in chosen])
    return torch.tensor(idx_out), torch.tensor(w_out, dtype=F64)


def expert(h, gate, up, down):
    g = h @ gate.T
    return ((g * torch.sigmoid(g)) * (h @ up.T)) @ down.T


def mixture_of_experts(h, w: Dict[str, torch.Tensor], p: str, f: dict):
    """The feed-forward of one layer on h [T, width]; p is the tensor prefix ('l0.mlp.')."""
    r = f["router"]
    g = r.get("groups") or {}
    groups = g.get("count", 1)
    idx, wt = route(h @ w[p + "router"].T, r["top"], groups, g.get("keep", groups))
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        y = expert(h, w[p + f"e{e}.gate"], w[p + f"e{e}.up"], w[p + f"e{e}.down"])
        share = (wt * (idx == e)).sum(-1, keepdim=True)
        out = out + share * y
    return out


def inject(x, x0, w_in):
    """x <- W_in [x ; x0]."""
    return torch.cat([x, x0], -1) @ w_in.T


def softcap(x, cap):
    return cap * torch.tanh(x / cap)


def layer_runs(cfg: dict):
    """(layer, opens a pass) for every run, in order."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(lp["start"])]
    for _ in range(lp["times"]):
        runs += [(i, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, False) for i in range(lp["stop"], n)]


def forward(w: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int], streams: Optional[List] = None,
            window: Optional[int] = None):
    """Logits [T, vocab] of a whole sequence.  `streams` collects the stream after the embedding and after
    every run of a layer.  `window` (no model of this design has one; the mixer does): every mixer sees the
    last `window` positions only."""
    def dyt(x, name):
        return dynamic_tanh(x, w[name], w[name + ".b"], w[name + ".alpha"])

    x = w["embed"][torch.tensor(list(tokens))] * cfg.get("embedding", {}).get("scale", 1.0)
    x = dyt(x, "embed.norm")
    x0 = x
    if streams is not None:
        streams.append(x.clone())
    m = cfg.get("residual_mult", 1.0)
    eps = cfg["norm"]["eps"]
    for i, opens in layer_runs(cfg):
        if opens:
            x = inject(x, x0, w["loop.in"])
        L = cfg["layers"][i]
        x = x + m * latent_attention(dyt(x, f"l{i}.norm1"), w, f"l{i}.mix.", L["mixer"], eps, window=window)
        if L.get("mlp") is not None:
            x = x + m * mixture_of_experts(dyt(x, f"l{i}.norm2"), w, f"l{i}.mlp.", L["mlp"])
        if streams is not None:
            streams.append(x.clone())
    logits = dyt(x, "final.norm") @ w["embed"].T
    cap = cfg.get("logit_softcap")
    return softcap(logits, cap) if cap else logits


def argmax_lowest(row) -> int:
    m = row.max()
    return int((row == m).nonzero()[0].item())
