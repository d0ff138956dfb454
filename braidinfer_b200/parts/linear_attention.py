"""Gated linear attention: a matrix of state per head instead of a cache of keys and values.

For the mixer's input x (a row per token), per head h with key size dk and value size dv:
    q = Wq x * dk^-1/2,   k = Wk x,   v = Wv x,   g = Wg x
    a = sigmoid(Wa2 (Wa1 x) + b)^(1/tau)            a decay per key channel, in (0, 1); the gate's map is low-rank
    S <- diag(a) S + k v^T                           S is [dk, dv], zero at the start of a sequence
    o = S^T q
    out = Wo concat_h( o / sqrt(mean(o^2) + eps) * w * silu(g) )        w: dv numbers shared by the heads
(Yang, Wang, Shen, Panda, Kim: "Gated Linear Attention Transformers with Hardware-Efficient Training", 2023.)
The state, the decay (through its logarithm), the recurrence and the norm are float32; S lives in the
sequence's slot of the state area and is carried from step to step, so a prompt may be cut anywhere.
Per step: one stacked product (q | k | v | g | Wa1 x), the small product Wa2 with float32 output, the
recurrence kernel (the decay is computed where it is used), the gated norm, the output product with the
residual sum in its epilogue.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import MIXERS, Mixer
from .linear import Linear
from .spec import TensorSpec


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    """params: hidden_size, num_heads, dim (key size a head), vdim (value size a head), tau, eps, out_mult
    (default 1), gate_rank (the inner size of the decay's low-rank map), and the tensor names q, k, v, g, a1, a2,
    a2_bias, norm, o (under the prefix)."""

    DECAY_IN_PLACE_ROWS = 64

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dk = int(p["dim"])
        self.dv = int(p["vdim"])
        self.rank = int(p["gate_rank"])
        self.tau = float(p["tau"])
        self.eps = float(p["eps"])
        self.out_mult = float(p.get("out_mult", 1.0))
        if self.tau <= 0:
            raise ValueError(f"gated_linear_attention: tau must be positive, got {self.tau}")
        if self.dk > 256:
            raise ValueError(f"gated_linear_attention: key sizes up to 256 a head are built, not {self.dk}")
        H, dk, dv = self.heads, self.dk, self.dv
        self.cols = [H * dk, H * dk, H * dv, H * dv, self.rank]
        self.proj = Linear(runtime, [prefix + p.get(n, "mix." + n) for n in ("q", "k", "v", "g", "a1")], self.cols, self.hidden)
        self.a2 = Linear(runtime, [prefix + p.get("a2", "mix.a2")], [H * dk], self.rank)
        self.a2_bias_name = prefix + p.get("a2_bias", "mix.a2.b")
        self.norm_name = prefix + p.get("norm", "mix.norm")
        self.o = Linear(runtime, [prefix + p.get("o", "mix.o")], [self.hidden], H * dv)
        self.a2_bias = self.norm_w = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.proj.tensor_specs())
        d.update(self.a2.tensor_specs())
        d[self.a2_bias_name] = TensorSpec((self.heads * self.dk,), std=1.0)
        d[self.norm_name] = TensorSpec((self.dv,), init="one_plus_normal")
        d.update(self.o.tensor_specs())
        return d

    def load(self, tensors) -> None:
        self.proj.load(tensors)
        w = self.proj.weight
        # every part of the stacked result starts on 16 bytes: the gate's low-rank part is read as a product's input
        pad = -w.shape[0] % 8
        if pad:
            self.proj.weight = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)]).contiguous()
        self.a2.load(tensors)
        self.o.load(tensors)
        self.a2_bias, self.norm_w = tensors[self.a2_bias_name], tensors[self.norm_name]

    def state_bytes(self) -> int:
        return self.heads * self.dk * self.dv * 4

    def forward(self, x, residual, ctx, cache, state):
        if state is None:
            raise RuntimeError("gated_linear_attention needs its state area")
        K = self.rt.kernels
        rows = x.shape[0]
        H, dk, dv = self.heads, self.dk, self.dv
        proj = self.proj.forward(x)                                     # [rows, q | k | v | g | a1 | padding]
        c = [0]
        for n in self.cols:
            c.append(c[-1] + n)
        q, k, v, g, a1 = (proj[:, c[i]:c[i + 1]] for i in range(5))
        if a1.data_ptr() % 16 or self.rank % 8:
            a1 = a1.contiguous()                                        # the tensor-core product wants aligned rows
        z = self.a2.forward(a1, out_dtype=torch.float32)                # the decay's logit, before its bias
        o = torch.empty((rows, H * dv), dtype=torch.float32, device=x.device)
        # in a long step every decay is read by many CTAs of the recurrence: computed once, in place; a short
        # step computes them where they are used and saves the launch
        ready = rows > self.DECAY_IN_PLACE_ROWS
        if ready:
            K.scan_decay(z, self.a2_bias, 1.0 / self.tau)
        K.linear_scan(q, k, v, z, self.a2_bias, o, state, 0, ctx, H, H, dk, dv, "channel",
                      q_scale=dk ** -0.5, inv_tau=1.0 / self.tau, gate_is_decay=ready)
        padded = ctx.rows > ctx.n_tokens
        y = torch.zeros((rows, H * dv), dtype=x.dtype, device=x.device) if padded else self.rt.empty(rows, H * dv)
        K.gated_norm(o, g, self.norm_w, y, ctx.token_seq, dv, False, self.eps, out_scale=self.out_mult)
        return self.o.forward(y, residual=residual, defer_to=ctx)
