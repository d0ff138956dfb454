"""Mamba-2: a state-space layer in its state-space-duality form (Dao, Gu: "Transformers are SSMs: Generalized
Models and Efficient Algorithms Through Structured State Space Duality", 2024).

For the mixer's input x (a row per token), with H heads of value size P, state size N and G groups:
    [z | u | B | C | d] = Win x              z, u: H P numbers; B, C: G N each; d: H
    [u | B | C] <- silu(conv(.) + bias)      a causal convolution per channel over the last `taps` tokens
    dt = softplus(d + dt_bias)               (no clamp)
    per head h, with its group's B and C:    S <- exp(-exp(A_log_h) dt) S + dt B u_h^T      (S is [N, P])
                                             y_h = S^T C + D_h u_h
    y <- y * silu(z), RMS-normed in `norm_groups` equal parts (each by its own root mean square), times w
    out = Wo y
The state of a sequence is S (float32) and the convolution's last taps - 1 inputs; both lie in its slot of the
state area, zero at the start, and are carried from step to step.  dt, the decay, the recurrence and the norm
are float32.  Per step: the stacked product, the convolution (and the move of its state), the recurrence
kernel (which computes dt and the decay where it uses them), the gated norm, the output product with the
residual sum in its epilogue.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import MIXERS, Mixer
from .linear import Linear
from .spec import TensorSpec


@MIXERS.register("mamba2")
class Mamba2(Mixer):
    """params: hidden_size, num_heads, vdim (P), state (N), groups (G), taps (of the convolution), norm_groups, eps,
    out_mult (default 1), and the tensor names in, conv, conv_bias, dt_bias, A_log, D, norm, o (under the prefix)."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.P = int(p["vdim"])
        self.N = int(p["state"])
        self.G = int(p["groups"])
        self.taps = int(p["taps"])
        self.norm_groups = int(p["norm_groups"])
        self.eps = float(p["eps"])
        self.out_mult = float(p.get("out_mult", 1.0))
        self.inner = self.heads * self.P
        if self.heads % self.G:
            raise ValueError(f"mamba2: {self.heads} heads do not divide into {self.G} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.inner} inner channels do not divide into {self.norm_groups} norm groups")
        if self.taps < 1:
            raise ValueError(f"mamba2: the convolution needs at least one tap, got {self.taps}")
        if self.N > 256:
            raise ValueError(f"mamba2: state sizes up to 256 are built, not {self.N}")
        self.channels = self.inner + 2 * self.G * self.N
        self.total = 2 * self.inner + 2 * self.G * self.N + self.heads
        name = lambda key, default: prefix + p.get(key, default)      # noqa: E731
        self.win = Linear(runtime, [name("in", "mix.in")], [self.total], self.hidden)
        self.o = Linear(runtime, [name("o", "mix.o")], [self.hidden], self.inner)
        self.names = {"conv": name("conv", "mix.conv"), "conv_bias": name("conv_bias", "mix.conv.b"),
                      "dt_bias": name("dt_bias", "mix.dt_bias"), "A_log": name("A_log", "mix.A_log"),
                      "D": name("D", "mix.D"), "norm": name("norm", "mix.norm")}
        self.t: Dict[str, torch.Tensor] = {}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.win.tensor_specs())
        n = self.names
        d[n["conv"]] = TensorSpec((self.channels, self.taps), std=0.3)
        d[n["conv_bias"]] = TensorSpec((self.channels,), std=0.1)
        d[n["dt_bias"]] = TensorSpec((self.heads,), std=1.0)
        d[n["A_log"]] = TensorSpec((self.heads,), std=0.5)
        d[n["D"]] = TensorSpec((self.heads,), init="one_plus_normal", std=0.2)
        d[n["norm"]] = TensorSpec((self.inner,), init="one_plus_normal")
        d.update(self.o.tensor_specs())
        return d

    def load(self, tensors) -> None:
        self.win.load(tensors)
        w = self.win.weight
        pad = -w.shape[0] % 8            # rows of zeros, so that a row of the result starts on 16 bytes
        if pad:
            self.win.weight = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)]).contiguous()
        self.o.load(tensors)
        self.t = {k: tensors[v].contiguous() for k, v in self.names.items()}

    def conv_state_bytes(self) -> int:
        return (self.taps - 1) * self.channels * 4

    def state_bytes(self) -> int:
        return self.conv_state_bytes() + self.heads * self.N * self.P * 4

    def forward(self, x, residual, ctx, cache, state):
        if state is None:
            raise RuntimeError("mamba2 needs its state area")
        K = self.rt.kernels
        rows = x.shape[0]
        H, P, N, G, inner = self.heads, self.P, self.N, self.G, self.inner
        proj = self.win.forward(x)                                      # [rows, z | u | B | C | d | padding]
        z = proj[:, :inner]
        d = proj[:, inner + self.channels:inner + self.channels + H]
        padded = ctx.rows > ctx.n_tokens
        make = torch.zeros if padded else torch.empty
        ubc = make((rows, self.channels), dtype=x.dtype, device=x.device)
        K.causal_conv(proj[:, inner:inner + self.channels], ubc, self.t["conv"], self.t["conv_bias"], state, 0, ctx, silu=True)
        u, B, C = ubc[:, :inner], ubc[:, inner:inner + G * N], ubc[:, inner + G * N:]
        y = make((rows, inner), dtype=torch.float32, device=x.device)
        K.linear_scan(C, B, u, d, self.t["dt_bias"], y, state, self.conv_state_bytes(), ctx, H, G, N, P, "head",
                      a_log=self.t["A_log"], skip=self.t["D"])
        out = make((rows, inner), dtype=x.dtype, device=x.device)
        K.gated_norm(y, z, self.t["norm"], out, ctx.token_seq, inner // self.norm_groups, True, self.eps,
                     out_scale=self.out_mult)
        return self.o.forward(out, residual=residual, defer_to=ctx)
