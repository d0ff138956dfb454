"""A layer's own token input: besides the stream, a layer may read a few numbers of its own about each token
from a table, gate them by the stream and add the result.

With e = table[token, index * dim : (index + 1) * dim] (every layer has its own columns of one table):
    g = act(Wgate h) * e,    y = Wproj g,    h <- h + y / sqrt(mean(y^2) + eps) * w
h is the float32 stream as the layer's other parts left it; the norm is an RMS norm with a plain weight.
Two small products, one kernel for the gate (activation, gather, product) and one for norm and sum.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import LAYER_INPUTS, LayerInput
from .linear import Linear
from .spec import TensorSpec


@LAYER_INPUTS.register("gated_token_table")
class GatedTokenTable(LayerInput):
    """params: vocab_size, hidden_size, dim, index (which block of `dim` columns of the table is this layer's),
    columns (the table's width: dim times the number of layers that read it), eps, activation (default
    "gelu_tanh"), table (the table's tensor name, NOT under the layer's prefix), and the names gate, proj, norm
    (under the prefix)."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.vocab = int(p["vocab_size"])
        self.hidden = int(p["hidden_size"])
        self.dim = int(p["dim"])
        self.index = int(p["index"])
        self.columns = int(p["columns"])
        self.eps = float(p["eps"])
        self.activation = p.get("activation", "gelu_tanh")
        from ..csrc.api import activation_code
        activation_code(self.activation)
        if (self.index + 1) * self.dim > self.columns:
            raise ValueError(f"gated_token_table: block {self.index} of {self.dim} columns lies outside the table's {self.columns}")
        self.table_name = p.get("table", "side.embed")
        self.gate = Linear(runtime, [prefix + p.get("gate", "side.gate")], [self.dim], self.hidden)
        self.proj = Linear(runtime, [prefix + p.get("proj", "side.proj")], [self.hidden], self.dim)
        self.norm_name = prefix + p.get("norm", "side.norm")
        self.table = self.norm_w = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = {self.table_name: TensorSpec((self.vocab, self.columns), std=1.0)}
        d.update(self.gate.tensor_specs())
        d.update(self.proj.tensor_specs())
        d[self.norm_name] = TensorSpec((self.hidden,), init="one_plus_normal")
        return d

    def load(self, tensors) -> None:
        self.table, self.norm_w = tensors[self.table_name], tensors[self.norm_name]
        self.gate.load(tensors)
        self.proj.load(tensors)

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        K = self.rt.kernels
        rows = h.shape[0]
        x = h
        if not self.rt.is_f32:
            x = self.rt.empty(rows, self.hidden)
            K.cast(h, x)
        gate = self.gate.forward(x)
        g = self.rt.empty(rows, self.dim)
        K.act_mul_gather(gate, self.table, ctx.token_ids, self.index * self.dim, g, self.activation)
        y = self.proj.forward(g, out_dtype=torch.float32)
        K.rmsnorm_add(h, y, self.norm_w, self.eps)
        return h
