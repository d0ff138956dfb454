"""Ways of feeding the embedding's output back into the stream.

"concat_linear": h <- W [h ; h0], W stored [width, 2 width] with the stream's columns first.  A model
whose block of layers runs several times in a row applies it at the start of every pass, so that each
pass sees both what the passes before made of the stream and the tokens themselves.  The two float32
streams are laid side by side in the run's element type and multiplied once; the result is the new
float32 stream.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import INJECTIONS, Injection
from .linear import Linear
from .spec import TensorSpec


@INJECTIONS.register("concat_linear")
class ConcatLinear(Injection):
    """params: width, name (tensor [width, 2 * width])."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.width = int(params["width"])
        self.linear = Linear(runtime, [prefix + params["name"]], [self.width], 2 * self.width)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return self.linear.tensor_specs()

    def load(self, tensors) -> None:
        self.linear.load(tensors)

    def forward(self, h: torch.Tensor, h0: torch.Tensor, ctx) -> torch.Tensor:
        both = self.rt.empty(h.shape[0], 2 * self.width)
        self.rt.kernels.concat2(h, h0, both)
        return self.linear.forward(both, out_dtype=torch.float32)
