"""Two mixers side by side: both read the same normed rows, and the layer's residual takes the weighted sum
of their results,  h <- h + a * left(x) + b * right(x).

The two are built from their own descriptions (any registered mixers: an attention beside a recurrence, for
one); each is handed its factor as its `out_mult` and adds its own result into the float32 stream.  At most one
of the two keeps keys and values (the cache manager gives a run one cache view); states lie one after the other
in the run's state area, and a child that shares the area is told where its part begins (`state_offset`).
"""
from __future__ import annotations

from typing import Dict, Optional

from .base import MIXERS, Mixer
from .spec import CacheRequest, PartSpec, TensorSpec


@MIXERS.register("parallel")
class ParallelMixers(Mixer):
    """params: left, right (PartSpecs of mixers that take `out_mult`; their tensor names lie under the layer's
    prefix like any mixer's), left_scale, right_scale (default 1)."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.children = []
        for side in ("left", "right"):
            spec: PartSpec = params[side]
            p = dict(spec.params)
            p["out_mult"] = float(p.get("out_mult", 1.0)) * float(params.get(side + "_scale", 1.0))
            self.children.append(MIXERS.get(spec.kind)(p, prefix, runtime))
        if sum(c.cache_request() is not None for c in self.children) > 1:
            raise ValueError("of two mixers side by side only one may keep keys and values")
        self.graph_safe = all(c.graph_safe for c in self.children)
        self.offsets = []
        at = 0
        for c in self.children:
            self.offsets.append(at)
            at += -(-int(c.state_bytes()) // 16) * 16        # every child's state starts on 16 bytes
        self._state_bytes = at

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d: Dict[str, TensorSpec] = {}
        for c in self.children:
            d.update(c.tensor_specs())
        return d

    def load(self, tensors) -> None:
        for c in self.children:
            c.load(tensors)

    def cache_request(self) -> Optional[CacheRequest]:
        for c in self.children:
            r = c.cache_request()
            if r is not None:
                return r
        return None

    def state_bytes(self) -> int:
        return self._state_bytes

    def forward(self, x, residual, ctx, cache, state):
        h = residual
        for c, off in zip(self.children, self.offsets):
            # a sum that the mixer before left deferred lives in the products' workspace: completed first
            h = ctx.resolve(h)
            own = None
            if c.state_bytes() > 0:
                own = state[:, off:off + int(c.state_bytes())]
            h = c.forward(x, h, ctx, cache if c.cache_request() is not None else None, own)
        return h
