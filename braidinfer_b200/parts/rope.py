"""Rotary position encoding, fused with the write of keys and values into the cache.

inv_freq[p] = theta^(-2p/rd) (reference: crates/braidinfer-runtime/src/weights.rs:743-751);
each pair (a, b) of a head becomes (a cos - b sin, a sin + b cos) with angle
pos * inv_freq[p] (kernels/megakernel_ops.hip:2019-2030).  The pair is (x[2p], x[2p+1])
for pairing "adjacent", as in that kernel, or (x[p], x[p + rd/2]) for "half".  Keys are
rotated once, before they are stored; attention never rotates a cached key again.
Angles, sine and cosine are float32.

`scaling` (optional) stretches the rotation for contexts beyond the length a model was trained at, pair by
pair (YaRN: Peng, Quesnelle, Fan, Shippole, "YaRN: Efficient Context Window Extension of Large Language
Models", 2023).  With f_p the plain frequency, d(t) = rd * ln(original / (2 pi t)) / (2 ln theta) the (real)
pair index that turns t times over the original length, lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)),
rd - 1) and ramp_p = clamp((p - lo) / max(hi - lo, 0.001), 0, 1):
    f'_p = f_p / factor * ramp_p + f_p * (1 - ramp_p),     amplitude = 0.1 ln(factor) + 1 on sine and cosine.
Fast pairs keep their frequency, slow pairs are divided by the factor, those between are blended.
"""
from __future__ import annotations

import torch

import math

from .base import POSITION_ENCODINGS, PositionEncoding


def rotary_frequencies(rope_dim: int, theta: float, scaling=None):
    """(inv_freq [rope_dim / 2] float64, amplitude) of a rotation, with the optional `scaling`
    {"factor", "original", "fast", "slow"} described in this module's head."""
    p = torch.arange(rope_dim // 2, dtype=torch.float64)
    inv = 1.0 / (theta ** (2.0 * p / rope_dim)) if rope_dim else p
    if not scaling:
        return inv, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    fast, slow = float(scaling["fast"]), float(scaling["slow"])
    if factor <= 0 or original <= 0 or fast <= 0 or slow <= 0:
        raise ValueError(f"rope scaling wants positive factor, original, fast and slow, got {dict(scaling)}")

    def pair_of(turns: float) -> float:
        return rope_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), rope_dim - 1)
    ramp = ((p - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return inv / factor * ramp + inv * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(PositionEncoding):
    """params: head_dim, theta, rope_dim (default head_dim), pairing ("half" | "adjacent"), scaling (None, or
    {"factor", "original", "fast", "slow"}: see the module's head)."""

    accepts_deferred = True      # adds a deferred q/k/v product in the same kernel as the rotation
    # ... in steps of up to this many rows.  That kernel runs a small CTA per row and head, which saves a
    # launch in a chain of few rows and loses to reduce kernel + rotation kernel beyond (8 layers of the 7B
    # sizes: 1.036 against 1.043 ms at 64 rows, 1.125 against 1.118 at 80, 1.56 against 1.42 at 256).
    FUSED_REDUCE_MAX_ROWS = 64

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.head_dim = int(params["head_dim"])
        self.rope_dim = int(params.get("rope_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.pairing = params.get("pairing", "half")
        if self.pairing not in ("half", "adjacent"):
            raise ValueError(f"rope pairing must be 'half' or 'adjacent', got {self.pairing!r}")
        if self.rope_dim % 2 or not (0 <= self.rope_dim <= self.head_dim):
            raise ValueError(f"rope_dim={self.rope_dim} must be even and within head_dim={self.head_dim}")
        inv, self.amplitude = rotary_frequencies(self.rope_dim, self.theta, params.get("scaling"))
        self.inv_freq = inv.to(torch.float32).to(runtime.device)

    def norm_encode_and_store(self, qk: torch.Tensor, nqh: int, nkh: int, ctx, cache, q_weight, k_weight, eps: float,
                              value_is_key: bool) -> None:
        """For mixers that norm their query and key heads: every head of qk [rows, (nqh + nkh (+ nkh)) * hd] is
        RMS-normed over the head (weights of head_dim numbers, shared by the heads; None: no norm), then rotated
        in place; keys go into `cache`, and so do the values: the value heads, or (`value_is_key`) the key heads as
        they came in, before norm and rotation.  One kernel."""
        ctx.resolve(qk)
        writable = cache is not None and not cache.read_only
        self.rt.kernels.head_norm_rope_kv(
            qk, q_weight, k_weight, self.inv_freq, ctx.positions, ctx.token_seq, cache.page_table if writable else None,
            cache.storage if writable else None, nqh, nkh, self.head_dim, self.rope_dim, self.pairing == "adjacent",
            value_is_key, cache.page_size if cache is not None else 1, eps, self.amplitude)

    def encode_and_store(self, qkv: torch.Tensor, nqh: int, nkh: int, ctx, cache) -> None:
        """Rotate the query and key heads of qkv [rows, (nqh + 2 nkh) * hd] in place and
        write keys and values into `cache` (a LayerCache, or None / read-only: no write)."""
        writable = cache is not None and not cache.read_only
        if self.amplitude != 1.0:
            # sine and cosine carry a factor: the kernel that also norms heads takes one (and no norm)
            ctx.resolve(qkv)
            self.rt.kernels.head_norm_rope_kv(
                qkv, None, None, self.inv_freq, ctx.positions, ctx.token_seq, cache.page_table if writable else None,
                cache.storage if writable else None, nqh, nkh, self.head_dim, self.rope_dim, self.pairing == "adjacent",
                False, cache.page_size if cache is not None else 1, 0.0, self.amplitude)
            return
        if qkv.shape[0] > self.FUSED_REDUCE_MAX_ROWS:
            ctx.resolve(qkv)
        d = ctx.take_deferred(qkv)
        if d is not None:
            handle, kind = d
            if kind != "store" or qkv.dtype != torch.bfloat16:
                raise RuntimeError("the rotary encoding can only complete a deferred bfloat16 product")
            self.rt.kernels.streamk_reduce_rope_kv(
                handle, qkv, self.inv_freq, ctx.positions, ctx.token_seq,
                cache.page_table if writable else None, cache.storage if writable else None,
                nqh, nkh, self.head_dim, self.rope_dim, self.pairing == "adjacent",
                cache.page_size if cache is not None else 1)
            return
        self.rt.kernels.rope_kv_write(
            qkv, self.inv_freq, ctx.positions, ctx.token_seq,
            cache.page_table if writable else None, cache.storage if writable else None,
            nqh, nkh, self.head_dim, self.rope_dim, self.pairing == "adjacent",
            cache.page_size if cache is not None else 1)


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(RotaryEncoding):
    """No position information in queries and keys: they pass through as the projections made
    them, and keys and values are stored.  (The rotation of zero elements: the same kernels.)
    params: head_dim."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__({"head_dim": params["head_dim"], "theta": 1.0, "rope_dim": 0}, prefix, runtime)
