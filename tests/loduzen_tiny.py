"""Small Loduzen configurations of the tests' own (config.json dictionaries) and helpers to write model folders
whose weights make faults show: streams of order one, peaked attention, decays close to one so that a token
far back still counts in a state.

LZ_A: attention beside linear attention, a state-space layer, attention again without a feed-forward; two unlike
windows (one shorter than a page, one longer); head sizes in multiples of 16; a side table.
LZ_B: a width that is no multiple of 8 (the plain products serve it), a state-space layer first, one attention head
of a size the tensor-core attention does not take, no scaling of the rotation, a window longer than any test
sequence, one norm group, one group of state-space heads, a convolution of two taps, a side table of 12 columns.
LZ_C: state-space layers only (no cache of keys at all), a convolution of one tap and one of five, no side table.
LZ_D: attention layers only, rotation of the whole head, kv_heads = heads, tau = 1, a window of 1 (a token sees
itself and the sink), no side table.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def _left(heads, kv, dim, window, base, dims, scale, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": window}, "rot": rot}


def _par(left, right, ls, rs):
    return {"left": left, "right": dict(zip(("heads", "dim", "vdim", "tau"), right)), "left_scale": ls, "right_scale": rs}


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


LZ_A: Dict = {
    "architecture": "Loduzen", "vocab": 311, "width": 96, "norm": {"eps": 1e-6}, "token_side": {"dim": 8},
    "layers": [
        {"type": "parallel", "mixer": _par(_left(4, 2, 32, 7, 10000.0, 16, 0.3, (4.0, 64, 16.0, 2.0)), (2, 24, 40, 8.0), 1.3, 0.6),
         "mlp": {"kind": "dense", "ff": 136}},
        {"type": "mamba2", "mixer": _ssm(4, 24, 16, 2, 4, 2), "mlp": {"kind": "dense", "ff": 72}},
        {"type": "parallel", "mixer": _par(_left(2, 1, 16, 70, 100.0, 8, 0.5, (1.5, 32, 8.0, 1.0)), (3, 16, 16, 32.0), 0.8, 1.1),
         "mlp": None},
    ],
}

LZ_B: Dict = {
    "architecture": "Loduzen", "vocab": 257, "width": 100, "norm": {"eps": 1e-5}, "token_side": {"dim": 12},
    "layers": [
        {"type": "mamba2", "mixer": _ssm(3, 20, 24, 1, 2, 1), "mlp": {"kind": "dense", "ff": 60}},
        {"type": "parallel", "mixer": _par(_left(1, 1, 40, 1000, 250000.0, 20, 0.2), (5, 12, 20, 2.0), 1.0, 1.0),
         "mlp": {"kind": "dense", "ff": 44}},
    ],
}

LZ_C: Dict = {
    "architecture": "Loduzen", "vocab": 128, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mamba2", "mixer": _ssm(2, 32, 8, 2, 1, 4), "mlp": None},
        {"type": "mamba2", "mixer": _ssm(8, 8, 72, 4, 5, 1), "mlp": {"kind": "dense", "ff": 96}},
    ],
}

LZ_D: Dict = {
    "architecture": "Loduzen", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "parallel", "mixer": _par(_left(2, 2, 64, 130, 10000.0, 64, 0.125, (8.0, 16, 4.0, 1.0)), (1, 136, 48, 1.0), 1.0, 1.0),
         "mlp": {"kind": "dense", "ff": 64}},
        {"type": "parallel", "mixer": _par(_left(8, 2, 16, 1, 50.0, 4, 1.0), (4, 8, 8, 4.0), 2.0, 0.25),
         "mlp": {"kind": "dense", "ff": 64}},
    ],
}

LZ_CONFIGS = {"A": LZ_A, "B": LZ_B, "C": LZ_C, "D": LZ_D}
LZ_SEEDS = {"A": 3, "B": 17, "C": 29, "D": 41}

# factors on the drawn tensors, by the end of their names
GAINS = {"embed": 40.0, "side.embed": 1.0, ".left.q": 12.0, ".left.k": 12.0, ".left.o": 6.0, ".right.q": 10.0, ".right.k": 10.0,
         ".right.v": 10.0, ".right.g": 20.0, ".right.o": 6.0, ".right.a1": 10.0, ".right.a2": 10.0, ".mix.in": 10.0, ".mix.o": 6.0,
         ".mlp.gate": 8.0, ".mlp.up": 8.0, ".mlp.down": 8.0, ".side.gate": 10.0, ".side.proj": 10.0}


def shape_weights(tensors: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for n, t in tensors.items():
        f = next((v for k, v in GAINS.items() if n.endswith(k)), 1.0)
        x = t.float() * f
        if n.endswith(".a2.b"):
            x = x + 3.0                    # decays near one: a state remembers hundreds of tokens
        if n.endswith(".A_log"):
            x = x - 2.0                    # slow state-space heads beside fast ones
        out[n] = x.to(t.dtype)
    return out


def make_loduzen_folder(tmp_path, name: str, cfg: Dict = None, seed: int = None) -> str:
    """Write a model folder for configuration `name` (or `cfg`) with shaped random weights."""
    from braidinfer_b200.weights import open_model_folder, save_file, write_random_model
    cfg = dict(cfg if cfg is not None else LZ_CONFIGS[name])
    seed = LZ_SEEDS.get(name, 1) if seed is None else seed
    folder = os.path.join(str(tmp_path), f"loduzen_{name}")
    write_random_model(cfg, folder, seed)
    tensors = {n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    save_file(shape_weights(tensors), os.path.join(folder, "model.safetensors"))
    return folder


def random_config(seed: int) -> Dict:
    """A configuration drawn from a seed: sizes, head counts, the order and number of layers, windows and constants
    all vary, within what a test can afford."""
    import random
    r = random.Random(seed)

    def divisor(n):
        return r.choice([d for d in range(1, n + 1) if n % d == 0])

    layers = []
    for _ in range(r.randint(2, 5)):
        mlp = {"kind": "dense", "ff": r.choice([24, 40, 56, 72, 100])} if r.random() < 0.8 else None
        if r.random() < 0.6:
            heads = r.choice([1, 2, 3, 4, 6, 8])
            dim = r.choice([8, 16, 24, 32, 48, 64, 80, 128])
            dims = 2 * r.randint(0, dim // 2)
            scaling = (r.choice([1.5, 2.0, 4.0, 8.0]), r.choice([16, 32, 64, 256]), r.choice([8.0, 16.0, 32.0]), r.choice([1.0, 2.0])) \
                if r.random() < 0.7 else None
            left = _left(heads, divisor(heads), dim, r.choice([1, 2, 5, 17, 33, 64, 65, 100, 500]), r.choice([100.0, 1e4, 1e6]), dims,
                         r.choice([dim ** -0.5, 0.2, 0.07]), scaling)
            right = (r.randint(1, 5), r.choice([4, 8, 12, 20, 32, 40, 72]), r.choice([4, 8, 12, 24, 36, 48]), r.choice([1.0, 2.0, 8.0, 32.0]))
            layers.append({"type": "parallel", "mixer": _par(left, right, r.choice([0.5, 1.0, 1.3]), r.choice([0.7, 1.0, 1.6])), "mlp": mlp})
        else:
            heads, vdim = r.choice([1, 2, 4, 6, 8]), r.choice([4, 8, 12, 16, 24, 40])
            layers.append({"type": "mamba2", "mixer": _ssm(heads, vdim, r.choice([4, 8, 16, 24, 48, 64, 80]), divisor(heads), r.randint(1, 5),
                                                            divisor(heads * vdim) if r.random() < 0.5 else divisor(heads)), "mlp": mlp})
    cfg = {"architecture": "Loduzen", "vocab": r.randint(90, 400), "width": r.choice([40, 48, 64, 72, 96, 100]),
           "norm": {"eps": r.choice([1e-6, 1e-5])}, "layers": layers}
    if r.random() < 0.7:
        cfg["token_side"] = {"dim": r.choice([4, 8, 12, 16, 24])}
    return cfg


def folder_config(folder: str) -> Dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)
