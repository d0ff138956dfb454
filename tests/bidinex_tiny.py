"""Small Bidinex configurations of the tests' own (config.json dictionaries) and helpers to write model
folders whose weights make faults show: peaked attention, experts that matter, routers with spread scores.

BX_A: three unlike layers (head counts, sizes, rotated parts smaller than rot_dim, one layer without a
feed-forward), a loop that starts after the first layer and runs three times, a residual multiplier
that is no power of two.  BX_B: no loop, no cap, a width that is no multiple of 8 (the plain products
serve it), one head, top = all experts, one group kept of two.  BX_C: every layer inside the loop,
sizes in multiples of 16.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def _mixer(heads, dim, rot_dim, rot_dims, vdim, kv_rank, scale, base):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "rot": {"base": base, "dims": rot_dims}, "vdim": vdim,
            "kv_rank": kv_rank, "scale": scale}


def _moe(ff, experts, top, count=None, keep=None):
    router = {"experts": experts, "top": top}
    if count is not None:
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


BX_A: Dict = {
    "architecture": "Bidinex", "vocab": 311, "width": 96, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-6},
    "residual_mult": 0.7, "logit_softcap": 3.0,
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(3, 16, 8, 8, 24, 40, 0.2, 10000.0), "mlp": _moe(48, 6, 2, 3, 2)},
        {"type": "latent_attention", "mixer": _mixer(2, 24, 16, 8, 16, 64, 0.15, 500000.0), "mlp": None},
        {"type": "latent_attention", "mixer": _mixer(4, 8, 8, 4, 8, 24, 0.25, 100.0), "mlp": _moe(40, 5, 3, 5, 3)},
    ],
    "loop": {"start": 1, "stop": 3, "times": 3},
}

BX_B: Dict = {
    "architecture": "Bidinex", "vocab": 257, "width": 100, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
    "residual_mult": 1.0,
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(1, 32, 32, 32, 32, 16, 0.125, 1e6), "mlp": _moe(24, 4, 4, 2, 2)},
        {"type": "latent_attention", "mixer": _mixer(5, 8, 4, 4, 12, 48, 0.3, 50.0), "mlp": _moe(16, 8, 2, 2, 1)},
    ],
    "loop": None,
}

BX_C: Dict = {
    "architecture": "Bidinex", "vocab": 400, "width": 128, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-5},
    "residual_mult": 0.25, "logit_softcap": 10.0,
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(4, 32, 16, 16, 16, 64, 0.14, 10000.0), "mlp": _moe(64, 8, 2)},
        {"type": "latent_attention", "mixer": _mixer(8, 16, 16, 16, 32, 48, 0.2, 10000.0), "mlp": _moe(32, 4, 1, 4, 2)},
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}

BX_CONFIGS = {"A": BX_A, "B": BX_B, "C": BX_C}
BX_SEEDS = {"A": 11, "B": 5, "C": 23}

# factors on the drawn tensors (N(0, 0.02)), by the end of their names: streams of order one, peaked attention
GAINS = {"embed": 10.0, ".mix.q": 10.0, ".mix.dkv": 5.0, ".mix.uk": 5.0, ".mix.uv": 5.0, ".mix.o": 5.0, ".mix.g": 20.0,
         ".gate": 6.0, ".up": 6.0, ".down": 6.0, "loop.in": 4.0, ".b": 10.0, ".mlp.router": 20.0}


def shape_weights(tensors: Dict[str, torch.Tensor], cfg: Dict, seed: int) -> Dict[str, torch.Tensor]:
    """Scale the drawn tensors (GAINS).  A router's choice between two experts whose scores nearly tie can still
    fall the other way in a bfloat16 run: the bfloat16 tests allow for a few such positions, the float32 tests for none."""
    out = {}
    for n, t in tensors.items():
        f = next((v for k, v in GAINS.items() if n.endswith(k)), 1.0)
        out[n] = (t.float() * f).to(t.dtype)
    return out


def make_bidinex_folder(tmp_path, name: str, cfg: Dict = None, seed: int = None) -> str:
    """Write a model folder for configuration `name` (or `cfg`) with shaped random weights."""
    from braidinfer_b200.weights import open_model_folder, save_file, write_random_model
    cfg = dict(cfg if cfg is not None else BX_CONFIGS[name])
    seed = BX_SEEDS.get(name, 1) if seed is None else seed
    folder = os.path.join(str(tmp_path), f"bidinex_{name}")
    write_random_model(cfg, folder, seed)
    tensors = {n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    save_file(shape_weights(tensors, cfg, seed), os.path.join(folder, "model.safetensors"))
    return folder


def folder_config(folder: str) -> Dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)
