"""The Bidinex decoder as a description of parts.

token embedding * scale -> Dynamic Tanh -> runs of layers -> Dynamic Tanh -> tied output head -> soft cap.
A layer: h += m * latent_attention(dyt(h)); h += m * moe(dyt(h)) (the feed-forward may be absent); m is
the model's residual multiplier.  A block of layers may run several times in a row with the same weights
and a cache of its own per run; each pass starts with h <- W_in [h ; embedding output].  Tensor names:
`embed`, `embed.norm{,.b,.alpha}`, `loop.in`, `l<i>.norm1..`, `l<i>.norm2..`, `l<i>.mix.*`, `l<i>.mlp.*`,
`final.norm..`.
"""
from __future__ import annotations

from ..config.bidinex import BidinexConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import Architecture, register_architecture


def build_bidinex_spec(cfg: BidinexConfig) -> ModelSpec:
    def dyt(name: str) -> PartSpec:
        return PartSpec("dyt", {"width": cfg.width, "name": name})

    layers = []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        rope = PartSpec("rope", {"head_dim": m.rot_dim, "theta": m.rot_base, "rope_dim": m.rot_dims, "pairing": "half"})
        mixer = PartSpec("latent_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
            "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "window": None,
            "out_mult": cfg.residual_mult, "gated": True, "position_encoding": rope})
        ffn = ffn_norm = None
        if L.mlp is not None:
            f = L.mlp
            ffn = PartSpec("moe", {"hidden_size": cfg.width, "intermediate_size": f.ff, "experts": f.experts,
                                   "top": f.top, "groups": f.groups, "keep": f.keep, "out_mult": cfg.residual_mult})
            ffn_norm = dyt("norm2")
        layers.append(LayerSpec(block="prenorm_residual", prefix=f"l{i}.", mixer=mixer, mixer_norm=dyt("norm1"),
                                feed_forward=ffn, feed_forward_norm=ffn_norm))
    schedule = tuple(ScheduleEntry(layer, inject=first) for layer, first in cfg.schedule())
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed",
                                               "scale": cfg.embedding_scale, "norm": dyt("embed.norm")}),
        layers=tuple(layers), schedule=schedule,
        final_norm=dyt("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "head",
                                      "tied": True, "softcap": cfg.logit_softcap}),
        max_position=cfg.max_position, eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id,
        injection=PartSpec("concat_linear", {"width": cfg.width, "name": "loop.in"}) if cfg.loop is not None else None)


BIDINEX = register_architecture(Architecture(
    name="Bidinex", config_from_dict=BidinexConfig.from_dict, build_spec=build_bidinex_spec))
