"""The Loduzen decoder as a description of parts.

token embedding -> layers -> RMS norm -> the embedding table as the output head.
A layer: h += mixer(rmsnorm(h)); h += feed_forward(rmsnorm(h)) (the feed-forward may be absent); then the
layer's own token input, h += rmsnorm(Wproj(gelu(Wgate h) * side_table[token, layer's columns])) * w.
Mixers: "parallel" puts a windowed grouped-query attention (heads normed before an interleaved, partly and
YaRN-scaled rotation; values are the keys as projected; a sink in the softmax) beside a gated linear attention
and adds a_left * left + a_right * right; "mamba2" is a state-space layer.  The feed-forward is gated with the
tanh form of gelu.  Tensor names: `embed`, `side.embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`
(`.left.*`, `.right.*`), `l<i>.mlp.{gate,up,down}`, `l<i>.side.{gate,proj,norm}`, `final.norm`.
"""
from __future__ import annotations

from ..config.loduzen import LoduzenConfig, sizes_from_shapes
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import Architecture, register_architecture


def build_loduzen_spec(cfg: LoduzenConfig) -> ModelSpec:
    def rms(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.norm_eps, "name": name})

    layers = []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "parallel":
            a, r = m.left, m.right
            sc = a.rot_scaling
            rope = PartSpec("rope", {
                "head_dim": a.dim, "theta": a.rot_base, "rope_dim": a.rot_dims, "pairing": "adjacent",
                "scaling": None if sc is None else {"factor": sc.factor, "original": sc.original, "fast": sc.fast,
                                                     "slow": sc.slow}})
            left = PartSpec("gqa_attention", {
                "hidden_size": cfg.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
                "window": a.window, "position_encoding": rope, "q_proj": "mix.left.q", "k_proj": "mix.left.k",
                "o_proj": "mix.left.o", "value_from_key": True, "scale": a.scale, "sink": 0.0,
                "qk_norm": {"eps": cfg.norm_eps, "q_name": "mix.left.q.norm", "k_name": "mix.left.k.norm"}})
            right = PartSpec("gated_linear_attention", {
                "hidden_size": cfg.width, "num_heads": r.heads, "dim": r.dim, "vdim": r.vdim, "tau": r.tau,
                "gate_rank": r.gate_rank, "eps": cfg.norm_eps,
                **{n: "mix.right." + n for n in ("q", "k", "v", "g", "a1", "a2", "norm", "o")}, "a2_bias": "mix.right.a2.b"})
            mixer = PartSpec("parallel", {"left": left, "right": right, "left_scale": m.left_scale,
                                          "right_scale": m.right_scale})
        else:
            mixer = PartSpec("mamba2", {"hidden_size": cfg.width, "num_heads": m.heads, "vdim": m.vdim, "state": m.state,
                                        "groups": m.groups, "taps": m.conv, "norm_groups": m.norm_groups,
                                        "eps": cfg.norm_eps})
        ffn = ffn_norm = None
        if L.ff is not None:
            ffn = PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": L.ff, "activation": "gelu_tanh",
                                      "gate_proj": "mlp.gate", "up_proj": "mlp.up", "down_proj": "mlp.down"})
            ffn_norm = rms("norm2")
        side = None
        if cfg.side_dim:
            side = PartSpec("gated_token_table", {
                "vocab_size": cfg.vocab, "hidden_size": cfg.width, "dim": cfg.side_dim, "index": i,
                "columns": cfg.side_dim * len(cfg.layers), "eps": cfg.norm_eps, "activation": "gelu_tanh",
                "table": "side.embed"})
        layers.append(LayerSpec(block="prenorm_residual", prefix=f"l{i}.", mixer=mixer, mixer_norm=rms("norm1"),
                                feed_forward=ffn, feed_forward_norm=ffn_norm, layer_input=side))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=rms("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "head", "tied": True}),
        max_position=cfg.max_position, eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id)


LODUZEN = register_architecture(Architecture(
    name="Loduzen", config_from_dict=LoduzenConfig.from_dict, build_spec=build_loduzen_spec,
    sizes_from_shapes=sizes_from_shapes))
