"""Loduzen without a GPU: configuration, recipe, cache plan, and the plain implementation's mechanisms by hand."""
import copy
import math

import pytest
import torch

import plain_loduzen as P
from loduzen_tiny import LZ_A, LZ_B, LZ_C, LZ_CONFIGS, LZ_D
from braidinfer_b200.config import ConfigError, LoduzenConfig
from braidinfer_b200.models import architecture_for, complete_config
from braidinfer_b200.parts.rope import rotary_frequencies
from braidinfer_b200.weights import tensor_specs_of

D = torch.float64


def spec_of(cfg):
    arch = architecture_for(cfg)
    return arch.build_spec(arch.config_from_dict(cfg))


def test_architecture_is_found_by_its_name_and_every_configuration_is_read():
    for cfg in LZ_CONFIGS.values():
        assert architecture_for(cfg).name == "Loduzen"
        c = LoduzenConfig.from_dict(cfg)
        assert c.vocab == cfg["vocab"] and len(c.layers) == len(cfg["layers"])
    c = LoduzenConfig.from_dict(LZ_A)
    assert c.side_dim == 8 and c.layers[0].mixer.left.window == 7 and c.layers[2].ff is None
    assert c.layers[1].mixer.conv == 4 and c.layers[0].mixer.right.tau == 8.0 and c.layers[0].mixer.left_scale == 1.3
    assert LoduzenConfig.from_dict(LZ_C).side_dim == 0


@pytest.mark.parametrize("path, value", [("layers.0.type", "conv"), ("layers.0.mixer.left.vdim", 16), ("layers.0.mixer.left.kv_heads", 3),
                                         ("layers.0.mixer.left.rot.dims", 34), ("layers.0.mixer.right.tau", 0.0),
                                         ("layers.1.mixer.groups", 3), ("layers.1.mixer.norm_groups", 5), ("layers.0.mlp.kind", "moe"),
                                         ("norm", None), ("layers.0.mixer.left.scale", None), ("layers.1.mixer.state", None)])
def test_a_value_nothing_computes_is_an_error_that_names_its_key(path, value):
    cfg = copy.deepcopy(LZ_A)
    cur = cfg
    keys = path.split(".")
    for k in keys[:-1]:
        cur = cur[int(k)] if k.isdigit() else cur[k]
    if value is None:
        del cur[keys[-1]]
    else:
        cur[keys[-1]] = value
    with pytest.raises(ConfigError) as e:
        LoduzenConfig.from_dict(cfg)
    assert keys[-1] in str(e.value) or keys[-2] in str(e.value)


def test_recipe_names_the_tensors_of_the_design_and_the_parts_beside_the_existing_ones():
    spec = spec_of(LZ_A)
    names = set(tensor_specs_of(spec))
    for n in ("embed", "side.embed", "final.norm", "l0.norm1", "l0.mix.left.q", "l0.mix.left.k", "l0.mix.left.q.norm",
              "l0.mix.left.k.norm", "l0.mix.left.o", "l0.mix.right.a1", "l0.mix.right.a2", "l0.mix.right.a2.b", "l0.mix.right.norm",
              "l1.mix.in", "l1.mix.conv", "l1.mix.conv.b", "l1.mix.dt_bias", "l1.mix.A_log", "l1.mix.D", "l1.mix.norm", "l1.mix.o",
              "l0.mlp.gate", "l2.side.gate", "l2.side.proj", "l2.side.norm"):
        assert n in names, n
    assert not any(n.startswith("l2.mlp") or n.startswith("l2.norm2") or ".left.v" in n for n in names)
    specs = tensor_specs_of(spec)
    assert specs["side.embed"].shape == (311, 24) and specs["l1.mix.in"].shape == (2 * 96 + 2 * 2 * 16 + 4, 96)
    assert specs["l1.mix.conv"].shape == (96 + 64, 4) and specs["l0.mix.right.a2"].shape == (48, 32)
    assert [l.mixer.kind for l in spec.layers] == ["parallel", "mamba2", "parallel"]
    assert spec.layers[0].mixer.params["left"].kind == "gqa_attention" and spec.layers[0].layer_input.kind == "gated_token_table"
    assert spec_of(LZ_C).layers[0].layer_input is None


def test_a_size_that_only_a_tensor_shape_gives_is_taken_from_the_shapes():
    shapes = {"l0.mix.right.a1": (24, 96), "l2.mix.right.a1": (8, 96)}
    full = complete_config(LZ_A, shapes)
    c = LoduzenConfig.from_dict(full)
    assert c.layers[0].mixer.right.gate_rank == 24 and c.layers[2].mixer.right.gate_rank == 8
    assert "gate_rank" not in LZ_A["layers"][0]["mixer"]["right"]            # the caller's dictionary is left alone
    assert tensor_specs_of(spec_of(full))["l0.mix.right.a2"].shape == (48, 24)


def test_cache_plan_one_window_group_per_window_and_state_for_every_recurrence():
    from braidinfer_b200.models import DecoderModel
    from braidinfer_b200.parts import Runtime
    model = DecoderModel(spec_of(LZ_A), Runtime(torch.float32, torch.device("cpu"), None))
    plan = model.cache_plan()
    assert [(r.kind, r.num_kv_heads, r.head_dim, r.window, r.planes) if r else None for r, _, _ in plan] == \
        [("window", 2, 32, 7, 2), None, ("window", 1, 16, 70, 2)]
    assert plan[0][2] == 2 * 24 * 40 * 4 and plan[2][2] == 3 * 16 * 16 * 4
    assert plan[1][2] == (3 * (96 + 64) + 4 * 16 * 24) * 4
    plan_c = DecoderModel(spec_of(LZ_C), Runtime(torch.float32, torch.device("cpu"), None)).cache_plan()
    assert all(r is None for r, _, _ in plan_c) and plan_c[0][2] == 2 * 8 * 32 * 4      # one tap: no inputs kept


def test_scaled_rotation_frequencies_by_hand_and_against_the_plain_table():
    # 8 numbers a head, base 100: plain frequencies 1, 100^-1/4, 100^-1/2, 100^-3/4
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 1.5, "original": 32, "fast": 8.0, "slow": 1.0}}
    f, amp = rotary_frequencies(8, 100.0, rot["scaling"])
    plain = torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=D)
    pair = lambda t: 8 * math.log(32 / (2 * math.pi * t)) / (2 * math.log(100.0))      # noqa: E731
    lo, hi = max(math.floor(pair(8.0)), 0), min(math.ceil(pair(1.0)), 7)
    assert (lo, hi) == (0, 2)
    ramp = torch.tensor([0.0, 0.5, 1.0, 1.0], dtype=D)
    assert torch.allclose(f, plain / 1.5 * ramp + plain * (1 - ramp), rtol=1e-14)
    assert amp == pytest.approx(0.1 * math.log(1.5) + 1)
    for cfg in (LZ_A, LZ_D):
        for L in cfg["layers"]:
            if L["type"] == "parallel":
                r = L["mixer"]["left"]["rot"]
                f1, a1 = rotary_frequencies(r["dims"], r["base"], r.get("scaling"))
                f2, a2 = P.rotation_table(r)
                assert torch.allclose(f1, f2, rtol=1e-14) and a1 == pytest.approx(a2)
    f0, a0 = rotary_frequencies(8, 100.0, None)
    assert torch.allclose(f0, plain) and a0 == 1.0


def test_plain_rotation_turns_neighbours_and_scores_depend_on_distance_only():
    rot = {"base": 50.0, "dims": 4}
    x = torch.arange(12, dtype=D).view(1, 2, 6) + 1
    y = P.rotate_pairs(x, torch.tensor([3]), rot)
    a = 3 * 1.0
    assert y[0, 0, 0].item() == pytest.approx(1 * math.cos(a) - 2 * math.sin(a)) and y[0, 0, 1].item() == pytest.approx(2 * math.cos(a) + 1 * math.sin(a))
    assert torch.equal(y[..., 4:], x[..., 4:])                             # beyond rot.dims nothing turns
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 6, generator=g, dtype=D), torch.randn(1, 1, 6, generator=g, dtype=D)
    s = [(P.rotate_pairs(q, torch.tensor([p + 5]), rot) * P.rotate_pairs(k, torch.tensor([p]), rot)).sum().item() for p in (0, 9, 40)]
    assert s[0] == pytest.approx(s[1]) and s[0] == pytest.approx(s[2])


def test_plain_sink_softmax_leaves_weight_for_nothing():
    s = torch.tensor([[0.0, 0.0, 5.0]], dtype=D)
    vis = torch.tensor([[True, True, False]])
    p = P.sink_softmax(s, vis)
    assert torch.allclose(p, torch.tensor([[1 / 3, 1 / 3, 0.0]], dtype=D))
    big = P.sink_softmax(torch.tensor([[800.0]], dtype=D), torch.tensor([[True]]))
    assert big.item() == pytest.approx(1.0)
    small = P.sink_softmax(torch.tensor([[-800.0]], dtype=D), torch.tensor([[True]]))
    assert small.item() == 0.0 or small.item() < 1e-300


def test_plain_recurrences_by_hand():
    # one head, key size 1, value size 1: S_t = a S_(t-1) + k v, o = S q
    w = {"q": torch.tensor([[2.0]], dtype=D), "k": torch.tensor([[1.0]], dtype=D), "v": torch.tensor([[3.0]], dtype=D),
         "g": torch.tensor([[0.0]], dtype=D), "a1": torch.tensor([[0.0]], dtype=D), "a2": torch.tensor([[0.0]], dtype=D),
         "a2.b": torch.tensor([0.0], dtype=D), "norm": torch.tensor([1.0], dtype=D), "o": torch.tensor([[1.0]], dtype=D)}
    h = torch.tensor([[1.0], [1.0], [1.0]], dtype=D)
    out = P.gated_linear_attention(h, w, "", {"heads": 1, "dim": 1, "vdim": 1, "tau": 1.0}, 0.0)
    # decay 1/2: S = 3, 4.5, 5.25; o = 2 S > 0, its unit norm is 1, the gate silu(0) = 0
    assert torch.equal(out, torch.zeros(3, 1, dtype=D))
    w["g"] = torch.tensor([[1.0]], dtype=D)
    out = P.gated_linear_attention(h, w, "", {"heads": 1, "dim": 1, "vdim": 1, "tau": 1.0}, 0.0)
    assert torch.allclose(out, torch.full((3, 1), 1 / (1 + math.exp(-1.0)), dtype=D))
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=D)
    y = P.causal_conv(x, torch.tensor([[10.0, 1.0]], dtype=D), torch.tensor([0.5], dtype=D))
    assert y.view(-1).tolist() == [1.5, 12.5, 24.5]
