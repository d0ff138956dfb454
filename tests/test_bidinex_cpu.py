"""Bidinex on the CPU: the configuration reader, the recipe (parts, tensor names, schedule, cache plan),
and hand-worked checks of the plain implementation that the GPU tests compare with."""
import copy
import math

import pytest
import torch

import plain_bidinex as P
from bidinex_tiny import BX_A, BX_B, BX_C, make_bidinex_folder
from braidinfer_b200.config import BidinexConfig, ConfigError
from braidinfer_b200.models import architecture_for
from braidinfer_b200.weights import tensor_specs_of


def spec_of(cfg):
    arch = architecture_for(cfg)
    return arch.build_spec(arch.config_from_dict(cfg))


def test_architecture_is_found_by_its_name_and_sizes_come_from_the_dictionary():
    assert architecture_for(BX_A).name == "Bidinex"
    c = BidinexConfig.from_dict(BX_A)
    assert (c.vocab, c.width, c.embedding_scale, c.norm_eps, c.residual_mult, c.logit_softcap) == (311, 96, 2.5, 1e-6, 0.7, 3.0)
    assert [l.mixer.heads for l in c.layers] == [3, 2, 4] and c.layers[1].mlp is None
    assert (c.layers[0].mixer.rot_dim, c.layers[1].mixer.rot_dims, c.layers[2].mlp.groups, c.layers[2].mlp.keep) == (8, 8, 5, 3)
    b = BidinexConfig.from_dict(BX_B)
    assert b.loop is None and b.logit_softcap is None and b.layers[0].mlp.top == 4
    no_groups = BidinexConfig.from_dict(BX_C).layers[0].mlp
    assert (no_groups.groups, no_groups.keep) == (1, 1)


def test_schedule_runs_the_looped_block_in_a_row_and_marks_the_start_of_every_pass():
    c = BidinexConfig.from_dict(BX_A)
    assert c.schedule() == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False)]
    assert BidinexConfig.from_dict(BX_B).schedule() == [(0, False), (1, False)]
    assert BidinexConfig.from_dict(BX_C).schedule() == [(0, True), (1, False), (0, True), (1, False)]
    assert P.layer_runs(BX_A) == c.schedule() and P.layer_runs(BX_C) == BidinexConfig.from_dict(BX_C).schedule()
    once = copy.deepcopy(BX_A)
    once["loop"] = {"start": 0, "stop": 1, "times": 1}
    assert BidinexConfig.from_dict(once).schedule() == [(0, True), (1, False), (2, False)]


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "ring_attention", "type"), (("layers", 0, "mixer", "rot", "dims"), 6, "rot.dims"),
    (("layers", 2, "mlp", "router", "top"), 4, "top"), (("layers", 0, "mlp", "kind"), "dense", "kind"),
    (("loop",), {"start": 2, "stop": 1, "times": 2}, "loop"), (("vocab",), None, "vocab"),
    (("layers", 1, "mixer", "kv_rank"), 0, "kv_rank"), (("logit_softcap",), -1.0, "logit_softcap"),
    (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups")])
def test_a_value_that_nothing_computes_is_refused_with_its_key(path, value, word):
    d = copy.deepcopy(BX_A)
    cur = d
    for k in path[:-1]:
        cur = cur[k]
    cur[path[-1]] = value
    if path == ("layers", 0, "mixer", "rot", "dims"):
        cur[path[-1]] = 10                       # more than rot_dim
    with pytest.raises(ConfigError, match=word):
        BidinexConfig.from_dict(d)


def test_recipe_names_the_stored_tensors_and_asks_for_one_plane_of_cache_per_run():
    from braidinfer_b200.models import DecoderModel
    from braidinfer_b200.parts import Runtime
    spec = spec_of(BX_A)
    names = tensor_specs_of(spec)
    for n, shape in {"embed": (311, 96), "embed.norm.alpha": (), "loop.in": (96, 192), "l0.mix.q": (3 * 24, 96),
                     "l0.mix.dkv": (48, 96), "l0.mix.dkv.norm": (40,), "l0.mix.uk": (48, 40), "l0.mix.uv": (72, 40),
                     "l0.mix.g": (3, 96), "l0.mix.o": (96, 72), "l0.mlp.router": (6, 96), "l0.mlp.e5.gate": (48, 96),
                     "l2.mlp.e4.down": (96, 40), "l1.norm1.b": (96,), "final.norm": (96,)}.items():
        assert tuple(names[n].shape) == shape, n
    assert not any(n.startswith("l1.mlp") or n.startswith("l1.norm2") for n in names) and "head" not in names
    assert "loop.in" not in tensor_specs_of(spec_of(BX_B))
    model = DecoderModel(spec, Runtime(act_dtype=torch.bfloat16, device=torch.device("cpu"), kernels=None))
    plan = model.cache_plan()
    assert len(plan) == 7 and all(co is None and sb == 0 for _, co, sb in plan)       # every run keeps its own
    req = [r for r, _, _ in plan]
    assert (req[0].planes, req[0].num_kv_heads, req[0].head_dim, req[0].kind) == (1, 1, 48, "full")
    assert req[1] == req[3] == req[5] and req[1].head_dim == 80 and req[2].head_dim == 32


def test_random_model_folder_round_trip_and_cache_groups(tmp_path):
    from braidinfer_b200.cache import CacheManager
    from braidinfer_b200.models import DecoderModel
    from braidinfer_b200.parts import Runtime
    from tiny import read_weights
    folder = make_bidinex_folder(tmp_path, "A")
    w = read_weights(folder)
    assert set(w) == set(tensor_specs_of(spec_of(BX_A)))
    lg = P.forward(w, BX_A, [5, 9, 200, 17])
    assert lg.shape == (4, 311) and torch.isfinite(lg).all() and lg.abs().max() <= 3.0
    model = DecoderModel(spec_of(BX_A), Runtime(act_dtype=torch.bfloat16, device=torch.device("cpu"), kernels=None))
    cache = CacheManager(model.cache_plan(), 256, 4, torch.bfloat16, "cpu")
    assert sorted(tuple(g.storage.shape) for g in cache.groups) == [(1, 4, 1, 1, 64, 48), (3, 4, 1, 1, 64, 32), (3, 4, 1, 1, 64, 80)]


# ------------------------------------------------------------------ the plain implementation, by hand
def test_plain_dynamic_tanh_and_softcap():
    x = torch.tensor([[0.0, 0.5, -2.0]], dtype=torch.float64)
    y = P.dynamic_tanh(x, torch.tensor([1.0, 2.0, 3.0]), torch.tensor([0.1, 0.0, -0.1]), torch.tensor(2.0))
    assert torch.allclose(y, torch.tensor([[0.1, 2 * math.tanh(1.0), 3 * math.tanh(-4.0) - 0.1]], dtype=torch.float64))
    assert abs(P.softcap(torch.tensor(100.0), 5.0).item() - 5.0) < 1e-9 and abs(P.softcap(torch.tensor(0.01), 5.0).item() - 0.01) < 1e-7


def test_plain_rotation_pairs_halves_and_scores_depend_on_distance_only():
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]], dtype=torch.float64)
    y = P.rotate(x, torch.tensor([3]), base=100.0, dims=4)
    a0, a1 = 3.0, 3.0 * 100.0 ** (-0.5)
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5.0, 6.0]
    assert torch.allclose(y, torch.tensor([want], dtype=torch.float64))
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 8, generator=g, dtype=torch.float64), torch.randn(1, 8, generator=g, dtype=torch.float64)
    s = [(P.rotate(q, torch.tensor([p + 4]), 1e4, 8) * P.rotate(k, torch.tensor([p]), 1e4, 8)).sum().item() for p in (0, 9, 300)]
    assert max(s) - min(s) < 1e-9


def test_plain_routing_by_hand():
    # six experts in three groups of two; scores fall with z.  Group scores: g0 = e1, g1 = e2, g2 = e5.
    z = torch.log(torch.tensor([[0.05, 0.30, 0.25, 0.10, 0.02, 0.28]], dtype=torch.float64))
    idx, w = P.route(z, top=2, groups=3, keep=2)         # keeps g0 and g2: e2 (third largest overall) is closed
    assert idx.tolist() == [[1, 5]] and torch.allclose(w, torch.tensor([[0.30 / 0.58, 0.28 / 0.58]], dtype=torch.float64))
    idx, w = P.route(z, top=3, groups=3, keep=2)
    assert idx.tolist() == [[1, 5, 0]]                   # then e0 of g0, not e2 or e3
    idx, w = P.route(z, top=3, groups=1, keep=1)
    assert idx.tolist() == [[1, 5, 2]] and abs(w.sum().item() - 1.0) < 1e-12
    idx, _ = P.route(torch.zeros(1, 4, dtype=torch.float64), top=2, groups=2, keep=1)
    assert idx.tolist() == [[0, 1]]                      # ties: the lower index


def test_plain_latent_attention_equals_attention_over_the_latent_itself():
    """The identity the package's kernels rest on, checked in float64 on the plain side: carrying the query
    into the latent space and attending over [c ; kr] gives what expanded keys and values give."""
    g = torch.Generator().manual_seed(3)
    m = {"heads": 3, "dim": 5, "rot_dim": 4, "vdim": 7, "kv_rank": 6, "scale": 0.3, "rot": {"base": 50.0, "dims": 4}}
    width, T, eps = 10, 9, 1e-5
    w = {"q": torch.randn(27, width, generator=g), "dkv": torch.randn(10, width, generator=g), "dkv.norm": torch.rand(6, generator=g) + 0.5,
         "uk": torch.randn(15, 6, generator=g), "uv": torch.randn(21, 6, generator=g), "g": torch.randn(3, width, generator=g),
         "o": torch.randn(width, 21, generator=g)}
    w = {"x." + k: v.double() for k, v in w.items()}
    h = torch.randn(T, width, generator=g).double()
    want = P.latent_attention(h, w, "x.", m, eps)
    pos = torch.arange(T)
    q = (h @ w["x.q"].T).view(T, 3, 9)
    dkv = h @ w["x.dkv"].T
    c = P.rms_norm(dkv[:, :6], w["x.dkv.norm"], eps)
    row = torch.cat([c, P.rotate(dkv[:, 6:], pos, 50.0, 4)], -1)                    # what a cache would hold
    out = torch.zeros(T, 3, 7, dtype=torch.float64)
    for hd in range(3):
        uk = w["x.uk"][hd * 5:(hd + 1) * 5]                                          # [dim, rank]
        q_lat = torch.cat([q[:, hd, :5] @ uk, P.rotate(q[:, hd, 5:], pos, 50.0, 4)], -1)
        s = (q_lat @ row.T * 0.3).masked_fill(pos[None, :] > pos[:, None], -math.inf)
        out[:, hd] = (torch.softmax(s, -1) @ c) @ w["x.uv"][hd * 7:(hd + 1) * 7].T * torch.sigmoid(h @ w["x.g"].T)[:, hd:hd + 1]
    assert torch.allclose(out.reshape(T, 21) @ w["x.o"].T, want, atol=1e-10)
