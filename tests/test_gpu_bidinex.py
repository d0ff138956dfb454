"""Bidinex on the GPU: every new kernel alone against plain float64 formulas, then the whole model through
the engine (prompts whole, in portions, token by token, in unequal batches, with slots and pages used
again, long decoding, greedy generation, trace replay) against tests/plain_bidinex.py."""
import dataclasses
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_bidinex as P
from bidinex_tiny import BX_CONFIGS, folder_config, make_bidinex_folder
from tiny import random_prompts, read_weights

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
TOL = {"float32": 4e-5, "bfloat16": 5e-2}             # on max |difference| / max |wanted|
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def rel(got, want) -> float:
    want = want.double()
    return ((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()


class Tally:
    """Errors of logits position by position (root mean square of the difference over that of the wanted rows).
    A float32 run must meet its tolerance at every position.  In a bfloat16 run a router may choose another expert
    where two scores nearly tie, which moves that position and, through attention, some later ones: there the
    median must be small and four positions in five within twice the tolerance; what only shows at single positions
    is the float32 run's to catch, and the kernel tests'."""

    def __init__(self, dtype):
        self.dtype, self.e = dtype, []

    def add(self, got, want, where=None):
        want = want.double().reshape(-1, want.shape[-1])
        d = got.double().cpu().reshape(want.shape) - want
        e = d.pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt().clamp_min(1e-30)
        if self.dtype == "float32":
            assert e.max().item() < TOL["float32"], (where, e.max().item())
        self.e += e.tolist()

    def close(self):
        e = torch.tensor(self.e)
        if self.dtype == "bfloat16":
            assert e.median().item() < TOL["bfloat16"] and (e < 2 * TOL["bfloat16"]).double().mean().item() >= 0.8, \
                (e.median().item(), (e < 2 * TOL["bfloat16"]).double().mean().item())


@pytest.fixture(scope="module")
def K():
    from braidinfer_b200.csrc.api import get_kernels
    return get_kernels(verbose=False)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("bidinex")
    return {n: make_bidinex_folder(root, n) for n in BX_CONFIGS}


class Oracle:
    def __init__(self, folder):
        self.cfg, self.w, self.memo = folder_config(folder), read_weights(folder), {}

    def logits(self, tokens, window=None):
        key = (tuple(tokens), window)
        if key not in self.memo:
            self.memo[key] = P.forward(self.w, self.cfg, list(tokens), window=window)
        return self.memo[key]


@pytest.fixture(scope="module")
def oracles(folders):
    return {n: Oracle(f) for n, f in folders.items()}


def engine(folder, dtype, **kw):
    from braidinfer_b200.engine import Engine
    kw.setdefault("max_tokens", 64 * 12)
    kw.setdefault("verbose", False)
    return Engine.from_folder(folder, dtype=dtype, **kw)


def dev(t, dtype):
    return t.to(TORCH[dtype]).cuda()


# ================================================================== kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_dynamic_tanh_kernel(K, dtype):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, 52, generator=g) * 2
    w, b, a = torch.randn(52, generator=g), torch.randn(52, generator=g), torch.tensor(0.7)
    wd, bd, ad = dev(w, dtype), dev(b, dtype), dev(a, dtype)
    want = P.dynamic_tanh(x.double(), wd.cpu().double(), bd.cpu().double(), ad.cpu().double())
    out = torch.empty(9, 52, dtype=TORCH[dtype], device="cuda")
    K.dyt(x.cuda(), wd, bd, ad, out)
    assert rel(out, want) < (1e-6 if dtype == "float32" else 5e-3)
    idx = torch.tensor([4, -1, 0], dtype=torch.int32, device="cuda")
    out3 = torch.empty(3, 52, dtype=torch.float32, device="cuda")
    K.dyt(x.cuda(), wd, bd, ad, out3, row_index=idx, in_scale=1.5)
    want3 = P.dynamic_tanh(1.5 * x.double()[[4, 0]], wd.cpu().double(), bd.cpu().double(), ad.cpu().double())
    assert rel(out3[[0, 2]], want3) < 1e-6 and out3[1].abs().max() == 0
    xin = x.cuda().clone()
    K.dyt(xin, wd, bd, ad, xin)                      # in place, as an embedding's norm runs
    assert rel(xin, want) < 1e-6


def test_softcap_and_two_streams_side_by_side(K):
    x = torch.linspace(-40, 40, 1001).reshape(7, 143).contiguous()
    y = x.cuda().clone()
    K.softcap(y, 6.5)
    assert rel(y, P.softcap(x.double(), 6.5)) < 1e-6
    a, b = torch.randn(5, 12), torch.randn(5, 12)
    for dt in (torch.float32, torch.bfloat16):
        out = torch.empty(5, 24, dtype=dt, device="cuda")
        K.concat2(a.cuda(), b.cuda(), out)
        assert torch.equal(out.cpu(), torch.cat([a, b], 1).to(dt))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, rot, rot_dims, rank", [(3, 16, 8, 8, 40), (2, 5, 12, 6, 7), (1, 8, 0, 0, 16)])
def test_latent_rows_are_normed_rotated_and_stored_at_their_positions(K, dtype, heads, dim, rot, rot_dims, rank):
    g = torch.Generator().manual_seed(2)
    D, q_cols, ps = rank + rot, heads * (dim + rot), 64
    positions = [62, 63, 64, 65, 0, 1, 130, 0]                   # two sequences and a padding row
    seq = [0, 0, 0, 0, 1, 1, 1, -1]
    rows = len(seq)
    ld = q_cols + D + 3
    proj = dev(torch.randn(rows, ld, generator=g), dtype)
    wn = dev(torch.rand(rank, generator=g) + 0.5, dtype)
    base = 1000.0
    inv = torch.tensor([base ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)], dtype=torch.float32).cuda() \
        if rot_dims else torch.zeros(1, device="cuda")
    table = torch.tensor([[5, 2, -1], [0, 4, 1]], dtype=torch.int32).cuda()
    cache = torch.zeros(6, 1, 1, ps, D, dtype=TORCH[dtype], device="cuda")
    q_lat = torch.zeros(rows, heads, D, dtype=TORCH[dtype], device="cuda")
    K.latent_prep(proj, q_cols, wn, inv, torch.tensor(positions, dtype=torch.int32).cuda(),
                  torch.tensor(seq, dtype=torch.int32).cuda(), table, cache, q_lat, heads, dim, rot, rank, rot_dims, ps, 1e-5)
    K.check_device_errors()
    p64 = proj.cpu().double()
    pos = torch.tensor(positions)
    c = P.rms_norm(p64[:, q_cols:q_cols + rank], wn.cpu().double(), 1e-5)
    kr = P.rotate(p64[:, q_cols + rank:q_cols + D], pos, base, rot_dims)
    qr = P.rotate(p64[:, :q_cols].view(rows, heads, dim + rot)[:, :, dim:], pos, base, rot_dims)
    tol = 2e-6 if dtype == "float32" else 1e-2
    used = set()
    for r in range(rows):
        if seq[r] < 0:
            continue
        page = table[seq[r], positions[r] // ps].item()
        used.add((page, positions[r] % ps))
        got = cache[page, 0, 0, positions[r] % ps]
        assert rel(got, torch.cat([c[r], kr[r]])) < tol, r
    assert rot == 0 or rel(q_lat[:, :, rank:], qr) < tol
    mask = torch.ones(6, ps, dtype=torch.bool)
    for page, off in used:
        mask[page, off] = False
    assert cache[:, 0, 0][mask.cuda()].abs().max() == 0          # nothing else was written, the padding row least of all


@pytest.mark.parametrize("dtype", DTYPES)
def test_per_head_products_with_and_without_gate(K, dtype):
    g = torch.Generator().manual_seed(3)
    rows, heads, k, j = 70, 3, 20, 37
    big = dev(torch.randn(rows, heads * (k + 4) + 5, generator=g), dtype)
    x = big[:, :heads * (k + 4)].view(rows, heads, k + 4)[:, :, :k]              # a view with gaps, as the mixer passes it
    gate = big[:, heads * (k + 4):heads * (k + 4) + heads]
    w = dev(torch.randn(heads, j, k, generator=g), dtype)
    out = torch.zeros(rows, heads, j + 2, dtype=TORCH[dtype], device="cuda")
    K.gemm_heads(x, w, out[:, :, :j])
    want = torch.einsum("nhk,hjk->nhj", x.cpu().double(), w.cpu().double())
    tol = 2e-6 if dtype == "float32" else 1e-2
    assert rel(out[:, :, :j], want) < tol and out[:, :, j:].abs().max() == 0
    K.gemm_heads(x, w, out[:, :, :j], gate=gate, mult=0.7)
    want = want * 0.7 * torch.sigmoid(gate.cpu().double())[:, :, None]
    assert rel(out[:, :, :j], want) < tol


def plain_latent_mqa(q_lat, keys, positions, rank, scale, window=None):
    """q_lat [rows, H, D], keys [T, D] (row j is position j), float64: attention over the rows themselves."""
    T = keys.shape[0]
    j = torch.arange(T)[None, :]
    p = torch.tensor(positions)[:, None]
    vis = j <= p
    if window:
        vis = vis & (p - j < window)
    s = torch.einsum("nhd,td->nht", q_lat, keys) * scale
    s = s.masked_fill(~vis[:, None, :], -math.inf)
    return torch.softmax(s, -1) @ keys[:, :rank]


def paged(keys, dtype, ps=64, seed=0):
    """Scatter rows [T, D] over shuffled pages; returns (cache [pages, 1, 1, ps, D], table [1, blocks])."""
    T, D = keys.shape
    blocks = -(-T // ps)
    perm = torch.randperm(blocks + 3, generator=torch.Generator().manual_seed(seed))[:blocks]
    cache = torch.zeros(blocks + 3, 1, 1, ps, D, dtype=TORCH[dtype])
    for b in range(blocks):
        n = min(ps, T - b * ps)
        cache[perm[b], 0, 0, :n] = keys[b * ps:b * ps + n].to(TORCH[dtype])
    return cache.cuda(), perm.to(torch.int32)[None, :].cuda()


def attend(K, kernel, q, out, cache, table, positions, rank, window, scale, n_splits=1):
    """One sequence whose rows stand at consecutive `positions`, through the plain or the tensor-core kernel."""
    rows = len(positions)
    if kernel == "simple":
        K.attn_latent_simple(q, out, cache, table, torch.tensor(positions, dtype=torch.int32).cuda(),
                             torch.zeros(rows, dtype=torch.int32).cuda(), rank, window, scale)
    else:
        i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
        K.attn_latent_mma(q, out, cache, table, i32([0]), i32([rows]), i32([positions[0]]), torch.zeros(rows, dtype=torch.int32).cuda(),
                          1, rows, rank, window, scale, n_splits=n_splits)
    K.check_device_errors()


# "mma64": a latent whose rank is a multiple of 64 and few heads, so that a decoded token runs the kernel for few pairs
KERNELS = [("float32", "simple", 1), ("bfloat16", "simple", 1), ("bfloat16", "mma", 1), ("bfloat16", "mma", 4),
           ("bfloat16", "mma64", 1), ("bfloat16", "mma64", 5)]


@pytest.mark.parametrize("dtype, kernel, n_splits", KERNELS)
@pytest.mark.parametrize("far", [0, 3, 31, 32, 63, 64, 65, 127, 128, 640, 699])
def test_one_far_key_that_stands_out_is_found_by_prompt_rows_and_by_a_decoded_token(K, dtype, kernel, n_splits, far):
    """Hundreds of keys with small scores and one, far back or at a page's edge, that every query points at:
    if it were missed the output would be another vector altogether."""
    g = torch.Generator().manual_seed(far)
    T, heads, rank, rot = {"simple": (700, 2, 24, 8), "mma": (700, 5, 32, 16), "mma64": (700, 3, 64, 16)}[kernel]
    D = rank + rot
    keys = torch.randn(T, D, generator=g) * 0.3
    u = torch.randn(D, generator=g)
    u = u / u.norm()
    keys[far] = 6.0 * u + 0.3 * torch.randn(D, generator=g)
    keys = keys.to(TORCH[dtype]).double()
    cache, table = paged(keys, dtype, seed=far)
    for positions in ([699], list(range(690, 700))):                # a decoded token; a prompt's last portion
        rows = len(positions)
        q = (4.0 * u[None, None, :] + 0.2 * torch.randn(rows, heads, D, generator=g)).to(TORCH[dtype])
        out = torch.empty(rows, heads, rank, dtype=TORCH[dtype], device="cuda")
        attend(K, kernel, q.cuda(), out, cache, table, positions, rank, None, 0.5, n_splits)
        want = plain_latent_mqa(q.double(), keys, positions, rank, 0.5)
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert rel(out, want) < tol
        without = plain_latent_mqa(q.double(), torch.cat([keys[:far], keys[far:far + 1] * 0, keys[far + 1:]]), positions, rank, 0.5)
        assert rel(without, want) > 0.5                              # the test would see a missed key


@pytest.mark.parametrize("dtype, kernel, n_splits", KERNELS)
@pytest.mark.parametrize("window", [1, 2, 5, 32, 33, 64, 65, 200])
def test_window_edges_just_inside_and_just_outside(K, dtype, kernel, n_splits, window):
    g = torch.Generator().manual_seed(window)
    T, heads, rank, rot = {"simple": (300, 3, 16, 4), "mma": (300, 3, 16, 16), "mma64": (300, 2, 128, 0)}[kernel]
    D = rank + rot
    u = torch.randn(D, generator=g)
    u = u / u.norm()
    for positions in ([299], [297, 298, 299]):
        for edge in (0, 1):                                           # 0: the last key the window keeps; 1: the first it drops
            keys = torch.randn(T, D, generator=g) * 0.3
            j_star = positions[-1] - window + 1 - edge
            keys[j_star] = 6.0 * u
            keys = keys.to(TORCH[dtype]).double()
            cache, table = paged(keys, dtype, seed=window)
            rows = len(positions)
            q = (4.0 * u[None, None, :] + 0.2 * torch.randn(rows, heads, D, generator=g)).to(TORCH[dtype])
            out = torch.empty(rows, heads, rank, dtype=TORCH[dtype], device="cuda")
            attend(K, kernel, q.cuda(), out, cache, table, positions, rank, window, 0.5, n_splits)
            want = plain_latent_mqa(q.double(), keys, positions, rank, 0.5, window)
            assert rel(out, want) < (1e-5 if dtype == "float32" else 2e-2)
            hit = (out[-1, 0].double().cpu() - keys[j_star, :rank]).abs().max().item() < 0.5
            assert hit == (edge == 0)                                 # seen just inside, not seen just outside


@pytest.mark.parametrize("n_splits", [1, 6])
@pytest.mark.parametrize("rank, rot, heads, n_seqs", [(64, 16, 4, 5), (192, 32, 16, 3), (256, 0, 1, 9)])
def test_decoded_tokens_of_few_heads_share_a_tile_among_the_warps(K, n_splits, rank, rot, heads, n_seqs):
    """One token a sequence (and one sequence with two), contexts that end at, before and after page borders."""
    g = torch.Generator().manual_seed(rank + heads)
    D, ps = rank + rot, 64
    before = [0, 63, 64, 130, 700, 31, 32, 1, 255][:n_seqs]
    q_len = [1] * n_seqs
    q_len[-1] = 2 if heads * 2 <= 32 else 1
    total = [b + n for b, n in zip(before, q_len)]
    blocks = [-(-t // ps) for t in total]
    order = torch.randperm(sum(blocks) + 1, generator=g).tolist()
    cache = torch.zeros(sum(blocks) + 1, 1, 1, ps, D, dtype=torch.bfloat16)
    table = torch.full((n_seqs, max(blocks)), -1, dtype=torch.int32)
    keys = []
    for s_, t in enumerate(total):
        k = (torch.randn(t, D, generator=g) * 0.7).to(torch.bfloat16)
        keys.append(k.double())
        for b in range(blocks[s_]):
            page = order.pop()
            table[s_, b] = page
            n = min(ps, t - b * ps)
            cache[page, 0, 0, :n] = k[b * ps:b * ps + n]
    rows = sum(q_len) + 2
    q = (torch.randn(rows, heads, D, generator=g) * 1.0).to(torch.bfloat16)
    q_start = [sum(q_len[:i]) for i in range(n_seqs)]
    token_seq = sum(([i] * n for i, n in enumerate(q_len)), []) + [-1] * 2
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    lib = K.latent_attention_library(rank, rot)
    assert lib.braid_latent_attn_tile_rows(max(q_len), heads) == 16
    out = torch.full((rows, heads, rank), 7.0, dtype=torch.bfloat16, device="cuda")
    K.attn_latent_mma(q.cuda(), out, cache.cuda(), table.cuda(), i32(q_start), i32(q_len), i32(before), i32(token_seq),
                      n_seqs, max(q_len), rank, None, 0.2, n_splits=n_splits)
    K.check_device_errors()
    for s_ in range(n_seqs):
        a, n = q_start[s_], q_len[s_]
        want = plain_latent_mqa(q[a:a + n].double(), keys[s_], list(range(before[s_], before[s_] + n)), rank, 0.2)
        assert rel(out[a:a + n], want) < 2e-2, s_
    assert (out[-2:] == 7.0).all()


@pytest.mark.parametrize("n_splits", [1, 3])
@pytest.mark.parametrize("rank, rot, heads", [(32, 16, 5), (48, 0, 2), (16, 32, 70)])
def test_tensor_core_attention_on_a_batch_of_unequal_sequences(K, n_splits, rank, rot, heads):
    """Prompts, a portion after a long context and a decoded token in one step, tiles that straddle tokens, rows
    of padding, every sequence on pages of its own order: against float64 and against the plain kernel."""
    g = torch.Generator().manual_seed(rank + heads)
    D, ps = rank + rot, 64
    before, q_len = [0, 100, 650, 63], [70, 1, 3, 2]
    total = [b + n for b, n in zip(before, q_len)]
    blocks = [-(-t // ps) for t in total]
    pages = sum(blocks) + 2
    order = torch.randperm(pages, generator=g).tolist()
    cache = torch.zeros(pages, 1, 1, ps, D, dtype=torch.bfloat16)
    table = torch.full((4, max(blocks)), -1, dtype=torch.int32)
    keys = []
    for s_, t in enumerate(total):
        k = (torch.randn(t, D, generator=g) * 0.7).to(torch.bfloat16)
        keys.append(k.double())
        for b in range(blocks[s_]):
            page = order.pop()
            table[s_, b] = page
            n = min(ps, t - b * ps)
            cache[page, 0, 0, :n] = k[b * ps:b * ps + n]
    rows = sum(q_len) + 4                                                  # four rows of padding
    q = (torch.randn(rows, heads, D, generator=g) * 1.5).to(torch.bfloat16)
    q_start = [sum(q_len[:i]) for i in range(4)]
    token_seq = sum(([i] * n for i, n in enumerate(q_len)), []) + [-1] * 4
    positions = sum((list(range(b, b + n)) for b, n in zip(before, q_len)), []) + [0] * 4
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    out = torch.full((rows, heads, rank), 7.0, dtype=torch.bfloat16, device="cuda")
    K.attn_latent_mma(q.cuda(), out, cache.cuda(), table.cuda(), i32(q_start), i32(q_len), i32(before), i32(token_seq),
                      4, max(q_len), rank, None, 0.3, n_splits=n_splits)
    twin = torch.empty_like(out)
    K.attn_latent_simple(q.cuda(), twin, cache.cuda(), table.cuda(), i32(positions), i32(token_seq), rank, None, 0.3)
    K.check_device_errors()
    for s_ in range(4):
        a, n = q_start[s_], q_len[s_]
        want = plain_latent_mqa(q[a:a + n].double(), keys[s_], list(range(before[s_], before[s_] + n)), rank, 0.3)
        assert rel(out[a:a + n], want) < 2e-2, s_
        assert rel(out[a:a + n], twin[a:a + n].double().cpu()) < 2e-2, s_
    assert (out[-4:] == 7.0).all()                                         # padding rows are left alone


@pytest.mark.parametrize("rows", [5, 70])
def test_tensor_core_per_head_products_against_the_plain_twin(K, rows):
    g = torch.Generator().manual_seed(rows)
    heads, k, j = 3, 24, 37
    big = (torch.randn(rows, heads * (k + 8) + 8, generator=g)).to(torch.bfloat16).cuda()
    x = big[:, :heads * (k + 8)].view(rows, heads, k + 8)[:, :, :k]
    gate = big[:, heads * (k + 8):heads * (k + 8) + heads]
    w = torch.randn(heads, j, k, generator=g).to(torch.bfloat16).cuda()
    for gt in (None, gate):
        out = torch.zeros(rows, heads, j + 1, dtype=torch.bfloat16, device="cuda")
        twin = torch.zeros_like(out)
        K.gemm_heads(x, w, out[:, :, :j], gate=gt, mult=0.7)
        K.gemm_heads(x, w, twin[:, :, :j], gate=gt, mult=0.7, tensor_cores=False)
        want = torch.einsum("nhk,hjk->nhj", x.cpu().double(), w.cpu().double())
        if gt is not None:
            want = want * 0.7 * torch.sigmoid(gt.cpu().double())[:, :, None]
        assert rel(out[:, :, :j], want) < 1e-2 and rel(out, twin.double().cpu()) < 1e-2 and out[:, :, j:].abs().max() == 0


@pytest.mark.parametrize("tile", [16, 64])
def test_tensor_core_expert_products_against_the_plain_twin(K, tile):
    g = torch.Generator().manual_seed(tile + 1)
    rows, width, ff, experts, top = 150, 40, 72, 5, 2
    x = torch.randn(rows, width, generator=g).to(torch.bfloat16).cuda()
    wg, wu = [(torch.randn(experts, ff, width, generator=g) * 0.3).to(torch.bfloat16).cuda() for _ in range(2)]
    wd = (torch.randn(experts, width, ff, generator=g) * 0.3).to(torch.bfloat16).cuda()
    idx = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).to(torch.int32)
    idx[idx == 3] = 0                                                      # no row goes to expert 3
    idx[:, 1][idx[:, 1] == idx[:, 0]] = 4
    seq = torch.zeros(rows, dtype=torch.int32)
    seq[-2:] = -1
    plan = K.moe_plan(idx.cuda(), seq.cuda(), experts, tile)
    slots = plan[4] * tile
    res = []
    for fn in (K.moe_gemm_mma, K.moe_gemm_simt):
        act = torch.zeros(slots, ff, dtype=torch.bfloat16, device="cuda")
        y = torch.zeros(slots, width, dtype=torch.bfloat16, device="cuda")
        fn(x, wg, wu, act, plan, top, tile)
        fn(act, wd, None, y, plan, top, tile)
        res.append((act, y))
    live = (plan[0] >= 0)
    assert rel(res[0][0][live], res[1][0][live].double().cpu()) < 1e-2 and rel(res[0][1][live], res[1][1][live].double().cpu()) < 2e-2
    assert res[0][0][~live[:slots]].abs().max() == 0                       # padding slots hold zeros


@pytest.mark.parametrize("experts, groups, keep, top", [(6, 3, 2, 2), (5, 5, 3, 3), (64, 8, 4, 6), (4, 1, 1, 1), (8, 2, 1, 4),
                                                         (3, 1, 1, 3)])
def test_routing_kernel_against_the_plain_choice(K, experts, groups, keep, top):
    g = torch.Generator().manual_seed(experts)
    z = torch.randn(41, experts, generator=g) * 2
    idx = torch.empty(41, top, dtype=torch.int32, device="cuda")
    w = torch.empty(41, top, dtype=torch.float32, device="cuda")
    K.moe_route(z.cuda(), idx, w, groups, keep, mult=0.7)
    want_idx, want_w = P.route(z.double(), top, groups, keep)
    assert torch.equal(idx.cpu().long(), want_idx)
    assert rel(w, 0.7 * want_w) < 1e-5
    K.moe_route(torch.zeros(2, experts).cuda(), idx[:2], w[:2], groups, keep)      # all equal: the lowest indices
    assert idx[0].tolist() == list(range(top))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tile", [16, 64])
def test_experts_over_sorted_rows_and_the_weighted_sum(K, dtype, tile):
    g = torch.Generator().manual_seed(tile)
    rows, width, ff, experts, top = 45, 40, 28, 5, 2
    x = dev(torch.randn(rows, width, generator=g), dtype)
    wg, wu = dev(torch.randn(experts, ff, width, generator=g) * 0.3, dtype), dev(torch.randn(experts, ff, width, generator=g) * 0.3, dtype)
    wd = dev(torch.randn(experts, width, ff, generator=g) * 0.3, dtype)
    idx = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).to(torch.int32)
    idx[:, 0][idx[:, 0] == 3] = 4                                          # expert 3 sees few rows or none
    idx[:, 1][idx[:, 1] == idx[:, 0]] = 0
    wt = torch.rand(rows, top, generator=g)
    seq = torch.zeros(rows, dtype=torch.int32)
    seq[-3:] = -1                                                          # padding rows take no slot and get nothing
    plan = K.moe_plan(idx.cuda(), seq.cuda(), experts, tile)
    slots = plan[4] * tile
    act = torch.empty(slots, ff, dtype=TORCH[dtype], device="cuda")
    y = torch.empty(slots, width, dtype=TORCH[dtype], device="cuda")
    K.moe_gemm_simt(x, wg, wu, act, plan, top, tile)
    K.moe_gemm_simt(act, wd, None, y, plan, top, tile)
    h0 = torch.randn(rows, width, generator=g)
    h = h0.cuda().clone()
    K.moe_combine(h, y, plan, wt.cuda())
    slot_pair, pair_slot, tile_expert, meta, _ = [t.cpu() if torch.is_tensor(t) else t for t in plan]
    live = (seq >= 0)
    assert (pair_slot.view(rows, top)[~live] == -1).all() and (pair_slot.view(rows, top)[live] >= 0).all()
    for pair, slot in enumerate(pair_slot.tolist()):
        if slot >= 0:
            assert slot_pair[slot] == pair and tile_expert[slot // tile] == idx.view(-1)[pair]
    assert (slot_pair >= 0).sum() == live.sum() * top and meta[0] <= plan[4]
    x64 = x.cpu().double()
    want = h0.double().clone()
    for r in range(rows - 3):
        for k in range(top):
            e = idx[r, k].item()
            want[r] += wt[r, k].double() * P.expert(x64[r:r + 1], wg[e].cpu().double(), wu[e].cpu().double(), wd[e].cpu().double())[0]
    assert rel(h, want) < (2e-6 if dtype == "float32" else 2e-2)


# ================================================================== the whole model through the engine
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_and_every_layer_run(folders, oracles, name, dtype):
    eng = engine(folders[name], dtype)
    cfg = oracles[name].cfg
    tally = Tally(dtype)
    for n, seed in ((1, 0), (2, 1), (67, 2), (130, 3)):
        toks = random_prompts(cfg["vocab"], [n], seed)[0]
        s = eng.open()
        taps = []
        got = eng.step([(s, toks)], want="all", tap=lambda i, h: taps.append(h.clone()))
        eng.close(s)
        eng.check()
        tally.add(got, oracles[name].logits(toks), (name, n))
        if n == 67:
            streams = []
            P.forward(oracles[name].w, cfg, toks, streams)
            assert len(taps) == len(streams) == 1 + len(P.layer_runs(cfg))
            for i, (a, b) in enumerate(zip(taps, streams)):
                Tally(dtype).add(a, b, (name, "after run", i))
    tally.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_token_by_token_from_the_first_token_equals_the_prompt_whole(folders, oracles, name, dtype):
    eng = engine(folders[name], dtype)
    toks = random_prompts(oracles[name].cfg["vocab"], [70], 7)[0]
    want = oracles[name].logits(toks)
    s, tally = eng.open(), Tally(dtype)
    for t, tok in enumerate(toks):
        tally.add(eng.step([(s, [tok])], want="last"), want[t:t + 1], t)
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 62, 1, 3, 64, 18], [63, 2, 2, 83], [128, 22], [1, 1, 2, 146]])
def test_a_prompt_in_portions(folders, oracles, dtype, cuts):
    eng = engine(folders["A"], dtype)
    toks = random_prompts(oracles["A"].cfg["vocab"], [150], 9)[0]
    want = oracles["A"].logits(toks)
    s, at, tally = eng.open(), 0, Tally(dtype)
    for c in cuts:
        tally.add(eng.step([(s, toks[at:at + c])], want="all"), want[at:at + c], (at, c))
        at += c
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_unequal_requests_in_one_batch_then_decoded_together_and_slots_used_again(folders, oracles, name, dtype):
    eng = engine(folders[name], dtype, max_tokens=64 * 10, max_slots=4)
    vocab = oracles[name].cfg["vocab"]
    prompts = random_prompts(vocab, [3 + 4, 70 + 9, 1 + 2, 129 + 6], 21)
    cut = [3, 70, 1, 129]
    want = [oracles[name].logits(p) for p in prompts]
    slots = [eng.open() for _ in prompts]
    lg = eng.step([(s, p[:c]) for s, p, c in zip(slots, prompts, cut)], want="all")
    off, tally = 0, Tally(dtype)
    for p, c, w in zip(prompts, cut, want):
        tally.add(lg[off:off + c], w[:c])
        off += c
    live = list(range(4))
    t = 0
    while live:
        lg = eng.step([(slots[i], [prompts[i][cut[i] + t]]) for i in live], want="last")
        for j, i in enumerate(live):
            tally.add(lg[j:j + 1], want[i][cut[i] + t:cut[i] + t + 1], (i, t))
        t += 1
        for i in list(live):
            if cut[i] + t == len(prompts[i]):
                eng.close(slots[i])                                  # the shorter requests end earlier
                live.remove(i)
    assert all(n == 0 for n in eng.cache.pages_in_use())
    # the freed slots and pages serve other requests; what they held before must not show
    again = random_prompts(vocab, [66, 5], 22)
    slots = [eng.open(), eng.open()]
    lg = eng.step([(slots[0], again[0]), (slots[1], again[1])], want="all")
    tally.add(lg[:66], oracles[name].logits(again[0]), "slot used again")
    tally.add(lg[66:], oracles[name].logits(again[1]), "slot used again")
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_across_page_borders(folders, oracles, dtype):
    eng = engine(folders["C"], dtype)
    toks = random_prompts(oracles["C"].cfg["vocab"], [5 + 140], 31)[0]
    want = oracles["C"].logits(toks)
    s, tally = eng.open(), Tally(dtype)
    eng.step([(s, toks[:5])], want=None)
    for t in range(5, len(toks)):
        tally.add(eng.step([(s, [toks[t]])], want="last"), want[t:t + 1], t)
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_window_on_the_mixer_through_a_hand_made_description(folders, oracles, dtype):
    """No model of this design has a window; the mixer and the cache do.  Prompt, portions and decoding with a
    window of 5 on every mixer against the plain implementation with the same window."""
    from braidinfer_b200.config import read_config_json
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.models import architecture_for
    cfg = read_config_json(folders["B"])
    arch = architecture_for(cfg)
    spec = arch.build_spec(arch.config_from_dict(cfg))
    layers = tuple(dataclasses.replace(l, mixer=dataclasses.replace(l.mixer, params={**l.mixer.params, "window": 5}))
                   for l in spec.layers)
    eng = Engine(None, folders["B"], dtype=dtype, max_tokens=64 * 6, verbose=False, spec=dataclasses.replace(spec, layers=layers))
    toks = random_prompts(cfg["vocab"], [80], 41)[0]
    want = oracles["B"].logits(toks, window=5)
    assert rel(want, oracles["B"].logits(toks)) > 0.1                  # the window matters here
    s, at, tally = eng.open(), 0, Tally(dtype)
    for c in [3, 4, 60] + [1] * 13:
        tally.add(eng.step([(s, toks[at:at + c])], want="all"), want[at:at + c], at)
        at += c
    tally.close()
    assert eng.cache.pages_in_use() == [1, 1]                           # the page the window has passed went back
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_library_entry_point(folders, oracles, dtype):
    import braidinfer_b200 as lib
    model = lib.load(folders["A"], dtype=dtype, max_seq_len=256, max_batch=3, verbose=False)
    prompts = random_prompts(oracles["A"].cfg["vocab"], [4, 61, 17, 9], 51)          # four requests, three slots
    outs = model.generate(prompts, lib.SamplingParams.greedy(), stop_tokens=(), max_new_tokens=[6, 8, 3, 5])
    for p, o, n in zip(prompts, outs, [6, 8, 3, 5]):
        assert len(o.tokens) == n
        toks = list(p)
        for t in o.tokens:
            row = oracles["A"].logits(toks)[-1]
            if dtype == "float32":
                assert t == P.argmax_lowest(row)
            else:
                assert row[t] >= row.max() - 2 * TOL[dtype] * row.abs().max()
            toks.append(t)
    model.engine.check()


def test_trace_replay_program_on_a_model_folder(folders, oracles, tmp_path):
    toks = random_prompts(oracles["C"].cfg["vocab"], [40, 9], 61)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[0][:33], "want": [0, 32]}, {"id": "b", "tokens": toks[1][:8], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [toks[0][33]], "want": [0]}, {"id": "b", "tokens": [toks[1][8]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [toks[0][34]], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": toks[0][35:], "want": [4]}], "end": ["a"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["C"], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps).encode(),
                       capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr.decode()[-2000:]
    assert [l for l in p.stdout.decode().split("\n") if l.startswith("done")] == [f"done {i}" for i in range(4)]
    import numpy as np
    vocab = oracles["C"].cfg["vocab"]
    wa, wb = oracles["C"].logits(toks[0]), oracles["C"].logits(toks[1])
    got = {i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab)) for i in (0, 1, 3)}
    assert not (out / "2.f32").exists()
    assert rel(got[0], wa[[0, 32]]) < TOL["float32"] and rel(got[1], torch.stack([wa[33], wb[8]])) < TOL["float32"]
    assert rel(got[3], wa[39:40]) < TOL["float32"]


def test_generate_command_line_on_a_model_folder(folders, oracles):
    env = dict(os.environ, MODEL=folders["B"], MAX_TOKENS="6", RAW="1", DTYPE="float32", MAX_SEQ_LEN="128")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "7, 200, 31, 4"], env=env, capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    toks, want = [7, 200, 31, 4], []
    for _ in range(6):
        t = P.argmax_lowest(oracles["B"].logits(toks)[-1])
        want.append(t)
        toks.append(t)
    assert [int(x) for x in p.stdout.split()] == want
