"""Loduzen on the GPU: every new kernel alone against plain float64 formulas, then the whole model through the
engine (prompts whole, in portions, token by token, in unequal batches, with slots and pages used again, long
decoding, greedy generation, trace replay, the command line) against tests/plain_loduzen.py."""
import dataclasses
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import plain_loduzen as P
from loduzen_tiny import LZ_CONFIGS, folder_config, make_loduzen_folder, random_config
from tiny import random_prompts, read_weights

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
TOL = {"float32": 2e-4, "bfloat16": 6e-2}              # on the root mean square of a row's error over that of the wanted rows
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
D = torch.float64


def rel(got, want) -> float:
    want = want.double()
    return ((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()


def dev(x, dtype):
    return x.to(TORCH[dtype]).cuda()


def back(x):
    return x.double().cpu()


class Tally:
    """Errors of logits (or streams) position by position: root mean square of the difference over that of all the
    wanted rows.  A float32 run must meet its tolerance at every position.  These models are made sensitive on
    purpose (peaked attention, norms of small vectors), and at a few positions a rounding error grows a hundred- to a
    thousandfold (the float32 run shows the same positions as its worst; its typical error is 1e-6, its tolerance
    2e-4, a lost key or state moves a position by 1e-2 and more): a bfloat16 run must be right in the median, within
    its tolerance at nine positions in ten, and nowhere off by more than the wanted rows' own size."""

    def __init__(self, dtype):
        self.dtype, self.e = dtype, []

    def add(self, got, want, where=None):
        want = want.double().reshape(-1, want.shape[-1])
        d = got.double().cpu().reshape(want.shape) - want
        e = d.pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt().clamp_min(1e-30)
        assert e.max().item() < (TOL["float32"] if self.dtype == "float32" else 1.0), (where, e.max().item())
        self.e += e.tolist()

    def close(self):
        e = torch.tensor(self.e)
        assert len(self.e) > 0
        if self.dtype == "bfloat16":
            assert e.median().item() < 0.5 * TOL["bfloat16"] and (e < TOL["bfloat16"]).double().mean().item() >= 0.9, \
                (e.median().item(), (e < TOL["bfloat16"]).double().mean().item())


@pytest.fixture(scope="module")
def K():
    from braidinfer_b200.csrc.api import get_kernels
    return get_kernels(verbose=False)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("loduzen")
    return {n: make_loduzen_folder(base, n) for n in LZ_CONFIGS}


class Oracle:
    def __init__(self, folder):
        self.cfg, self.w, self.memo = folder_config(folder), read_weights(folder), {}

    def logits(self, tokens, cfg=None):
        key = (tuple(tokens), json.dumps(cfg, sort_keys=True) if cfg else None)
        if key not in self.memo:
            self.memo[key] = P.forward(self.w, cfg or self.cfg, list(tokens))
        return self.memo[key]


@pytest.fixture(scope="module")
def oracles(folders):
    return {n: Oracle(f) for n, f in folders.items()}


def engine(folder, dtype, **kw):
    from braidinfer_b200.engine import Engine
    kw.setdefault("max_tokens", 64 * 16)
    kw.setdefault("verbose", False)
    return Engine.from_folder(folder, dtype=dtype, **kw)


def step_tables(lengths, before=None, slots=None, pad=0):
    """The device tables of a step whose sequences bring `lengths` tokens (as the step packer lays them out)."""
    n = len(lengths)
    before = before or [0] * n
    rows = sum(lengths) + pad
    token_seq = torch.full((rows,), -1, dtype=torch.int32)
    positions = torch.zeros(rows, dtype=torch.int32)
    q_start, r = [], 0
    for i, (ln, b) in enumerate(zip(lengths, before)):
        q_start.append(r)
        token_seq[r:r + ln] = i
        positions[r:r + ln] = torch.arange(b, b + ln, dtype=torch.int32)
        r += ln
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()      # noqa: E731
    return SimpleNamespace(rows=rows, n_tokens=sum(lengths), n_seqs=n, token_seq=token_seq.cuda(), positions=positions.cuda(),
                           q_start=i32(q_start), q_len=i32(lengths), kv_before=i32(before),
                           slot_ids=i32(slots if slots is not None else list(range(n))), max_q_len=max(lengths),
                           host_q_start=q_start)


# ================================================================== kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("adjacent, hd, rope_dim, value_is_key, normed", [(True, 32, 16, True, True), (True, 40, 40, True, True),
                                                                          (False, 32, 16, False, True), (True, 16, 0, True, False),
                                                                          (False, 48, 48, False, False), (True, 6, 4, True, True)])
def test_head_norm_rotation_and_cache_write(K, dtype, adjacent, hd, rope_dim, value_is_key, normed):
    g = torch.Generator().manual_seed(hd + rope_dim)
    nqh, nkh, page = 4, 2, 64
    lengths, before = [3, 70, 1], [0, 60, 129]
    t = step_tables(lengths, before, pad=2)
    heads = nqh + nkh * (1 if value_is_key else 2)
    stride = -(-heads * hd // 8) * 8
    qk0 = torch.randn(t.rows, stride, generator=g)
    qk = dev(qk0, dtype)
    src = back(qk)
    wq, wk = dev(1 + 0.3 * torch.randn(hd, generator=g), dtype), dev(1 + 0.3 * torch.randn(hd, generator=g), dtype)
    rot = {"base": 100.0, "dims": rope_dim, "scaling": {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    f, amp = P.rotation_table(rot)
    pages = torch.tensor([[5, 1, -1, -1], [0, 7, 2, -1], [3, 4, 6, -1]], dtype=torch.int32).cuda()
    cache = torch.zeros(8, 2, nkh, page, hd, dtype=TORCH[dtype], device="cuda")
    K.head_norm_rope_kv(qk, wq if normed else None, wk if normed else None, f.float().cuda(), t.positions, t.token_seq, pages, cache,
                        nqh, nkh, hd, rope_dim, adjacent, value_is_key, page, 1e-5, amp)
    K.check_device_errors()
    tol = 2e-5 if dtype == "float32" else 1.2e-2           # angles are float32: half a unit in the last place of 130 radians
    got = back(qk)
    assert torch.equal(got[-2:], src[-2:])                                  # rows of padding are left alone
    pos = t.positions.cpu()[:t.n_tokens]

    def turned(x, w):
        x = x.clone()
        if normed:
            x = P.rms(x, 1e-5, back(w))
        if adjacent:
            return P.rotate_pairs(x, pos, rot)
        half = rope_dim // 2
        ang = pos.to(D)[:, None] * f[None, :]
        c, s = (torch.cos(ang) * amp)[:, None], (torch.sin(ang) * amp)[:, None]
        a, b = x[..., :half], x[..., half:rope_dim]
        return torch.cat([a * c - b * s, b * c + a * s, x[..., rope_dim:]], -1)

    q_in = src[:t.n_tokens, :nqh * hd].view(-1, nqh, hd)
    k_in = src[:t.n_tokens, nqh * hd:(nqh + nkh) * hd].view(-1, nkh, hd)
    q_want, k_want = turned(q_in, wq), turned(k_in, wk)
    assert rel(got[:t.n_tokens, :nqh * hd].view(-1, nqh, hd), q_want) < tol
    assert rel(got[:t.n_tokens, nqh * hd:(nqh + nkh) * hd].view(-1, nkh, hd), k_want) < tol
    v_want = k_in if value_is_key else src[:t.n_tokens, (nqh + nkh) * hd:(nqh + 2 * nkh) * hd].view(-1, nkh, hd)
    c = back(cache)
    seq = t.token_seq.cpu()
    for r in range(t.n_tokens):
        p_ = int(pos[r])
        pg = int(pages[int(seq[r]), p_ // page])
        assert rel(c[pg, 0, :, p_ % page], k_want[r]) < tol
        assert torch.equal(c[pg, 1, :, p_ % page], v_want[r])               # values are copied as they came in
    assert c.abs().sum(dim=(1, 2, 4)).ne(0).sum().item() == t.n_tokens      # nothing else was written


def plain_attention(q, keys, values, pos, kv_len, window, scale, sink, nkh):
    """q [rows, heads, hd] at positions `pos` over keys/values [kv_len, nkh, hd] of one sequence."""
    rows, heads, hd = q.shape
    j = torch.arange(kv_len)[None, :]
    vis = (j <= pos[:, None]) & ((pos[:, None] - j < window) if window else True)
    out = torch.zeros(rows, heads, hd, dtype=D)
    for h in range(heads):
        s = (q[:, h] @ keys[:, h // (heads // nkh)].T) * scale
        if sink:
            p = P.sink_softmax(s, vis)
        else:
            p = torch.softmax(torch.where(vis, s, torch.full_like(s, -1e300)), -1)
        out[:, h] = p @ values[:, h // (heads // nkh)]
    return out


@pytest.mark.parametrize("kernel", ["simple_f32", "simple_bf16", "mma_prompt", "mma_few_1", "mma_few_9", "tcgen05_prompt", "tcgen05_prompt_128"])
@pytest.mark.parametrize("window", [0, 70, 1])
def test_attention_with_a_sink_and_a_factor_on_its_result(K, kernel, window):
    g = torch.Generator().manual_seed(window + len(kernel))
    dtype = "float32" if kernel == "simple_f32" else "bfloat16"
    nqh, nkh, hd, page, scale, factor = 4, 2, {"tcgen05_prompt": 64, "tcgen05_prompt_128": 128}.get(kernel, 32), 64, 0.35, 1.3
    few = kernel.startswith("mma_few")
    lengths, before = ([1, 2], [700, 130]) if few else ([150, 37], [0, 200])
    t = step_tables(lengths, before, pad=1)
    total = [b + n for b, n in zip(before, lengths)]
    blocks = max(-(-x // page) for x in total)
    perm = torch.randperm(2 * blocks + 1, generator=g)
    table = torch.full((2, 16), -1, dtype=torch.int32)
    cache = torch.zeros(2 * blocks + 1, 2, nkh, page, hd, dtype=TORCH[dtype], device="cuda")
    q0 = torch.randn(t.rows, nqh, hd, generator=g)
    q0[:, :, 0] = 4.0
    q = dev(q0.view(t.rows, nqh * hd), dtype)
    kv = []
    for s in range(2):
        keys = torch.randn(total[s], nkh, hd, generator=g)
        vals = torch.randn(total[s], nkh, hd, generator=g)
        # scores below the sink's everywhere (the first number of every key against that of every query) but at two
        # keys, one just inside a window of 70 for the last query and one just outside: leaving the sink out, or
        # moving the window by one, shows at once
        keys *= 0.3
        keys[:, :, 0] = -3.0
        for off in (69, 70):
            if total[s] - 1 - off >= 0:
                keys[total[s] - 1 - off, :, 0] = 1.5
        keys, vals = keys.to(TORCH[dtype]), vals.to(TORCH[dtype])
        kv.append((keys.double(), vals.double()))
        for b in range(-(-total[s] // page)):
            pg = int(perm[s * blocks + b])
            table[s, b] = pg
            n = min(page, total[s] - b * page)
            cache[pg, 0, :, :n] = keys[b * page:b * page + n].transpose(0, 1).cuda()
            cache[pg, 1, :, :n] = vals[b * page:b * page + n].transpose(0, 1).cuda()
    table = table.cuda()
    for sink in (0.0, None):
        out = torch.zeros(t.rows, nqh * hd, dtype=TORCH[dtype], device="cuda")
        if kernel.startswith("simple"):
            K.attn_simple(q, out, cache, table, t.positions, t.token_seq, nqh, nkh, hd, page, window or None, scale, sink=sink,
                          out_scale=factor)
        elif kernel.startswith("tcgen05_prompt"):
            K.attn_tc(q, out, cache, table, t.q_start, t.q_len, t.kv_before, 2, max(lengths), nqh, nkh, hd, window or None, scale,
                      sink=sink, out_scale=factor)
        else:
            splits = {"mma_prompt": 1, "mma_few_1": 1, "mma_few_9": 9}[kernel]
            K.attn_mma(q, out, cache, table, t.q_start, t.q_len, t.kv_before, t.token_seq, 2, max(lengths), nqh, nkh, hd,
                       window or None, scale, n_splits=splits, few_tokens=few, sink=sink, out_scale=factor)
        K.check_device_errors()
        r0 = 0
        for s in range(2):
            qs = back(q[r0:r0 + lengths[s]]).view(-1, nqh, hd)
            pos = torch.arange(before[s], total[s])
            want = factor * plain_attention(qs, kv[s][0], kv[s][1], pos, total[s], window, scale, sink is not None, nkh)
            got = back(out[r0:r0 + lengths[s]]).view(-1, nqh, hd)
            assert (got - want).abs().max().item() < (3e-6 if dtype == "float32" else 2.5e-2), (kernel, window, sink, s)
            r0 += lengths[s]
    # with and without the sink the results differ by far more than the tolerance: the test can tell
    with_sink = plain_attention(qs, kv[1][0], kv[1][1], pos, total[1], window, scale, True, nkh)
    assert (with_sink - want / factor).abs().max().item() > 0.05


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps, C, stride, first", [(1, 21, 40, 3), (2, 21, 40, 3), (4, 21, 40, 3), (4, 48, 64, 8), (3, 16, 16, 0)])
def test_causal_convolution_in_steps_of_any_size_with_slots_used_again(K, dtype, taps, C, stride, first):
    """The last two cases allow aligned 16-byte loads and take the kernel that moves neighbouring channels together."""
    g = torch.Generator().manual_seed(taps)
    offset = 16
    w = dev(torch.randn(C, taps, generator=g), dtype)
    b = dev(torch.randn(C, generator=g), dtype)
    state_bytes = offset + (taps - 1) * C * 4 + 8
    state = torch.zeros(3, state_bytes, dtype=torch.uint8, device="cuda")
    for round_ in range(2):                                                 # the second round uses the slots again
        state[[2, 0]] = 0                                                   # as the cache manager does when a slot is taken
        xs = [dev(torch.randn(n, stride, generator=g), dtype) for n in (23, 9)]
        want = [P.silu(P.causal_conv(back(x)[:, first:first + C], back(w), back(b))) for x in xs]
        at = [0, 0]
        for cut in ([1, 2], [2, 1], [3, 1], [1, 0], [9, 5], [7, 0]):        # 0: the sequence sits this step out
            live = [i for i in range(2) if cut[i]]
            rows = torch.cat([xs[i][at[i]:at[i] + cut[i]] for i in live] + [torch.zeros(1, stride, dtype=TORCH[dtype], device="cuda")])
            t = step_tables([cut[i] for i in live], slots=[[2, 0][i] for i in live], pad=1)
            y = torch.zeros(t.rows, C, dtype=TORCH[dtype], device="cuda")
            K.causal_conv(rows[:, first:first + C], y, w, b, state, offset, t, silu=True)
            r = 0
            for i in live:
                assert rel(y[r:r + cut[i]], want[i][at[i]:at[i] + cut[i]]) < (2e-6 if dtype == "float32" else 1e-2), (round_, cut, i)
                r += cut[i]
                at[i] += cut[i]
        assert at == [23, 9]
    assert state[1].abs().sum() == 0 and state[:, :offset].abs().sum() == 0   # nothing outside the own part of the own slots


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode, heads, groups, dk, dv", [("channel", 3, 3, 24, 40), ("channel", 1, 1, 136, 8), ("channel", 2, 2, 8, 70),
                                                         ("head", 4, 2, 16, 24), ("head", 3, 1, 72, 33), ("head", 2, 2, 200, 5)])
def test_recurrence_whole_in_portions_and_token_by_token(K, dtype, mode, heads, groups, dk, dv):
    g = torch.Generator().manual_seed(dk + dv)
    lengths = [41, 7]
    tau = 4.0
    seqs = []
    for n in lengths:
        q = dev(torch.randn(n, groups * dk + 8, generator=g), dtype)         # views with a stride of their own
        k = dev(torch.randn(n, groups * dk, generator=g) * 0.5, dtype)
        v = dev(torch.randn(n, heads * dv + 3, generator=g), dtype)
        if mode == "channel":
            gate = (torch.randn(n, heads * dk, generator=g) * 2 + 2).cuda()
        else:
            gate = dev(torch.randn(n, heads + 2, generator=g), dtype)
        seqs.append((q, k, v, gate))
    if mode == "channel":
        bias = dev(torch.randn(heads * dk, generator=g), dtype)
        a_log = skip = None
    else:
        bias = dev(torch.randn(heads, generator=g), dtype)
        a_log, skip = dev(torch.randn(heads, generator=g) - 1, dtype), dev(torch.randn(heads, generator=g), dtype)
    hg = torch.arange(heads) // (heads // groups)

    def plain(q, k, v, gate):
        n = q.shape[0]
        q, k = back(q)[:, :groups * dk].view(n, groups, dk)[:, hg], back(k).view(n, groups, dk)[:, hg]
        v = back(v)[:, :heads * dv].view(n, heads, dv)
        S, out = torch.zeros(heads, dk, dv, dtype=D), torch.zeros(n, heads, dv, dtype=D)
        for t in range(n):
            if mode == "channel":
                a = torch.sigmoid(back(gate)[t].view(heads, dk) + back(bias).view(heads, dk)).pow(1 / tau)[:, :, None]
                S = a * S + k[t][:, :, None] * v[t][:, None, :]
                out[t] = (S * (q[t] * dk ** -0.5)[:, :, None]).sum(1)
            else:
                dt = P.softplus(back(gate)[t, :heads] + back(bias))
                a = torch.exp(-torch.exp(back(a_log)) * dt)[:, None, None]
                S = a * S + dt[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
                out[t] = (S * q[t][:, :, None]).sum(1) + back(skip)[:, None] * v[t]
        return out.reshape(n, heads * dv), S

    want = [plain(*s) for s in seqs]
    offset, sbytes = 32, 32 + heads * dk * dv * 4
    tol = 1e-5                                           # the recurrence itself is float32 in both runs: same inputs, same sums
    # the last walks go in chunks of 8 and of 16 tokens side by side (three passes) where a sequence brings two or more
    for cuts, chunk in (([[41, 7]], 0), ([[1, 1], [2, 2], [38, 4]], 0), ([[20, 0], [1, 7], [20, 0]], 0), ([[41, 7]], 8),
                        ([[3, 2], [38, 5]], 16)):
        state = torch.zeros(4, sbytes, dtype=torch.uint8, device="cuda")
        at = [0, 0]
        for cut in cuts:
            live = [i for i in range(2) if cut[i]]
            t = step_tables([cut[i] for i in live], slots=[[3, 1][i] for i in live], pad=2)
            cat = lambda j: torch.cat([seqs[i][j][at[i]:at[i] + cut[i]] for i in live] + [seqs[0][j][:2] * 0])      # noqa: E731
            q, k, v, gate = cat(0), cat(1), cat(2), cat(3)
            out = torch.zeros(t.rows, heads * dv, dtype=torch.float32, device="cuda")
            if mode == "channel":
                ready = chunk == 16                    # the decays computed once, in place, before the walk
                if ready:
                    gate = gate.clone()
                    K.scan_decay(gate, bias, 1 / tau)
                K.linear_scan(q[:, :groups * dk], k, v[:, :heads * dv], gate, bias, out, state, offset, t, heads, groups, dk, dv,
                              "channel", q_scale=dk ** -0.5, inv_tau=1 / tau, chunk=chunk, gate_is_decay=ready)
            else:
                K.linear_scan(q[:, :groups * dk], k, v[:, :heads * dv], gate[:, :heads], bias, out, state, offset, t, heads, groups,
                              dk, dv, "head", a_log=a_log, skip=skip, chunk=chunk)
            r = 0
            for i in live:
                assert rel(out[r:r + cut[i]], want[i][0][at[i]:at[i] + cut[i]]) < tol, (cuts, chunk, cut, i)
                r += cut[i]
                at[i] += cut[i]
        S = state[[3, 1], offset:].contiguous().view(torch.float32).view(2, heads, dk, dv)
        assert rel(S[0], want[0][1]) < tol and rel(S[1], want[1][1]) < tol
        assert state[[0, 2]].abs().sum() == 0 and state[:, :offset].abs().sum() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("gate_first, width, group, per_column", [(False, 120, 40, False), (True, 96, 48, True), (True, 35, 35, True),
                                                                  (False, 64, 8, False), (True, 600, 300, True), (False, 516, 258, False)])
def test_gated_norm_in_both_orders(K, dtype, gate_first, width, group, per_column):
    g = torch.Generator().manual_seed(width)
    rows = 9
    y = torch.randn(rows, width, generator=g).cuda()
    gate = dev(torch.randn(rows, width + 5, generator=g), dtype)
    w = dev(1 + 0.2 * torch.randn(width if per_column else group, generator=g), dtype)
    seq = torch.zeros(rows, dtype=torch.int32)
    seq[-1] = -1
    out = torch.zeros(rows, width, dtype=TORCH[dtype], device="cuda")
    K.gated_norm(y, gate[:, :width], w, out, seq.cuda(), group, gate_first, 1e-5, out_scale=0.7)
    sg = P.silu(back(gate)[:, :width])
    wv = back(w) if per_column else back(w).repeat(width // group)
    u = back(y) * sg if gate_first else back(y)
    n = P.rms(u.view(rows, width // group, group), 1e-5).reshape(rows, width) * wv
    want = 0.7 * (n if gate_first else n * sg)
    assert rel(out[:-1], want[:-1]) < (2e-6 if dtype == "float32" else 8e-3) and out[-1].abs().max() == 0


@pytest.mark.parametrize("rows", [5, 100, 300])
def test_gelu_in_the_epilogues_of_the_gated_product_and_beside_them(K, rows):
    from braidinfer_b200.csrc.api import interleave_gate_up
    g = torch.Generator().manual_seed(rows)
    k, inter = 64, 72
    x = torch.randn(rows, k, generator=g).to(torch.bfloat16).cuda()
    wg, wu = [(torch.randn(inter, k, generator=g) * 0.2).to(torch.bfloat16).cuda() for _ in range(2)]
    want = P.gelu_tanh(back(x) @ back(wg).T) * (back(x) @ back(wu).T)
    assert rel(P.gelu_tanh(torch.tensor([1.0], dtype=D)), torch.tensor([0.8411919906082768], dtype=D)) < 1e-12
    w = interleave_gate_up(wg, wu)
    for stream_k in (False, True):
        if stream_k and rows > 128:
            continue
        out = torch.zeros(rows, inter, dtype=torch.bfloat16, device="cuda")
        K.gemm_tc(x, w, out, swiglu=True, stream_k=stream_k, activation="gelu_tanh")
        assert rel(out, want) < 1e-2, stream_k
        K.gemm_tc(x, w, out, swiglu=True, stream_k=stream_k)                  # the default stays silu
        assert rel(out, P.silu(back(x) @ back(wg).T) * (back(x) @ back(wu).T)) < 1e-2
    for dtype in DTYPES:
        gu = dev(torch.cat([back(x) @ back(wg).T, back(x) @ back(wu).T], 1), dtype)
        out = torch.zeros(rows, inter, dtype=TORCH[dtype], device="cuda")
        K.act_mul(gu, out, "gelu_tanh")
        assert rel(out, P.gelu_tanh(back(gu)[:, :inter]) * back(gu)[:, inter:]) < (2e-6 if dtype == "float32" else 8e-3)
    K.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_table_gate_and_normed_sum(K, dtype):
    g = torch.Generator().manual_seed(1)
    rows, dim, vocab, width = 11, 12, 50, 100
    gate = dev(torch.randn(rows, dim + 4, generator=g), dtype)
    table = dev(torch.randn(vocab, 3 * dim, generator=g), dtype)
    ids = torch.randint(0, vocab, (rows,), generator=g).to(torch.int32)
    out = torch.zeros(rows, dim, dtype=TORCH[dtype], device="cuda")
    K.act_mul_gather(gate[:, :dim], table, ids.cuda(), 2 * dim, out, "gelu_tanh")
    want = P.gelu_tanh(back(gate)[:, :dim]) * back(table)[ids.long()][:, 2 * dim:]
    assert rel(out, want) < (2e-6 if dtype == "float32" else 8e-3)
    h0, y = torch.randn(rows, width, generator=g), torch.randn(rows, width, generator=g) * 3
    w = dev(1 + 0.2 * torch.randn(width, generator=g), dtype)
    h = h0.cuda().clone()
    K.rmsnorm_add(h, y.cuda(), w, 1e-5)
    assert rel(h, h0.double() + P.rms(y.double(), 1e-5, back(w))) < 2e-6


# ================================================================== the whole model through the engine
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts_and_every_layer(folders, oracles, name, dtype):
    eng = engine(folders[name], dtype)
    cfg = oracles[name].cfg
    tally = Tally(dtype)
    for n, seed in ((1, 0), (2, 1), (67, 2), (200, 3)):
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
            assert len(taps) == len(streams) == 1 + len(cfg["layers"])
            for i, (a, b) in enumerate(zip(taps, streams)):
                t2 = Tally(dtype)
                t2.add(a, b, (name, "after layer", i))
                t2.close()
    tally.close()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_token_by_token_from_the_first_token_equals_the_prompt_whole(folders, oracles, name, dtype):
    eng = engine(folders[name], dtype)
    toks = random_prompts(oracles[name].cfg["vocab"], [150], 7)[0]
    want = oracles[name].logits(toks)
    s, tally = eng.open(), Tally(dtype)
    for t, tok in enumerate(toks):
        tally.add(eng.step([(s, [tok])], want="last"), want[t:t + 1], t)
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, cuts", [("A", [2, 62, 1, 3, 64, 18]), ("A", [63, 2, 2, 83]), ("B", [128, 22]), ("A", [1, 1, 2, 146]),
                                        ("C", [2, 2, 2, 3, 141]), ("D", [5, 60, 64, 2, 19])])
def test_a_prompt_in_portions(folders, oracles, dtype, name, cuts):
    eng = engine(folders[name], dtype)
    toks = random_prompts(oracles[name].cfg["vocab"], [150], 9)[0]
    want = oracles[name].logits(toks)
    s, at, tally = eng.open(), 0, Tally(dtype)
    for c in cuts:
        tally.add(eng.step([(s, toks[at:at + c])], want="all"), want[at:at + c], (at, c))
        at += c
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_unequal_requests_in_one_batch_then_decoded_together_and_slots_used_again(folders, oracles, name, dtype):
    eng = engine(folders[name], dtype, max_tokens=64 * 12, max_slots=4)
    vocab = oracles[name].cfg["vocab"]
    prompts = random_prompts(vocab, [3 + 4, 70 + 9, 1 + 2, 129 + 12], 21)
    cut = [3, 70, 1, 129]
    want = [oracles[name].logits(p) for p in prompts]
    slots = [eng.open() for _ in prompts]
    lg = eng.step([(s, p[:c]) for s, p, c in zip(slots, prompts, cut)], want="all")
    off, tally = 0, Tally(dtype)
    for i, (p, c, w) in enumerate(zip(prompts, cut, want)):
        tally.add(lg[off:off + c], w[:c], ("prompt", i))
        off += c
    live, t = list(range(4)), 0
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
    # the freed slots (state areas) and pages serve other requests; what they held before must not show
    again = random_prompts(vocab, [66, 5], 22)
    slots = [eng.open(), eng.open()]
    lg = eng.step([(slots[0], again[0]), (slots[1], again[1])], want="all")
    tally.add(lg[:66], oracles[name].logits(again[0]), "slot used again")
    tally.add(lg[66:], oracles[name].logits(again[1]), "slot used again")
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "D"])
def test_long_decoding_across_page_borders_and_past_every_window(folders, oracles, name, dtype):
    eng = engine(folders[name], dtype)
    toks = random_prompts(oracles[name].cfg["vocab"], [5 + 215], 31)[0]
    want = oracles[name].logits(toks)
    s, tally = eng.open(), Tally(dtype)
    eng.step([(s, toks[:5])], want=None)
    for t in range(5, len(toks)):
        tally.add(eng.step([(s, [toks[t]])], want="last"), want[t:t + 1], t)
    tally.close()
    eng.check()
    if name == "A":
        assert eng.cache.pages_in_use() == [1, 2]          # windows of 7 and 70: the pages they have passed went back


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_token_far_back_still_counts_through_the_states_and_not_through_the_windows(folders, oracles, dtype):
    """Two prompts that differ in their first token only: 140 tokens on, beyond every window of configuration A,
    the logits still differ (the recurrent states carry the token), and the engine follows the plain
    implementation on both, whole and decoded."""
    cfg = oracles["A"].cfg
    a = random_prompts(cfg["vocab"], [150], 77)[0]
    b = [(a[0] + 1) % cfg["vocab"]] + a[1:]
    wa, wb = oracles["A"].logits(a), oracles["A"].logits(b)
    assert rel(wa[140:], wb[140:]) > 0.05
    eng = engine(folders["A"], dtype)
    for toks, want in ((a, wa), (b, wb)):
        s, tally = eng.open(), Tally(dtype)
        tally.add(eng.step([(s, toks[:130])], want="all"), want[:130])
        for t in range(130, 150):
            tally.add(eng.step([(s, [toks[t]])], want="last"), want[t:t + 1], t)
        tally.close()
        eng.close(s)
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_no_window_on_the_attention_through_a_hand_made_description(folders, oracles, dtype):
    """A model whose attention sees every earlier token (no mask in its description): the same parts, one group of
    full pages; decoding over a context long enough that the decode kernel slices it and merges, sink included."""
    from braidinfer_b200.config import read_config_json
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.models import architecture_for, complete_config
    from braidinfer_b200.weights import tensor_shapes
    cfg = complete_config(read_config_json(folders["D"]), tensor_shapes(folders["D"]))
    arch = architecture_for(cfg)
    spec = arch.build_spec(arch.config_from_dict(cfg))

    def without_window(mixer):
        left = mixer.params["left"]
        return dataclasses.replace(mixer, params={**mixer.params, "left": dataclasses.replace(left, params={**left.params, "window": None})})

    layers = tuple(dataclasses.replace(l, mixer=without_window(l.mixer)) for l in spec.layers)
    eng = Engine(None, folders["D"], dtype=dtype, max_tokens=64 * 12, verbose=False, spec=dataclasses.replace(spec, layers=layers))
    plain_cfg = json.loads(json.dumps(oracles["D"].cfg))
    for L in plain_cfg["layers"]:
        del L["mixer"]["left"]["mask"]
    toks = random_prompts(cfg["vocab"], [330], 41)[0]
    want = oracles["D"].logits(toks, plain_cfg)
    assert rel(want, oracles["D"].logits(toks)) > 0.05                  # the window matters here
    s, at, tally = eng.open(), 0, Tally(dtype)
    for c in [3, 250, 60] + [1] * 17:
        tally.add(eng.step([(s, toks[at:at + c])], want="all"), want[at:at + c], at)
        at += c
    tally.close()
    assert eng.cache.pages_in_use() == [6, 6]
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_configurations_drawn_from_a_seed(tmp_path, seed, dtype):
    """Other sizes, head counts, layer orders, windows and constants than any written by hand: a prompt in two
    portions beside a second request, then both decoded together, against the plain implementation."""
    cfg = random_config(seed)
    folder = make_loduzen_folder(tmp_path, f"r{seed}", cfg=cfg, seed=100 + seed)
    oracle = Oracle(folder)
    eng = engine(folder, dtype, max_tokens=64 * 8, max_slots=3)
    a, b = random_prompts(cfg["vocab"], [150, 21], seed)
    wa, wb = oracle.logits(a), oracle.logits(b)
    sa, sb, tally = eng.open(), eng.open(), Tally(dtype)
    tally.add(eng.step([(sa, a[:3])], want="all"), wa[:3], "first tokens")
    lg = eng.step([(sa, a[3:135]), (sb, b[:9])], want="all")
    tally.add(lg[:132], wa[3:135], "portion")
    tally.add(lg[132:], wb[:9], "beside it")
    for t in range(12):
        lg = eng.step([(sa, [a[135 + t]]), (sb, [b[9 + t]])], want="last")
        tally.add(lg[:1], wa[135 + t:136 + t], ("decoded", t))
        tally.add(lg[1:], wb[9 + t:10 + t], ("decoded beside", t))
    tally.close()
    eng.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_library_entry_point(folders, oracles, name, dtype):
    import braidinfer_b200 as lib
    model = lib.load(folders[name], dtype=dtype, max_seq_len=256, max_batch=3, verbose=False)
    prompts = random_prompts(oracles[name].cfg["vocab"], [4, 61, 17, 9], 51)          # four requests, three slots
    outs = model.generate(prompts, lib.SamplingParams.greedy(), stop_tokens=(), max_new_tokens=[6, 8, 3, 5])
    for p, o, n in zip(prompts, outs, [6, 8, 3, 5]):
        assert len(o.tokens) == n
        toks = list(p)
        for t in o.tokens:
            row = oracles[name].logits(toks)[-1]
            if dtype == "float32":
                assert t == P.argmax_lowest(row)
            else:
                assert row[t] >= row.max() - 2 * TOL[dtype] * row.abs().max()
            toks.append(t)
    model.engine.check()


def test_graphs_on_and_off_give_the_same_logits(folders, oracles):
    toks = random_prompts(oracles["A"].cfg["vocab"], [40], 5)[0]
    res = []
    for graphs in (True, False):
        eng = engine(folders["A"], "bfloat16", use_graphs=graphs)
        s = eng.open()
        out = [eng.step([(s, toks[:20])], want="last")]
        out += [eng.step([(s, [t])], want="last") for t in toks[20:]]
        res.append(torch.cat(out))
        if graphs:
            assert eng.graph_replays > 10
    assert torch.equal(res[0], res[1])


def test_trace_replay_program_on_a_model_folder(folders, oracles, tmp_path):
    toks = random_prompts(oracles["A"].cfg["vocab"], [40, 9], 61)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[0][:33], "want": [0, 32]}, {"id": "b", "tokens": toks[1][:8], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [toks[0][33]], "want": [0]}, {"id": "b", "tokens": [toks[1][8]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [toks[0][34]], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": toks[0][35:], "want": [4]}], "end": ["a"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps).encode(),
                       capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr.decode()[-2000:]
    assert [l for l in p.stdout.decode().split("\n") if l.startswith("done")] == [f"done {i}" for i in range(4)]
    import numpy as np
    vocab = oracles["A"].cfg["vocab"]
    wa, wb = oracles["A"].logits(toks[0]), oracles["A"].logits(toks[1])
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
