"""Besavik on the GPU: each new kernel alone against the plain function of its mechanism
(tests/plain_besavik.py), then whole models through replay, the engine and the command line."""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import besavik_helpers as bh
import plain_besavik as plain
from helpers import random_tokens, run_steps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, BF16, F64 = torch.float32, torch.bfloat16, torch.float64
DTYPES = [F32, BF16]


@pytest.fixture(scope="module")
def ops():
    from qwen_engine_b200 import ops as _ops
    _ops.lib()
    return _ops


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("besavik_gpu")
    return {name: bh.make_folder(str(root / name), name) for name in bh.BESAVIK}


def _close(got, want, dtype, what="", tol=None):
    got, want = got.detach().to("cpu", F64), want.to(F64)
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    tol = tol if tol is not None else {F32: 2e-5, BF16: 1.5e-2}[dtype]
    err = float((got - want).abs().max())
    scale = max(1e-6, float(want.abs().max()))
    assert err <= tol * scale, f"{what}: max |diff| {err:.3e} > {tol} * {scale:.3e}"


def _ctx(q_lens, ctx_lens, slots, plan=None):
    from qwen_engine_b200.parts.base import Arena
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(cu_q=i32(cu), ctx_lens=i32(ctx_lens), slot_ids=i32(slots), num_reqs=len(q_lens),
                           max_q_len=max(q_lens), q_lens_host=list(q_lens), ctx_lens_host=list(ctx_lens),
                           attn_plan=plan, arena=Arena(DEV))


# three steps that cut four unequal requests differently: (tokens of each request in the step)
CUTS = [[5, 1, 40, 2], [1, 33, 2, 0], [17, 1, 1, 9]]
SLOTS = [2, 0, 3, 1]


def _rows_of(cuts, r):
    """The flat rows of request r in each step, and the whole sequence's length."""
    return [(sum(step[:r]), step[r]) for step in cuts], sum(step[r] for step in cuts)


# ---- latent attention: what happens per token before the attention kernel ---------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dn,R,Dr,dims,P", [(3, 8, 24, 8, 8, 4), (1, 16, 16, 16, 8, 16), (2, 6, 10, 4, 4, 8), (8, 32, 64, 64, 64, 16),
                                              (2, 8, 8, 6, 0, 4)])
def test_latent_prepare(ops, dtype, H, dn, R, Dr, dims, P):
    g = torch.Generator().manual_seed(H * R + Dr)
    T, D, base = 21, R + Dr, 300.0
    wide = torch.randn(T, 5 + D + 3, generator=g).to(dtype)                 # the rows lie inside a wider product
    q = torch.randn(T, H * (dn + Dr), generator=g).to(dtype)
    norm_w = 1.0 + 0.2 * torch.randn(R, generator=g)
    positions = torch.randint(0, 3000, (T,), generator=g, dtype=torch.int32)
    inv_freq = (base ** (-2.0 * torch.arange(max(dims // 2, 1), dtype=F64) / max(dims, 1))).to(F32)
    n_pages = -(-T // P) + 1
    slots = torch.randperm(n_pages * P, generator=g)[:T].to(torch.int32)
    cache = torch.full((n_pages, 1, 1, P, D), 7.0, dtype=dtype, device=DEV)
    qlat = torch.full((T, H * D), 3.0, dtype=dtype, device=DEV)
    ops.latent_prepare(wide.to(DEV)[:, 5:5 + D], q.to(DEV), norm_w.to(DEV), 1e-5, positions.to(DEV), inv_freq.to(DEV), dims,
                       cache, slots.to(DEV), qlat, H, dn, R, Dr)
    down = wide[:, 5:5 + D].double()
    c = plain.rms_norm(down[:, :R], norm_w.double(), 1e-5)
    k_rot = plain.rotate_half_pairs(down[:, R:], positions, base, dims) if dims else down[:, R:]
    q_rot = q.double().reshape(T, H, dn + Dr)[:, :, dn:]
    q_rot = plain.rotate_half_pairs(q_rot, positions, base, dims) if dims else q_rot
    rows = cache.reshape(-1, D)[slots.long().to(DEV)]
    # angles are float32 products of positions in the thousands: 1e-4 of a radian is their rounding
    tol = {F32: 5e-4, BF16: 1.5e-2}[dtype]
    _close(rows[:, :R], c, dtype, "latent", tol={F32: 2e-5, BF16: 1.5e-2}[dtype])
    _close(rows[:, R:], k_rot, dtype, "rotated key part", tol=tol)
    _close(qlat.reshape(T, H, D)[:, :, R:], q_rot, dtype, "rotated query parts", tol=tol)
    assert bool((qlat.reshape(T, H, D)[:, :, :R] == 3.0).all())               # the room of the folded part is left alone
    untouched = torch.ones(n_pages * P, dtype=torch.bool)
    untouched[slots.long()] = False
    assert bool((cache.reshape(-1, D)[untouched.to(DEV)] == 7.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,H,N,K", [(1, 3, 24, 8), (7, 1, 16, 16), (70, 2, 10, 6), (130, 8, 64, 32), (65, 4, 96, 200), (33, 5, 129, 65)])
def test_a_product_with_one_matrix_per_head(ops, dtype, M, H, N, K):
    g = torch.Generator().manual_seed(M + N)
    xs, os_ = K + 3, N + 5                                                  # heads lie apart in their rows
    x = torch.randn(M, H * xs + 2, generator=g).to(dtype)
    w = (torch.randn(H, N, K, generator=g) / math.sqrt(K)).to(dtype)
    out = torch.full((M, H * os_), 9.0, dtype=dtype, device=DEV)
    ops.head_linear(x.to(DEV), w.to(DEV), out, xs, os_)
    xh = torch.stack([x[:, h * xs:h * xs + K] for h in range(H)], dim=1).double()
    want = torch.einsum("mhk,hnk->mhn", xh, w.double())
    got = out.reshape(M, H, os_)
    _close(got[:, :, :N], want, dtype, "head_linear")
    assert bool((got[:, :, N:] == 9.0).all())


def _latent_case(H, D, R, P, q_lens, ctx_lens, dtype, seed, spikes=()):
    g = torch.Generator().manual_seed(seed)
    n_req = len(q_lens)
    blocks = [-(-(c + n) // P) for c, n in zip(ctx_lens, q_lens)]
    n_pages = sum(blocks) + 2
    perm = iter(torch.randperm(n_pages, generator=g).tolist())
    table = torch.full((n_req, max(blocks)), -1, dtype=torch.int32)
    for r in range(n_req):
        for b in range(blocks[r]):
            table[r, b] = next(perm)
    cache = torch.randn(n_pages, 1, 1, P, D, generator=g).to(dtype)
    q = torch.randn(sum(q_lens), H * D, generator=g).to(dtype)
    for r, q_index, key_pos, head in spikes:
        # one key decides the row if it is seen: its score stands out by far, and its first channels are its value
        d = torch.randn(D, generator=g)
        d = d / d.norm()
        cache[int(table[r, key_pos // P]), 0, 0, key_pos % P] = (d * 8.0).to(dtype)
        q[sum(q_lens[:r]) + q_index, head * D:(head + 1) * D] = (d * 8.0 * math.sqrt(D)).to(dtype)
    return q, cache, table


def _plain_latent_rows(q, cache, table, H, D, R, P, q_lens, ctx_lens, scale):
    """Softmax attention over one shared key of D channels whose first R channels are the value."""
    out = torch.zeros(q.shape[0], H, R, dtype=F64)
    row = 0
    for r, (n, c) in enumerate(zip(q_lens, ctx_lens)):
        pos = torch.arange(c + n)
        keys = cache[table[r, pos // P].long(), 0, 0, pos % P].double()
        qs = q[row:row + n].double().reshape(n, H, D)
        zero = torch.zeros(n, H, 0, dtype=F64)
        out[row:row + n] = plain.latent_softmax(zero, qs, torch.zeros(c + n, H, 0, dtype=F64), keys,
                                                keys[:, None, :R].expand(c + n, H, R), scale, first=c)
        row += n
    return out


def _run_latent(ops, q, cache, table, H, D, P, q_lens, ctx_lens, scale, dtype, flash):
    from qwen_engine_b200.engine.runner import ModelRunner
    geo = (H, 1, D, 0, False, 1)
    geos = (geo,) if flash else ()
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, geos, dtype)
    devplan = ModelRunner._device_plan(plan, {"plan_" + k: torch.tensor(v, dtype=torch.int32, device=DEV) for k, v in plan.items()}, geos)
    ctx = _ctx(q_lens, ctx_lens, [0] * len(q_lens), devplan)
    out = torch.zeros(q.shape[0], H * D, dtype=dtype, device=DEV)
    ops.paged_attention(q.to(DEV), cache.to(DEV), table.to(DEV), ctx, out, scale, 0, H, 1, D)
    torch.cuda.synchronize()
    return out, ops.last_attention_kernel


LATENT_SHAPES = [(3, 32, 24, 4), (1, 48, 16, 16), (2, 14, 10, 8), (8, 128, 64, 16), (16, 256, 192, 16), (4, 80, 72, 16)]
LATENT_BATCHES = [([30], [0]), ([1], [95]), ([1, 1, 1], [4, 77, 31]), ([7, 1, 2, 40], [9, 40, 0, 63]), ([2, 33], [64, 31]), ([150], [20])]


@pytest.mark.parametrize("dtype,flash", [(F32, False), (BF16, False), (BF16, True)])
@pytest.mark.parametrize("H,D,R,P", LATENT_SHAPES)
@pytest.mark.parametrize("q_lens,ctx_lens", LATENT_BATCHES)
def test_attention_over_a_cache_of_one_plane(ops, dtype, flash, H, D, R, P, q_lens, ctx_lens):
    q, cache, table = _latent_case(H, D, R, P, q_lens, ctx_lens, dtype, H * D + len(q_lens))
    scale = 0.9 / math.sqrt(D)
    got, kernel = _run_latent(ops, q, cache, table, H, D, P, q_lens, ctx_lens, scale, dtype, flash)
    want = _plain_latent_rows(q, cache, table, H, D, R, P, q_lens, ctx_lens, scale)
    _close(got.reshape(-1, H, D)[:, :, :R], want, dtype, f"one plane on {kernel}", tol={F32: 2e-5, BF16: 2e-2}[dtype])
    if flash and D % 16 == 0:
        assert kernel != "paged_attention_generic" and kernel != "flash_attention_tc"


@pytest.mark.parametrize("dtype,flash", [(F32, False), (BF16, True)])
@pytest.mark.parametrize("H,D,R,P", [(4, 128, 96, 16), (2, 48, 40, 8)])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_far_key_among_hundreds_decides_the_row(ops, dtype, flash, H, D, R, P, decoded):
    """A key 700 tokens back, at a page's first place, whose score stands out: the row's output is that key's first
    channels, in a prompt's portion and for a decoded token; a causal mask that is off by one loses the key that is the
    query's own position."""
    far, own = 3 * P, 730
    q_lens, ctx_lens = ([1, 1], [own, own]) if decoded else ([40, 731], [own - 39, 0])
    q_index = 0 if decoded else q_lens[0] - 1
    # request 0: the far key; request 1: the key at the query's own position
    spikes = [(0, q_index, far, 1), (1, q_lens[1] - 1, own, 0)]
    q, cache, table = _latent_case(H, D, R, P, q_lens, ctx_lens, dtype, 5, spikes)
    scale = 1.0 / math.sqrt(D)
    got, kernel = _run_latent(ops, q, cache, table, H, D, P, q_lens, ctx_lens, scale, dtype, flash)
    want = _plain_latent_rows(q, cache, table, H, D, R, P, q_lens, ctx_lens, scale)
    _close(got.reshape(-1, H, D)[:, :, :R], want, dtype, f"far key on {kernel}", tol={F32: 2e-5, BF16: 2e-2}[dtype])
    rows = got.reshape(-1, H, D).float().cpu()
    key_far = cache[int(table[0, far // P]), 0, 0, far % P, :R].float()
    key_own = cache[int(table[1, own // P]), 0, 0, own % P, :R].float()
    assert float((rows[q_index, 1, :R] - key_far).abs().max()) < 0.05
    assert float((rows[-1, 0, :R] - key_own).abs().max()) < 0.05


# ---- the short convolution ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,taps", [(5, 1), (40, 2), (130, 4), (24, 5), (300, 16)])
def test_short_convolution_in_portions_through_used_slots(ops, dtype, C, taps):
    g = torch.Generator().manual_seed(C + taps)
    w = torch.randn(C, taps, generator=g)
    state = torch.full((4, taps - 1, C), 50.0, device=DEV)                  # what other requests left in the slots
    seqs = [torch.randn(_rows_of(CUTS, r)[1], C + 4, generator=g).to(dtype) for r in range(4)]
    done = [0] * 4
    got = [[] for _ in range(4)]
    for step in CUTS:
        live = [r for r in range(4) if step[r] > 0]
        x = torch.cat([seqs[r][done[r]:done[r] + step[r]] for r in live]).to(DEV)
        ctx = _ctx([step[r] for r in live], [done[r] for r in live], [SLOTS[r] for r in live])
        out = torch.empty(x.shape[0], C, dtype=F32, device=DEV)
        ops.short_conv(x[:, 2:2 + C], w.to(DEV), state, ctx, out)
        row = 0
        for r in live:
            got[r].append(out[row:row + step[r]].cpu())
            row += step[r]
            done[r] += step[r]
    for r in range(4):
        y = plain.short_conv(seqs[r][:, 2:2 + C].double(), w.double())
        _close(torch.cat(got[r]), torch.nn.functional.silu(y), F32, f"request {r}", tol=3e-6)
        if taps > 1:
            tail = seqs[r][:, 2:2 + C].float()[-(taps - 1):]
            assert torch.equal(state[SLOTS[r]].cpu()[-tail.shape[0]:], tail)


def test_unit_norm_of_heads_inside_wider_rows(ops):
    g = torch.Generator().manual_seed(1)
    for H, D in [(1, 7), (3, 24), (2, 128), (5, 6)]:
        wide = torch.randn(11, H * D + 9, generator=g)
        dev = wide.to(DEV)
        ops.unit_norm(dev[:, 4:4 + H * D], H, D, 1e-6, 0.3)
        x = wide[:, 4:4 + H * D].double().reshape(11, H, D)
        want = x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6) * 0.3
        _close(dev[:, 4:4 + H * D].reshape(11, H, D), want, F32, "unit norm", tol=3e-6)
        assert torch.equal(dev[:, :4].cpu(), wide[:, :4]) and torch.equal(dev[:, 4 + H * D:].cpu(), wide[:, 4 + H * D:])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,dk,R", [(1, 2, 4, 1), (19, 5, 40, 3), (40, 3, 43, 16), (5, 4, 96, 64)])
def test_decay_from_a_rate_and_a_softplus(ops, dtype, T, H, dk, R):
    g = torch.Generator().manual_seed(T + dk)
    N = H * dk
    wide = torch.randn(T, R + 5, generator=g).to(dtype)
    w = (torch.randn(N, R, generator=g) * 2).to(dtype)
    bias = torch.randn(N, generator=g) * 3
    bias[0], bias[-1] = 30.0, -30.0                                          # both ends of the softplus
    log_rate = torch.randn(H, generator=g)
    out = torch.empty(T, N, dtype=F32, device=DEV)
    ops.channel_decay(wide.to(DEV)[:, 3:3 + R], w.to(DEV), bias.to(DEV), 1.0, out, log_rate=log_rate.to(DEV))
    z = wide[:, 3:3 + R].double() @ w.double().T + bias.double()
    want = torch.exp(-torch.exp(log_rate.double()).repeat_interleave(dk)[None, :] * torch.nn.functional.softplus(z))
    _close(out, want, F32, "decay", tol=5e-6)
    assert float(out.min()) >= 0.0 and float(out.max()) <= 1.0


# ---- the recurrences ---------------------------------------------------------------------------------------------
DELTA_SHAPES = [(4, 2, 8, 12), (2, 2, 16, 16), (3, 1, 6, 10), (4, 2, 128, 64), (2, 1, 64, 128), (1, 1, 256, 20), (6, 3, 32, 7)]


def _delta_inputs(H, G, dk, dv, T, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    wide = torch.randn(T, 2 * G * dk + H * dv + 6, generator=g)              # q, k, v side by side, as the convolution leaves them
    q, k = wide[:, 1:1 + G * dk], wide[:, 1 + G * dk:1 + 2 * G * dk]
    q /= q.reshape(T, G, dk).norm(dim=-1).repeat_interleave(dk, dim=1)
    k /= k.reshape(T, G, dk).norm(dim=-1).repeat_interleave(dk, dim=1)
    decay = torch.rand(T, H * dk, generator=g) * 0.6 + 0.4
    beta = (torch.randn(T, H + 3, generator=g) * 2).to(dtype)
    return wide, decay, beta


def _plain_delta(wide, decay, beta, H, G, dk, dv):
    T = wide.shape[0]
    rep = H // G
    q = wide[:, 1:1 + G * dk].double().reshape(T, G, dk).repeat_interleave(rep, dim=1)
    k = wide[:, 1 + G * dk:1 + 2 * G * dk].double().reshape(T, G, dk).repeat_interleave(rep, dim=1)
    v = wide[:, 1 + 2 * G * dk:1 + 2 * G * dk + H * dv].double().reshape(T, H, dv)
    return plain.delta_recurrence(q, k, v, decay.double().reshape(T, H, dk), torch.sigmoid(beta[:, 2:2 + H].double()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dk,dv", DELTA_SHAPES)
def test_delta_rule_of_unequal_requests_in_portions(ops, dtype, H, G, dk, dv):
    state = torch.full((4, H, dv, dk), 9.0, device=DEV)                      # what other requests left in the slots
    ins = [_delta_inputs(H, G, dk, dv, _rows_of(CUTS, r)[1], 10 * r + dk, dtype) for r in range(4)]
    done = [0] * 4
    got = [[] for _ in range(4)]
    qk = G * dk
    for step in CUTS:
        live = [r for r in range(4) if step[r] > 0]
        cat = lambda i: torch.cat([ins[r][i][done[r]:done[r] + step[r]] for r in live]).to(DEV)
        wide, decay, beta = cat(0), cat(1), cat(2)
        ctx = _ctx([step[r] for r in live], [done[r] for r in live], [SLOTS[r] for r in live])
        out = torch.empty(wide.shape[0], H * dv, dtype=F32, device=DEV)
        ops.delta_rule_scan(wide[:, 1:1 + qk], wide[:, 1 + qk:1 + 2 * qk], wide[:, 1 + 2 * qk:1 + 2 * qk + H * dv], decay,
                            beta[:, 2:2 + H], state, ctx, out, H, G, dk, dv)
        row = 0
        for r in live:
            got[r].append(out[row:row + step[r]].cpu())
            row += step[r]
            done[r] += step[r]
    for r in range(4):
        o, S = _plain_delta(*ins[r], H, G, dk, dv)
        _close(torch.cat(got[r]).reshape(-1, H, dv), o, F32, f"request {r}", tol=2e-5)
        _close(state[SLOTS[r]], S.transpose(1, 2), F32, f"state of request {r}", tol=2e-5)


def test_delta_rule_long_whole_and_token_by_token_to_the_bit(ops):
    H, G, dk, dv, T = 2, 1, 64, 32, 700
    wide, decay, beta = _delta_inputs(H, G, dk, dv, T, 3, F32)
    decay[:, :dk] = 1.0                                  # a head that forgets nothing: the first tokens stay in its state
    qk = G * dk
    dev = lambda t: t.to(DEV)
    w, d, b = dev(wide), dev(decay), dev(beta)
    args = lambda a, z: (w[a:z, 1:1 + qk], w[a:z, 1 + qk:1 + 2 * qk], w[a:z, 1 + 2 * qk:1 + 2 * qk + H * dv], d[a:z], b[a:z, 2:2 + H])
    state = torch.zeros(1, H, dv, dk, device=DEV)
    whole = torch.empty(T, H * dv, dtype=F32, device=DEV)
    ops.delta_rule_scan(*args(0, T), state, _ctx([T], [0], [0]), whole, H, G, dk, dv)
    o, S = _plain_delta(wide, decay, beta, H, G, dk, dv)
    _close(whole.reshape(T, H, dv), o, F32, "700 tokens", tol=5e-5)
    state2 = torch.full((1, H, dv, dk), 4.0, device=DEV)
    single = torch.empty(T, H * dv, dtype=F32, device=DEV)
    for t in range(T):
        ops.delta_rule_scan(*args(t, t + 1), state2, _ctx([1], [t], [0]), single[t:t + 1], H, G, dk, dv)
    assert torch.equal(single, whole) and torch.equal(state, state2)
    # a state that is only read stays as it was
    before = state.clone()
    ops.delta_rule_scan(*args(0, 9), state, _ctx([9], [T], [0]), single[:9], H, G, dk, dv, write_state=False)
    assert torch.equal(state, before)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dk,dv", [(2, 32, 64), (1, 10, 6), (4, 8, 8), (2, 64, 128), (3, 128, 40)])
def test_linear_attention_with_one_decay_per_head(ops, dtype, H, dk, dv):
    decays = torch.tensor([1.0, 0.999, 0.6, 0.0][:H], dtype=F32)
    g = torch.Generator().manual_seed(dk)
    seqs = [torch.randn(_rows_of(CUTS, r)[1], 2 * H * dk + H * dv + 3, generator=g).to(dtype) for r in range(4)]
    state = torch.full((4, H, dv, dk), 9.0, device=DEV)
    done = [0] * 4
    got = [[] for _ in range(4)]
    kw = H * dk
    for step in CUTS:
        live = [r for r in range(4) if step[r] > 0]
        wide = torch.cat([seqs[r][done[r]:done[r] + step[r]] for r in live]).to(DEV)
        ctx = _ctx([step[r] for r in live], [done[r] for r in live], [SLOTS[r] for r in live])
        out = torch.empty(wide.shape[0], H * dv, dtype=F32, device=DEV)
        ops.linear_attention_scan(wide[:, 1:1 + kw], wide[:, 1 + kw:1 + 2 * kw], wide[:, 1 + 2 * kw:1 + 2 * kw + H * dv], None, state,
                                  ctx, out, 1.0, H, dk, dv, head_decay=decays.to(DEV))
        row = 0
        for r in live:
            got[r].append(out[row:row + step[r]].cpu())
            row += step[r]
            done[r] += step[r]
    for r in range(4):
        T = seqs[r].shape[0]
        x = seqs[r].double()
        o, S = plain.decayed_recurrence(x[:, 1:1 + kw].reshape(T, H, dk), x[:, 1 + kw:1 + 2 * kw].reshape(T, H, dk),
                                        x[:, 1 + 2 * kw:1 + 2 * kw + H * dv].reshape(T, H, dv), decays.double())
        _close(torch.cat(got[r]).reshape(T, H, dv), o, F32, f"request {r}", tol=2e-5)
        _close(state[SLOTS[r]], S.transpose(1, 2), F32, f"state of request {r}", tol=2e-5)


# ---- routed experts and the limited feed-forward -----------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,E,top", [(1, 40, 2, 1), (9, 64, 5, 2), (70, 96, 8, 3), (33, 50, 200, 8), (5, 32, 4, 4)])
def test_router(ops, dtype, T, W, E, top):
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g).to(dtype)
    w = torch.randn(E, W, generator=g)
    bias = torch.randn(E, generator=g)
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wgt = torch.empty(T, top, dtype=F32, device=DEV)
    ops.moe_route(x.to(DEV), w.to(DEV), bias.to(DEV), idx, wgt)
    want_idx, want_w = plain.route(x.double(), w.double(), bias.double(), top)
    assert torch.equal(idx.cpu().long(), want_idx)
    _close(wgt, want_w, F32, "weights", tol=1e-5)


def _plain_experts(x, idx, wgt, w_gate_up, w_down, limit):
    I = w_gate_up.shape[1] // 2
    out = torch.zeros(x.shape[0], w_down.shape[1], dtype=F64)
    for t in range(x.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wgt[t, j] * plain.limited_glu(x[t:t + 1].double(), w_gate_up[e, :I].double(), w_gate_up[e, I:].double(),
                                                    w_down[e].double(), limit)[0]
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,I,E,top,limit", [(1, 40, 12, 2, 1, 3.0), (9, 64, 24, 5, 2, 0.8), (300, 96, 70, 3, 2, 1.0), (70, 128, 64, 16, 4, 0.5),
                                               (5, 32, 16, 4, 4, 2.0), (130, 50, 33, 6, 1, 1.0), (9, 64, 520, 4, 2, 1.0), (40, 128, 1536, 8, 2, 4.0)])
def test_experts_with_many_few_and_no_tokens(ops, dtype, T, W, I, E, top, limit):
    from qwen_engine_b200.parts.base import Arena
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g).to(dtype)
    w_gate_up = (torch.randn(E, 2 * I, W, generator=g) / math.sqrt(W) * 2).to(dtype)
    w_down = (torch.randn(E, W, I, generator=g) / math.sqrt(I)).to(dtype)
    # choices that leave the last expert without a token where there are enough experts, and pile many on the first
    allowed = E - 1 if E > top else E
    rows = []
    for t in range(T):
        perm = torch.randperm(allowed, generator=g)[:top].tolist()
        if t < T // 2 and 0 not in perm:
            perm[0] = 0
        rows.append(perm)
    idx = torch.tensor(rows, dtype=torch.int32)
    wgt = torch.softmax(torch.randn(T, top, generator=g), dim=-1)
    out = torch.empty(T, W, dtype=dtype, device=DEV)
    arena = Arena(DEV, 1 << 24)
    ops.moe_experts(x.to(DEV), idx.to(DEV), wgt.to(DEV), w_gate_up.to(DEV), w_down.to(DEV), out, ("swish_limit", limit), arena.alloc)
    want = _plain_experts(x, idx, wgt.double(), w_gate_up, w_down, limit)
    _close(out, want, dtype, "experts", tol={F32: 2e-5, BF16: 2e-2}[dtype])
    # a token's row does not depend on what else is in the batch: the first token alone and among a few, to the bit (steps
    # of many rows add up the down product's K in one piece, steps of a few in shares: those differ by rounding)
    n = min(T, 7)
    few = torch.empty(n, W, dtype=dtype, device=DEV)
    ops.moe_experts(x[:n].to(DEV), idx[:n].to(DEV), wgt[:n].to(DEV), w_gate_up.to(DEV), w_down.to(DEV), few, ("swish_limit", limit), arena.alloc)
    alone = torch.empty(1, W, dtype=dtype, device=DEV)
    ops.moe_experts(x[:1].to(DEV), idx[:1].to(DEV), wgt[:1].to(DEV), w_gate_up.to(DEV), w_down.to(DEV), alone, ("swish_limit", limit), arena.alloc)
    assert torch.equal(alone[0], few[0])
    _close(few, want[:n], dtype, "a few rows", tol={F32: 2e-5, BF16: 2e-2}[dtype])
    if T * top <= 256 or dtype == F32:
        assert torch.equal(few, out[:n])


@pytest.mark.parametrize("dtype", DTYPES)
def test_limited_activation_alone(ops, dtype):
    g = torch.Generator().manual_seed(2)
    for T, I, limit in [(3, 24, 1.0), (17, 130, 0.4), (64, 512, 7.0)]:
        gate_up = (torch.randn(T, 2 * I, generator=g) * 3).to(dtype)
        out = torch.empty(T, I, dtype=dtype, device=DEV)
        ops.act_mul(gate_up.to(DEV), out, ("swish_limit", limit))
        gv, uv = gate_up[:, :I].double().clamp(max=limit), gate_up[:, I:].double().clamp(-limit, limit)
        _close(out, gv * torch.sigmoid(1.702 * gv) * (uv + 1.0), dtype, "limited", tol={F32: 2e-6, BF16: 8e-3}[dtype])


@pytest.mark.parametrize("M,I,K", [(3, 96, 64), (16, 3072, 1024), (1200, 3072, 512)])
def test_gate_up_products_with_the_limited_form_in_their_epilogue(ops, M, I, K):
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).to(BF16)
    w = (torch.randn(2 * I, K, generator=g) / math.sqrt(K) * 2).to(BF16)
    limit = 1.25
    gate_up = (x.double() @ w.double().T).to(BF16).double()
    gv, uv = gate_up[:, :I].clamp(max=limit), gate_up[:, I:].clamp(-limit, limit)
    want = gv * torch.sigmoid(1.702 * gv) * (uv + 1.0)
    out = torch.empty(M, I, dtype=BF16, device=DEV)
    if M <= 16:
        ops.linear_swiglu_small(x.to(DEV), w.to(DEV), out, ("swish_limit", limit))
    else:
        ops.linear_swiglu(x.to(DEV), w.to(DEV), out, ("swish_limit", limit))
    _close(out, want, BF16, "fused", tol=2e-2)


# ---- whole models ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,name", [(d, n) for n in bh.BESAVIK for d in DTYPES])
def test_replay_against_the_plain_model(folders, dtype, name):
    folder = folders[name]
    bh.replay_cases(lambda n: bh.make_replayer(folder, name, dtype, n, poison=1.0e4), folder, name, dtype, f"{name}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_every_position_of_a_long_prompt_whole_and_decoded(folders, dtype):
    """Prompts of several pages at all positions: whole, and from the first token on one by one (the steps of single
    tokens are replayed from a CUDA graph): first tokens and pages' borders lie among them, in prompts and in decoding."""
    for name, n in (("b-b", 120), ("b-d", 330)):
        folder = folders[name]
        toks = random_tokens(bh.vocab_of(name), n, 31)
        whole = [{"entries": [{"id": "a", "tokens": toks, "want": list(range(n))}], "end": ["a"]}]
        bh.check_requests(run_steps(bh.make_replayer(folder, name, dtype, 384), whole), folder, {"a": toks}, dtype, f"{name} whole")
        single = [{"entries": [{"id": "a", "tokens": [t], "want": [0]}]} for t in toks]
        rep = bh.make_replayer(folder, name, dtype, 384)
        bh.check_requests(run_steps(rep, single), folder, {"a": toks}, dtype, f"{name} decoded")
        assert rep.runner.num_graph_replays > n // 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_in_portions_then_decoded(folders, dtype):
    """600 tokens: whole; and in portions of changing sizes (two tokens among them, cuts inside pages) with the last 40
    tokens one by one, beside a second request that comes and goes (its slot and pages are used again)."""
    name = "b-d"
    folder = folders[name]
    V = bh.vocab_of(name)
    toks, other = random_tokens(V, 600, 3), random_tokens(V, 50, 4)
    want = sorted(set(range(0, 600, 7)) | set(range(560, 600)))
    whole = [{"entries": [{"id": "a", "tokens": toks, "want": want}], "end": ["a"]}]
    bh.check_requests(run_steps(bh.make_replayer(folder, name, dtype, 640), whole), folder, {"a": toks}, dtype, "whole")
    steps, p = [], 0
    for i, n in enumerate([64, 64, 100, 2, 30, 129, 16, 3, 95, 57] + [1] * 40):
        entries = [{"id": "a", "tokens": toks[p:p + n], "want": [w - p for w in want if p <= w < p + n]}]
        if i in (1, 5, 12):
            entries.append({"id": f"b{i}", "tokens": other, "want": [49]})
        steps.append({"entries": entries, "end": [f"b{i}"] if i in (1, 5, 12) else []})
        p += n
    assert p == 600
    rep = bh.make_replayer(folder, name, dtype, 704)
    got = run_steps(rep, steps)
    bh.check_requests(got, folder, {"a": toks, "b1": other, "b5": other, "b12": other}, dtype, "portions")


def test_greedy_generation_through_the_engine(folders):
    from qwen_engine_b200.sampling.params import SamplingParams
    for name in ("b-a", "b-c"):
        folder = folders[name]
        cfg, w = bh.plain_model(folder)
        V = bh.vocab_of(name)
        prompts = [random_tokens(V, n, 40 + i) for i, n in enumerate([5, 19, 33, 2, 11, 26, 47])]
        eng = bh.make_engine(folder, name, F32, max_num_seqs=3, max_num_batched_tokens=24, prefill_chunk_size=7)
        ids = [eng.add_request(p, SamplingParams(max_new_tokens=8, temperature=0.0)) for p in prompts]
        outs = {o.request_id: o for o in eng.serving()}
        for rid, p in zip(ids, prompts):
            assert list(outs[rid].output_token_ids) == plain.greedy(cfg, w, p, 8), f"{name}: prompt of {len(p)} tokens"
        assert eng.cache.slots.num_free == eng.cache.slots.num_slots and eng.cache.pages_in_use() == 0


def test_the_command_line_replays_a_trace(folders, tmp_path):
    name = "b-c"
    folder = folders[name]
    toks = random_tokens(bh.vocab_of(name), 30, 8)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:21], "want": [0, 20]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[21:23], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[23:], "want": [6]}, {"id": "y", "tokens": toks[:4], "want": [3]}],
              "end": ["x", "y"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    V = bh.vocab_of(name)
    want = bh.plain_logits(folder, toks)
    first = torch.frombuffer(bytearray((out / "0.f32").read_bytes()), dtype=F32).reshape(-1, V)
    last = torch.frombuffer(bytearray((out / "2.f32").read_bytes()), dtype=F32).reshape(-1, V)
    bh.assert_close_rows(first, want[[0, 20]], F32, "step 0")
    bh.assert_close_rows(last, torch.stack([want[29], want[3]]), F32, "step 2")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_alone_shares_the_pages_of_equal_prefixes(folders, dtype):
    """A model of latent attention alone keeps no state of fixed size, so a second request with the same first tokens takes
    the first one's pages in both groups of pages (a prompt found whole gets a private copy of its last page)."""
    name = "b-f"
    folder = folders[name]
    V = bh.vocab_of(name)
    first = random_tokens(V, 40, 5)
    second = first[:24] + random_tokens(V, 10, 6)
    rep = bh.make_replayer(folder, name, dtype, 256)
    assert rep.cache.prefix_cache and len(rep.cache.paged_groups) == 2
    steps = [{"entries": [{"id": "a", "tokens": first, "want": [39]}]},
             {"entries": [{"id": "b", "tokens": second, "want": [30, 33]}, {"id": "c", "tokens": first, "want": [39]}], "end": ["a", "b", "c"]}]
    got = run_steps(rep, steps)
    assert rep.cache.prefix_hit_tokens == 24 + 39
    bh.check_requests(got, folder, {"a": first, "b": second, "c": first}, dtype, "shared prefix")
