"""Ganidra on the GPU: each new kernel alone against the plain function of its mechanism
(tests/plain_ganidra.py), then whole models through replay, the engine and the command line."""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import ganidra_helpers as gh
import plain_ganidra as plain
from helpers import TOL, random_tokens, run_steps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, BF16 = torch.float32, torch.bfloat16
DTYPES = [F32, BF16]


@pytest.fixture(scope="module")
def ops():
    from qwen_engine_b200 import ops as _ops
    _ops.lib()
    return _ops


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("ganidra_gpu")
    return {name: gh.make_folder(str(root / name), name) for name in gh.GANIDRA}


def _close(got, want, dtype, what="", tol=None):
    got, want = got.detach().to("cpu", torch.float64), want.to(torch.float64)
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


# ---- the decay ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,N,R,tau", [(1, 8, 1, 1.0), (19, 200, 3, 16.0), (40, 129, 16, 4.0), (5, 384, 64, 0.5)])
def test_channel_decay(ops, dtype, T, N, R, tau):
    g = torch.Generator().manual_seed(T + N)
    wide = torch.randn(T, R + 5, generator=g).to(dtype)              # the rank's columns lie inside a wider product
    a = wide[:, 3:3 + R]
    w = (torch.randn(N, R, generator=g) * 2).to(dtype)
    bias = torch.randn(N, generator=g) * 3
    bias[0], bias[-1] = 40.0, -40.0                                    # both ends of the sigmoid
    out = torch.empty(T, N, dtype=F32, device=DEV)
    ops.channel_decay(wide.to(DEV)[:, 3:3 + R], w.to(DEV), bias.to(DEV), tau, out)
    want = plain.channel_decay(a.double(), torch.eye(R, dtype=torch.float64), w.double(), bias.double(), tau)
    _close(out, want, F32, "decay", tol=3e-6)
    assert float(out.min()) >= 0.0 and float(out.max()) <= 1.0


# ---- the recurrence ----------------------------------------------------------------------------------------
def _scan_inputs(H, dk, dv, T, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    wide = torch.randn(T, 2 * H * dk + H * dv + 3, generator=g).to(dtype)      # q, k, v side by side in one product's rows
    alpha = torch.rand(T, H * dk, generator=g) * 0.5 + 0.5
    return wide, alpha


def _plain_scan(wide, alpha, H, dk, dv, q_scale, rows):
    q, k, v = wide[rows, :H * dk].double() * q_scale, wide[rows, H * dk:2 * H * dk].double(), wide[rows, 2 * H * dk:2 * H * dk + H * dv].double()
    a = alpha[rows].double()
    return torch.cat([plain.linear_attention_recurrence(q[:, h * dk:(h + 1) * dk], k[:, h * dk:(h + 1) * dk],
                                                        v[:, h * dv:(h + 1) * dv], a[:, h * dk:(h + 1) * dk])
                      for h in range(H)], dim=1)


SCAN_SHAPES = [(1, 10, 7), (2, 16, 24), (3, 128, 128), (1, 256, 64), (2, 64, 200), (5, 4, 4), (1, 48, 96), (1, 512, 8), (1, 1024, 4)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dk,dv", SCAN_SHAPES)
def test_scan_of_unequal_requests_in_portions(ops, dtype, H, dk, dv):
    """Four requests of unequal lengths run as one batch, in three steps cut at other places for each, with
    slots that held another request's state before: against the recurrence of each request alone."""
    lens = [37, 1, 64, 18]
    cuts = [[5, 30, 2], [1, 0, 0], [62, 1, 1], [2, 2, 14]]
    slots = [3, 0, 5, 1]
    T = sum(lens)
    wide, alpha = _scan_inputs(H, dk, dv, T, dtype, 100 * H + dk)
    starts = [sum(lens[:r]) for r in range(4)]
    state = torch.full((6, H, dv, dk), 7.5, dtype=F32, device=DEV)            # what an earlier request left behind
    got = torch.zeros(T, H * dv, dtype=F32)
    done = [0] * 4
    q_scale = dk ** -0.5
    for step in range(3):
        live = [r for r in range(4) if cuts[r][step] > 0]
        rows = [i for r in live for i in range(starts[r] + done[r], starts[r] + done[r] + cuts[r][step])]
        sub, al = wide[rows].to(DEV), alpha[rows].contiguous().to(DEV)
        out = torch.empty(len(rows), H * dv, dtype=F32, device=DEV)
        ctx = _ctx([cuts[r][step] for r in live], [done[r] for r in live], [slots[r] for r in live])
        ops.linear_attention_scan(sub[:, :H * dk], sub[:, H * dk:2 * H * dk], sub[:, 2 * H * dk:2 * H * dk + H * dv], al, state,
                                  ctx, out, q_scale, H, dk, dv)
        got[rows] = out.cpu()
        for r in live:
            done[r] += cuts[r][step]
    assert done == lens
    for r in range(4):
        rows = list(range(starts[r], starts[r] + lens[r]))
        _close(got[rows], _plain_scan(wide, alpha, H, dk, dv, q_scale, rows), F32, f"request {r}", tol=2e-5)
    assert float(state[2].min()) == 7.5 and float(state[4].max()) == 7.5     # slots nobody holds are not touched


def test_scan_long_and_a_state_that_is_read_only(ops):
    """700 tokens in one step against the same tokens one by one (to the bit: the order of every sum is the
    sizes' alone), a far token that one channel never forgets, and a run that leaves the state as it was."""
    H, dk, dv, T = 2, 32, 40, 700
    wide, alpha = _scan_inputs(H, dk, dv, T, F32, 5)
    alpha[:, 3] = 1.0                                   # channel 3 of head 0 keeps everything
    alpha[:, 4:dk] = 0.3                                # its neighbours forget at once
    wide[2, H * dk + 3] = 500.0                         # k of token 2, channel 3: a far key among hundreds
    wide[T - 1, 3] = 20.0                               # the last query asks for channel 3
    q_scale = dk ** -0.5
    args = lambda t: (t[:, :H * dk], t[:, H * dk:2 * H * dk], t[:, 2 * H * dk:2 * H * dk + H * dv])
    whole = torch.empty(T, H * dv, dtype=F32, device=DEV)
    state = torch.zeros(2, H, dv, dk, dtype=F32, device=DEV)
    ops.linear_attention_scan(*args(wide.to(DEV)), alpha.to(DEV), state, _ctx([T], [0], [1]), whole, q_scale, H, dk, dv)
    want = _plain_scan(wide, alpha, H, dk, dv, q_scale, list(range(T)))
    _close(whole, want, F32, "long", tol=2e-5)
    far = 500.0 * wide[2, 2 * H * dk:2 * H * dk + dv].double() * 20.0 * q_scale
    assert float((want[T - 1, :dv] - far).abs().max()) < 0.2 * float(far.abs().max())      # the far token decides the last output
    single = torch.empty(T, H * dv, dtype=F32, device=DEV)
    state2 = torch.zeros(2, H, dv, dk, dtype=F32, device=DEV)
    w_dev, a_dev = wide.to(DEV), alpha.to(DEV)
    for t in range(T):
        ops.linear_attention_scan(*args(w_dev[t:t + 1]), a_dev[t:t + 1], state2, _ctx([1], [t], [0]), single[t:t + 1], q_scale, H, dk, dv)
    assert torch.equal(single, whole) and torch.equal(state2[0], state[1])
    before = state.clone()
    ops.linear_attention_scan(*args(w_dev[:9]), a_dev[:9], state, _ctx([9], [T], [1]), single[:9], q_scale, H, dk, dv, write_state=False)
    assert torch.equal(state, before)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dk,dv,R", [(2, 16, 24, 3), (3, 128, 64, 16), (1, 10, 7, 1), (4, 64, 128, 32)])
def test_scan_of_single_tokens_that_forms_the_decay_itself(ops, dtype, H, dk, dv, R):
    """A step of single tokens with the decay's inputs in the place of alpha: the same bits as decay kernel + scan."""
    g = torch.Generator().manual_seed(H + dk + R)
    B = 5
    wide = torch.randn(B, 2 * H * dk + H * dv + R + 2, generator=g).to(dtype).to(DEV)
    q, k, v = wide[:, :H * dk], wide[:, H * dk:2 * H * dk], wide[:, 2 * H * dk:2 * H * dk + H * dv]
    a = wide[:, 2 * H * dk + H * dv:2 * H * dk + H * dv + R]
    w = torch.randn(H * dk, R, generator=g).to(dtype).to(DEV)
    bias = (torch.randn(H * dk, generator=g) * 2).to(DEV)
    state0 = torch.randn(B + 1, H, dv, dk, generator=g).to(DEV)
    ctx = _ctx([1] * B, [3, 0, 9, 1, 40], [4, 0, 2, 5, 1])
    alpha = torch.empty(B, H * dk, dtype=F32, device=DEV)
    ops.channel_decay(a, w, bias, 4.0, alpha)
    s1, s2 = state0.clone(), state0.clone()
    o1, o2 = torch.empty(B, H * dv, dtype=F32, device=DEV), torch.empty(B, H * dv, dtype=F32, device=DEV)
    ops.linear_attention_scan(q, k, v, alpha, s1, ctx, o1, dk ** -0.5, H, dk, dv)
    ops.linear_attention_scan(q, k, v, None, s2, ctx, o2, dk ** -0.5, H, dk, dv, decay=(a, w, bias, 4.0))
    assert torch.equal(o1, o2) and torch.equal(s1, s2)


# ---- norm of a head with its gate, the feed-forward's activation, the embedding -------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D", [(1, 7), (3, 24), (2, 128), (6, 32), (3, 256)])
def test_head_norm_gate(ops, dtype, H, D):
    g = torch.Generator().manual_seed(H * D)
    T = 21
    x = torch.randn(T, H * D, generator=g) * 3
    wide = torch.randn(T, H * D + 12, generator=g).to(dtype)      # (strides that let heads of 128 and 256 take 16-byte pieces)
    gate = wide[:, 4:4 + H * D]
    w = torch.randn(D, generator=g)
    buf = torch.zeros(T, 2 * H * D + 4, dtype=dtype, device=DEV)
    out = buf[:, H * D:2 * H * D]                                   # a column slice of a wider buffer
    ops.head_norm_gate(x.to(DEV), wide.to(DEV)[:, 4:4 + H * D], w.to(DEV), 1e-5, out, H, D, gate_kind="silu", scale=0.6)
    want = torch.cat([plain.norm_plain(x[:, h * D:(h + 1) * D].double(), w.double(), 1e-5) for h in range(H)], dim=1)
    want = want * plain.silu(gate.double()) * 0.6
    _close(out, want, dtype, "norm and silu gate")
    assert float(buf[:, :H * D].abs().max()) == 0 and float(buf[:, 2 * H * D:].abs().max()) == 0
    xa = x.to(dtype)
    out2 = torch.empty(T, H * D, dtype=dtype, device=DEV)
    ops.head_norm_gate(xa.to(DEV), wide.to(DEV)[:, 4:4 + H * D], None, 0.0, out2, H, D, gate_kind="sigmoid", scale=1.0)
    _close(out2, xa.double() * torch.sigmoid(gate.double()), dtype, "sigmoid gate")


@pytest.mark.parametrize("dtype", DTYPES)
def test_gelu_mul_and_scaled_embedding(ops, dtype):
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(13, 2 * 56, generator=g) * 3).to(dtype)
    out = torch.empty(13, 56, dtype=dtype, device=DEV)
    ops.act_mul(gu.to(DEV), out, "gelu_tanh")
    _close(out, plain.gelu_tanh(gu[:, :56].double()) * gu[:, 56:].double(), dtype, "gelu")
    table = torch.randn(50, 40, generator=g).to(dtype)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    stream = torch.empty(4, 40, dtype=F32, device=DEV)
    ops.embedding(ids.to(DEV), table.to(DEV), stream, scale=3.0)
    want = plain.embed_tokens(ids.tolist(), table.double(), 3.0)
    _close(stream, want, F32, "embedding", tol=1e-6)
    ops.embedding(ids.to(DEV), table.to(DEV), stream, scale=3.0, accumulate=True)
    _close(stream, 2 * want, F32, "embedding added again", tol=1e-6)


@pytest.mark.parametrize("M,I,K", [(3, 96, 64), (16, 3072, 1024), (1200, 3072, 512), (2048, 3072, 1024)])
def test_gate_up_product_with_gelu_in_its_epilogue(ops, M, I, K):
    """The two products that form act(gate) * up themselves (a few rows; many rows), with the tanh form of gelu."""
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, K, generator=g).to(BF16)
    w = (torch.randn(2 * I, K, generator=g) * (2.0 / math.sqrt(K))).to(BF16)
    out = torch.empty(M, I, dtype=BF16, device=DEV)
    if M <= 16:
        assert ops.swiglu_small_applies(M, I, K, BF16)
        ops.linear_swiglu_small(x.to(DEV), w.to(DEV), out, "gelu_tanh")
    else:
        assert ops.swiglu_fused_applies(M, I, K, BF16)
        ops.linear_swiglu(x.to(DEV), w.to(DEV), out, "gelu_tanh")
    gate, up = x.double() @ w[:I].double().T, x.double() @ w[I:].double().T
    _close(out, plain.gelu_tanh(gate) * up, BF16, "gelu in the epilogue")


# ---- windowed attention with a distance bias ------------------------------------------------------------------------------
def _attention_case(Hq, Hkv, D, P, q_lens, ctx_lens, dtype, seed, spikes=()):
    g = torch.Generator().manual_seed(seed)
    R = len(q_lens)
    totals = [c + n for c, n in zip(ctx_lens, q_lens)]
    blocks = [-(-t // P) for t in totals]
    n_pages = sum(blocks) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((R, max(blocks)), -1, dtype=torch.int32)
    it = iter(perm)
    for r in range(R):
        for b in range(blocks[r]):
            table[r, b] = next(it)
    cache = torch.randn(n_pages, 2, Hkv, P, D, generator=g).to(dtype)
    qkv = torch.randn(sum(q_lens), (Hq + 2 * Hkv) * D, generator=g).to(dtype)
    for r, q_index, key_pos, head in spikes:
        # one key decides the row if it is seen: its score stands out by far
        d = torch.randn(D, generator=g)
        d = d / d.norm()
        cache[int(table[r, key_pos // P]), 0, head // (Hq // Hkv), key_pos % P] = (d * 8.0).to(dtype)
        qkv[sum(q_lens[:r]) + q_index, head * D:(head + 1) * D] = (d * 8.0 * math.sqrt(D)).to(dtype)
    return qkv, cache, table


def _plain_attention(qkv, cache, table, Hq, Hkv, D, P, q_lens, ctx_lens, scale, slopes, window):
    out = torch.zeros(qkv.shape[0], Hq * D, dtype=torch.float64)
    row = 0
    for r, (n, c) in enumerate(zip(q_lens, ctx_lens)):
        total = c + n
        pos = torch.arange(total)
        pages = table[r, pos // P].long()
        for h in range(Hq):
            kvh = h // (Hq // Hkv)
            k = cache[pages, 0, kvh, pos % P].double()
            v = cache[pages, 1, kvh, pos % P].double()
            q = torch.zeros(total, D, dtype=torch.float64)
            q[c:] = qkv[row:row + n, h * D:(h + 1) * D].double()
            out[row:row + n, h * D:(h + 1) * D] = plain.windowed_softmax_attention(q, k, v, scale, slopes[h], window)[c:]
        row += n
    return out


def _run_attention(ops, qkv, cache, table, Hq, Hkv, D, P, q_lens, ctx_lens, scale, slopes, window, dtype, flash):
    from qwen_engine_b200.engine.runner import ModelRunner
    geo = (Hq, Hkv, D, window, True)
    geos = (geo,) if flash else ()
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, geos, dtype)
    devplan = ModelRunner._device_plan(plan, {"plan_" + k: torch.tensor(v, dtype=torch.int32, device=DEV) for k, v in plan.items()}, geos)
    ctx = _ctx(q_lens, ctx_lens, [0] * len(q_lens), devplan)
    out = torch.zeros(qkv.shape[0], Hq * D, dtype=dtype, device=DEV)
    ops.paged_attention(qkv.to(DEV), cache.to(DEV), table.to(DEV), ctx, out, scale, window, Hq, Hkv, D,
                        slopes=torch.tensor(slopes, dtype=F32, device=DEV))
    torch.cuda.synchronize()
    return out, ops.last_attention_kernel


BIASED_SHAPES = [(4, 2, 16, 4, 9), (3, 3, 48, 8, 20), (8, 2, 128, 16, 70), (2, 1, 32, 16, 1), (6, 3, 96, 16, 33)]
BIASED_BATCHES = [([30], [0]), ([1], [95]), ([1, 1, 1], [4, 77, 31]), ([7, 1, 2, 40], [9, 40, 0, 63]), ([2, 33], [64, 31])]


@pytest.mark.parametrize("dtype,flash", [(F32, False), (BF16, False), (BF16, True)])
@pytest.mark.parametrize("Hq,Hkv,D,P,window", BIASED_SHAPES)
@pytest.mark.parametrize("q_lens,ctx_lens", BIASED_BATCHES)
def test_attention_with_window_and_distance_bias(ops, dtype, flash, Hq, Hkv, D, P, window, q_lens, ctx_lens):
    slopes = [2.0 ** (-6.0 * (h + 1) / Hq) for h in range(Hq)]
    qkv, cache, table = _attention_case(Hq, Hkv, D, P, q_lens, ctx_lens, dtype, Hq * D + len(q_lens))
    scale = 0.9 / math.sqrt(D)
    got, kernel = _run_attention(ops, qkv, cache, table, Hq, Hkv, D, P, q_lens, ctx_lens, scale, slopes, window, dtype, flash)
    assert kernel in (("flash_attention", "flash_attention_tc", "decode_attention_mma") if flash else ("paged_attention_generic",))
    want = _plain_attention(qkv, cache, table, Hq, Hkv, D, P, q_lens, ctx_lens, scale, slopes, window)
    _close(got, want, dtype, kernel, tol={F32: 2e-5, BF16: 2e-2}[dtype])


@pytest.mark.parametrize("q_lens,ctx_lens,kernel", [([300], [0], "flash_attention_tc"), ([130], [77], "flash_attention_tc"),
                                                    ([1, 1, 1, 1], [300, 17, 512, 64], "decode_attention_mma"),
                                                    ([2, 1], [200, 90], "decode_attention_mma")])
@pytest.mark.parametrize("window", [64, 200])
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 4), (16, 2)])
def test_biased_attention_on_the_kernels_of_head_size_128(ops, q_lens, ctx_lens, kernel, window, Hq, Hkv):
    """Head size 128: prompt portions on the tcgen05 kernel, decoded tokens on the warp-pipelined kernel, both with
    the distance bias and a window that ends inside their key steps."""
    D, P = 128, 16
    slopes = [2.0 ** (-8.0 * (h + 1) / Hq) for h in range(Hq)]
    qkv, cache, table = _attention_case(Hq, Hkv, D, P, q_lens, ctx_lens, BF16, 5 + len(q_lens))
    scale = 1.0 / math.sqrt(D)
    got, used = _run_attention(ops, qkv, cache, table, Hq, Hkv, D, P, q_lens, ctx_lens, scale, slopes, window, BF16, True)
    assert used == kernel
    want = _plain_attention(qkv, cache, table, Hq, Hkv, D, P, q_lens, ctx_lens, scale, slopes, window)
    _close(got, want, BF16, kernel, tol=2e-2)


@pytest.mark.parametrize("dtype,flash", [(F32, False), (BF16, True)])
@pytest.mark.parametrize("window,P", [(24, 8), (33, 16), (16, 16)])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_key_just_inside_and_just_outside_the_window(ops, dtype, flash, window, P, decoded):
    """The last query's score for one key stands out by far.  With that key window - 1 tokens back the output
    is that key's value; one token further back it is not seen and the output is another."""
    Hq, Hkv, D, total = 2, 1, 32, 90
    q_lens, ctx_lens = ([1], [total - 1]) if decoded else ([40], [total - 40])
    slopes = [0.02, 0.3]
    scale = 1.0 / math.sqrt(D)
    last = total - 1
    for back, seen in ((window - 1, True), (window, False)):
        key_pos = last - back
        qkv, cache, table = _attention_case(Hq, Hkv, D, P, q_lens, ctx_lens, dtype, 77, spikes=[(0, q_lens[0] - 1, key_pos, 1)])
        got, _ = _run_attention(ops, qkv, cache, table, Hq, Hkv, D, P, q_lens, ctx_lens, scale, slopes, window, dtype, flash)
        want = _plain_attention(qkv, cache, table, Hq, Hkv, D, P, q_lens, ctx_lens, scale, slopes, window)
        _close(got, want, dtype, f"key {back} back", tol={F32: 2e-5, BF16: 2e-2}[dtype])
        value = cache[int(table[0, key_pos // P]), 1, 0, key_pos % P].double()
        near = float((want[-1, D:2 * D] - value).abs().max()) < 0.05 * float(value.abs().max())
        assert near == seen, f"a key {back} tokens back must {'decide' if seen else 'not touch'} the output"


# ---- whole models ------------------------------------------------------------------------------------------
# g-c (heads of 7 and 4 value channels, whose norms run over a handful of numbers) runs in float32 only: in bfloat16
# the rounding of a head's few outputs moves lone positions by tens of per cent, which no bound tells from a fault
@pytest.mark.parametrize("dtype,name", [(d, n) for n in gh.GANIDRA for d in DTYPES if not (n == "g-c" and d == BF16)])
def test_replay_against_the_plain_model(folders, dtype, name):
    folder = folders[name]
    gh.replay_cases(lambda n: gh.make_replayer(folder, name, dtype, n, poison=1.0e4), folder, name, dtype, f"{name}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_every_position_of_a_long_prompt_whole_and_decoded(folders, dtype):
    """Prompts longer than every window and several pages, at all positions: whole, and from the first token
    on one by one (the steps of single tokens are replayed from a CUDA graph): first tokens, pages' borders
    and the windows' edges lie among them, in prompts and in decoding."""
    for name, n in (("g-b", 120), ("g-d", 330)):
        folder = folders[name]
        toks = random_tokens(gh.vocab_of(name), n, 31)
        whole = [{"entries": [{"id": "a", "tokens": toks, "want": list(range(n))}], "end": ["a"]}]
        gh.check_requests(run_steps(gh.make_replayer(folder, name, dtype, 384), whole), folder, {"a": toks}, dtype, f"{name} whole")
        single = [{"entries": [{"id": "a", "tokens": [t], "want": [0]}]} for t in toks]
        rep = gh.make_replayer(folder, name, dtype, 384)
        gh.check_requests(run_steps(rep, single), folder, {"a": toks}, dtype, f"{name} decoded")
        assert rep.runner.num_graph_replays > n // 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_in_portions_then_decoded_at_a_middle_size(folders, dtype):
    """600 tokens: whole; and in portions of changing sizes (two tokens among them, cuts inside pages and windows)
    with the last 40 tokens one by one, beside a second request that comes and goes (its slot and pages are used again)."""
    name = "g-e"
    folder = folders[name]
    V = gh.vocab_of(name)
    toks, other = random_tokens(V, 600, 3), random_tokens(V, 50, 4)
    want = sorted(set(range(0, 600, 7)) | set(range(560, 600)))
    whole = [{"entries": [{"id": "a", "tokens": toks, "want": want}], "end": ["a"]}]
    gh.check_requests(run_steps(gh.make_replayer(folder, name, dtype, 640), whole), folder, {"a": toks}, dtype, "whole")
    steps, p = [], 0
    for i, n in enumerate([64, 64, 100, 2, 30, 129, 16, 3, 95, 57] + [1] * 40):
        entries = [{"id": "a", "tokens": toks[p:p + n], "want": [w - p for w in want if p <= w < p + n]}]
        if i in (1, 5, 12):                        # a short request beside it, three times over: admitted, run, ended
            entries.append({"id": f"b{i}", "tokens": other, "want": [49]})
        steps.append({"entries": entries, "end": [f"b{i}"] if i in (1, 5, 12) else []})
        p += n
    assert p == 600
    rep = gh.make_replayer(folder, name, dtype, 704)
    got = run_steps(rep, steps)
    gh.check_requests(got, folder, {"a": toks, "b1": other, "b5": other, "b12": other}, dtype, "portions")


def test_greedy_generation_through_the_engine(folders):
    from qwen_engine_b200.sampling.params import SamplingParams
    for name in ("g-a", "g-c"):
        folder = folders[name]
        cfg, w = gh.plain_model(folder)
        V = gh.vocab_of(name)
        prompts = [random_tokens(V, n, 40 + i) for i, n in enumerate([5, 19, 33, 2, 11, 26, 47])]
        eng = gh.make_engine(folder, name, F32, max_num_seqs=3, max_num_batched_tokens=24, prefill_chunk_size=7)
        ids = [eng.add_request(p, SamplingParams(max_new_tokens=8, temperature=0.0)) for p in prompts]
        outs = {o.request_id: o for o in eng.serving()}
        for rid, p in zip(ids, prompts):
            assert list(outs[rid].output_token_ids) == plain.greedy(cfg, w, p, 8), f"{name}: prompt of {len(p)} tokens"
        assert eng.cache.slots.num_free == eng.cache.slots.num_slots and eng.cache.pages_in_use() == 0


def test_the_command_line_replays_a_trace(folders, tmp_path):
    name = "g-c"
    folder = folders[name]
    toks = random_tokens(gh.vocab_of(name), 30, 8)
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
    V = gh.vocab_of(name)
    want = gh.plain_logits(folder, toks)
    first = torch.frombuffer(bytearray((out / "0.f32").read_bytes()), dtype=F32).reshape(-1, V)
    last = torch.frombuffer(bytearray((out / "2.f32").read_bytes()), dtype=F32).reshape(-1, V)
    gh.assert_close_rows(first, want[[0, 20]], F32, "step 0")
    gh.assert_close_rows(last, torch.stack([want[29], want[3]]), F32, "step 2")
