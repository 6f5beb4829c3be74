"""Shared by the Ganidra tests: small configurations that differ in every size and constant, model
folders with seeded random weights, and the plain implementation's logits."""
from __future__ import annotations

import torch

import plain_ganidra
from qwen_engine_b200.registry import config_from_dict
from qwen_engine_b200.weights import write_model_folder


def _gla(heads, dim, vdim, tau, rank):
    return dict(heads=heads, dim=dim, vdim=vdim, tau=tau, rank=rank)


def _soft(heads, kv, dim, vdim, window, scale):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, mask=dict(size=window), scale=scale)


def _layer(kind, mixer, ff=None):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff))


GANIDRA = {
    # values of another size than keys in both mixers, grouped heads, a loop over the first two layers
    "g-a": dict(cfg=dict(architecture="Ganidra", vocab=211, width=64, embedding=dict(scale=3.0), norm=dict(eps=1e-5),
                         layers=[_layer("gla", _gla(2, 16, 24, 8.0, 4)),
                                 _layer("parallel", dict(left=_soft(4, 2, 16, 32, 9, 0.3), right=_gla(3, 8, 16, 4.0, 3),
                                                         left_scale=0.7, right_scale=1.1), ff=96),
                                 _layer("gla", _gla(4, 8, 8, 2.0, 5), ff=80)],
                         loop=dict(start=0, stop=2, times=2)),
                seed=3, std=0.12, norm_std=0.2, page=4),
    # no loop; a parallel layer without feed-forward first; one key/value head; a window of one page and one token
    "g-b": dict(cfg=dict(architecture="Ganidra", vocab=300, width=96, embedding=dict(scale=1.0), norm=dict(eps=1e-6),
                         layers=[_layer("parallel", dict(left=_soft(2, 1, 32, 32, 17, 0.18), right=_gla(2, 32, 32, 16.0, 8),
                                                         left_scale=1.0, right_scale=0.5)),
                                 _layer("gla", _gla(4, 12, 20, 1.0, 2), ff=128),
                                 _layer("parallel", dict(left=_soft(3, 3, 16, 16, 40, 0.25), right=_gla(1, 64, 48, 32.0, 6),
                                                         left_scale=-0.4, right_scale=1.3), ff=64)],
                         loop=dict(start=0, stop=0, times=1)),
                seed=5, std=0.1, norm_std=0.1, page=16),
    # sizes that are no multiples of four, one head, a window that sees the token alone, the last layers three times
    "g-c": dict(cfg=dict(architecture="Ganidra", vocab=97, width=40, embedding=dict(scale=0.5), norm=dict(eps=3e-6),
                         layers=[_layer("gla", _gla(1, 10, 7, 3.0, 1), ff=56),
                                 _layer("parallel", dict(left=_soft(1, 1, 8, 24, 1, 0.35), right=_gla(2, 6, 10, 5.0, 2),
                                                         left_scale=0.9, right_scale=0.6)),
                                 _layer("parallel", dict(left=_soft(2, 2, 24, 8, 5, 0.2), right=_gla(3, 4, 4, 7.0, 2),
                                                         left_scale=0.5, right_scale=0.5), ff=48)],
                         loop=dict(start=1, stop=3, times=3)),
                seed=9, std=0.15, norm_std=0.3, page=8),
    # the head sizes of real models: 128 for the softmax mixer (the kernels' fast paths), 128 and 256 key channels
    "g-d": dict(cfg=dict(architecture="Ganidra", vocab=513, width=256, embedding=dict(scale=4.0), norm=dict(eps=1e-6),
                         layers=[_layer("gla", _gla(2, 128, 128, 16.0, 16)),
                                 _layer("parallel", dict(left=_soft(4, 2, 128, 128, 150, 0.088), right=_gla(1, 256, 64, 16.0, 8),
                                                         left_scale=0.8, right_scale=0.8), ff=384)],
                         loop=dict(start=0, stop=2, times=2)),
                seed=13, std=0.05, norm_std=0.1, page=16),
    # a middle size: five layers, the second and third passed twice, a window longer than several pages and one shorter
    # than two, grouped heads, keys smaller than values
    "g-e": dict(cfg=dict(architecture="Ganidra", vocab=1000, width=384, embedding=dict(scale=8.0), norm=dict(eps=1e-6),
                         layers=[_layer("gla", _gla(6, 32, 64, 16.0, 16)),
                                 _layer("parallel", dict(left=_soft(6, 2, 64, 64, 100, 0.125), right=_gla(3, 32, 32, 8.0, 8),
                                                         left_scale=0.6, right_scale=0.9), ff=768),
                                 _layer("gla", _gla(4, 48, 96, 12.0, 12), ff=512),
                                 _layer("parallel", dict(left=_soft(4, 4, 48, 80, 31, 0.15), right=_gla(6, 16, 32, 2.0, 4),
                                                         left_scale=1.0, right_scale=1.0)),
                                 _layer("gla", _gla(6, 32, 64, 16.0, 16))],
                         loop=dict(start=1, stop=3, times=2)),
                seed=21, std=0.04, norm_std=0.1, page=16),
}


def make_folder(path: str, name: str) -> str:
    spec = GANIDRA[name]
    write_model_folder(config_from_dict(spec["cfg"]), path, spec["seed"], spec["std"], spec["norm_std"], torch.bfloat16)
    return path


_plain: dict = {}


def plain_model(folder: str):
    if folder not in _plain:
        _plain[folder] = plain_ganidra.read_model_folder(folder)
    return _plain[folder]


def plain_logits(folder: str, tokens) -> torch.Tensor:
    key = (folder, tuple(tokens))
    if key not in _plain:
        cfg, w = plain_model(folder)
        _plain[key] = plain_ganidra.forward(cfg, w, list(tokens)).to(torch.float32)
    return _plain[key]


def vocab_of(name: str) -> int:
    return GANIDRA[name]["cfg"]["vocab"]


def make_replayer(folder, name, dtype, max_tokens, device="cuda:0", slots=4, poison=False):
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.engine.trace import TraceReplayer
    page = GANIDRA[name]["page"]
    unit = max(64, page)
    unit = -(-unit // page) * page
    num_pages = -(-max_tokens // unit) * (unit // page)
    loaded = load_model(folder, dtype, device, page, num_pages, slots, poison_cache=poison, check_device=(device != "cpu"))
    return TraceReplayer(folder, dtype, max_tokens, page_size=page, loaded=loaded)


# A position's error is the root mean square over the vocabulary of the difference of the logits (mean taken off),
# over the root mean square of the plain logits there.  float32: the order of sums only.  bfloat16: every product,
# norm, gate and cache entry is rounded to 8 bits of mantissa, which these narrow random models amplify to 1-2.5 %
# at the logits (measured layer by layer: 0.5 % after one layer, growing evenly), and a lone position goes to 10-15 %
# where a head's output of the recurrence nearly cancels and its norm divides by what is left (one of 120 positions
# in one measured prompt, the others at 1-3 %).  So in bfloat16 19 of 20 positions (all but one of a few) must be within ROW_TOL and none
# beyond ROW_WORST; float32 has one bound for all.  A window that is one token off, a lost state or a wrong slot
# moves the positions it touches by tens of per cent, in float32 as in bfloat16.
ROW_TOL = {torch.float32: 1e-4, torch.bfloat16: 6e-2}
ROW_WORST = {torch.float32: 1e-4, torch.bfloat16: 0.3}


def assert_close_rows(got: torch.Tensor, want: torch.Tensor, dtype, what: str = "") -> None:
    got = got.detach().to("cpu", torch.float64)
    want = want.to(torch.float64)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    d = got - want
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / (want - want.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt()
    worst = int(torch.argmax(err))
    assert float(err[worst]) <= ROW_WORST[dtype], f"{what}: row {worst} is off by {float(err[worst]):.3e} > {ROW_WORST[dtype]}"
    over = int((err > ROW_TOL[dtype]).sum())
    assert over <= max(1, err.numel() // 20), f"{what}: {over} of {err.numel()} rows are off by more than {ROW_TOL[dtype]}"


def check_requests(got, folder, requests, dtype, what):
    for rid, toks in requests.items():
        want = plain_logits(folder, toks)
        rows = got[rid]
        idx = sorted(rows)
        assert_close_rows(torch.stack([rows[i] for i in idx]), want[idx], dtype, f"{what} {rid} (positions {idx[0]}..)")


def make_engine(folder, name, dtype, device="cuda:0", **engine_kwargs):
    from qwen_engine_b200.config import EngineConfig
    from qwen_engine_b200.engine.llm import LLMEngine
    from qwen_engine_b200.engine.loading import load_model
    kw = dict(dtype=dtype, device=device, block_size=GANIDRA[name]["page"], max_model_len=160, max_num_seqs=4,
              max_num_batched_tokens=48)
    kw.update(engine_kwargs)
    ec = EngineConfig(**kw)
    loaded = load_model(folder, ec.dtype, ec.device, ec.block_size, ec.resolved_num_blocks(), ec.max_num_seqs,
                        ec.enable_prefix_cache, check_device=(device != "cpu"))
    return LLMEngine(loaded, ec)


def replay_cases(rep_factory, folder, name, dtype, what):
    """The four ways of cutting requests into steps, each against the plain implementation: whole prompts;
    a prompt and then single tokens; portions of changing sizes down to two tokens; up to four live requests
    mixed, with pages and slots that come back and go out again."""
    from helpers import live_tokens_needed, mixed_steps, random_tokens, run_steps
    V = vocab_of(name)
    # whole
    reqs = {"w0": random_tokens(V, 61, 1), "w1": random_tokens(V, 9, 2)}
    steps = [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}], "end": [r]} for r, t in reqs.items()]
    check_requests(run_steps(rep_factory(128), steps), folder, reqs, dtype, f"{what} whole")
    # a prompt, then token by token (prefill against decoding: every decoded token's logits are checked)
    toks = random_tokens(V, 75, 3)
    steps = [{"entries": [{"id": "d", "tokens": toks[:35], "want": [0, 17, 34]}]}]
    steps += [{"entries": [{"id": "d", "tokens": [t], "want": [0]}]} for t in toks[35:]]
    check_requests(run_steps(rep_factory(128), steps), folder, {"d": toks}, dtype, f"{what} decode")
    # the same request from its first token on, one token a step: the first tokens of a sequence
    steps = [{"entries": [{"id": "s", "tokens": [t], "want": [0]}]} for t in toks[:20]]
    check_requests(run_steps(rep_factory(64), steps), folder, {"s": toks[:20]}, dtype, f"{what} single tokens")
    # portions
    toks = random_tokens(V, 90, 4)
    steps, p = [], 0
    for n in [2, 7, 3, 2, 16, 5, 2, 13, 9, 2, 11] + [1] * 18:
        steps.append({"entries": [{"id": "c", "tokens": toks[p:p + n], "want": list(range(n))}]})
        p += n
    assert p == len(toks)
    check_requests(run_steps(rep_factory(128), steps), folder, {"c": toks}, dtype, f"{what} portions")
    # mixed: unequal requests side by side against each alone, in a pool that is just large enough
    reqs = {f"m{i}": random_tokens(V, n, 20 + i) for i, n in enumerate([40, 64, 23, 90, 17, 55, 70, 33])}
    steps = mixed_steps(reqs, seed=7)
    rep = rep_factory(live_tokens_needed(steps, 64))
    check_requests(run_steps(rep, steps), folder, reqs, dtype, f"{what} mixed")
    assert rep.cache.pages_in_use() == 0 and rep.cache.slots.num_free == rep.cache.slots.num_slots
