"""Shared by the Besavik tests: small configurations that differ in every size and constant, model folders with
seeded random weights, and the plain implementation's logits."""
from __future__ import annotations

import torch

import plain_besavik
from ganidra_helpers import assert_close_rows
from qwen_engine_b200.registry import config_from_dict
from qwen_engine_b200.weights import write_model_folder


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, dims=None):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale,
                rot=dict(base=base, dims=rot_dim if dims is None else dims))


def _lightning(heads, dim, vdim, decay):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay))


def _delta(heads, kv_heads, dim, vdim, conv, rank):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, rank=rank)


def _dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


def _moe(experts, top, ff, limit):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))


def _layer(kind, mixer, mlp=None):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def _model(vocab, width, logit_scale, eps, layers):
    return dict(architecture="Besavik", vocab=vocab, width=width, logit_scale=logit_scale, norm=dict(eps=eps), layers=layers)


BESAVIK = {
    # grouped key heads in the delta mixer, three heads of latent attention, a layer without feed-forward last
    "b-a": dict(cfg=_model(211, 64, 0.5, 1e-5, [
        _layer("channel_delta", _delta(4, 2, 8, 12, 3, 5), _moe(5, 2, 24, 0.8)),
        _layer("latent_attention", _latent(3, 8, 8, 12, 24, 20, 0.2, 10000.0), _dense(48, 1.5)),
        _layer("lightning", _lightning(2, 16, 8, (0.9, 0.5)))]), seed=3, std=0.12, norm_std=0.2, page=4),
    # latent attention first, with one head and fewer rotated channels than its rotated part has; one expert of three
    # per token, and all four of four; a convolution of two taps
    "b-b": dict(cfg=_model(300, 96, 1.0, 1e-6, [
        _layer("latent_attention", _latent(1, 16, 16, 32, 16, 8, 0.15, 500.0, dims=8), _moe(3, 1, 16, 2.0)),
        _layer("lightning", _lightning(4, 8, 8, (0.99, 0.7, 0.3, 1.0)), _dense(64, 0.5)),
        _layer("channel_delta", _delta(2, 2, 16, 16, 2, 7), _moe(4, 4, 32, 1.0)),
        _layer("latent_attention", _latent(2, 24, 8, 16, 40, 16, 0.3, 100.0), None)]), seed=5, std=0.1, norm_std=0.1, page=16),
    # sizes that are no multiples of four, one key head for three heads, convolutions of five taps and of one
    "b-c": dict(cfg=_model(97, 40, 2.0, 3e-6, [
        _layer("lightning", _lightning(1, 10, 6, (0.8,)), _moe(2, 1, 12, 3.0)),
        _layer("channel_delta", _delta(3, 1, 6, 10, 5, 3), _dense(56, 1.0)),
        _layer("latent_attention", _latent(2, 6, 4, 10, 10, 7, 0.4, 50.0), _moe(6, 3, 20, 0.7)),
        _layer("channel_delta", _delta(2, 2, 12, 4, 1, 2))]), seed=9, std=0.15, norm_std=0.3, page=8),
    # sizes of real heads: a cache row of 128 channels (the kernels' fast paths), 128 key channels in the delta mixer
    "b-d": dict(cfg=_model(513, 256, 0.3, 1e-6, [
        _layer("lightning", _lightning(2, 64, 128, (0.95, 0.999)), _dense(384, 1.0)),
        _layer("latent_attention", _latent(8, 32, 64, 32, 64, 48, 0.1, 200000.0), _moe(8, 3, 128, 1.0)),
        _layer("channel_delta", _delta(4, 2, 128, 64, 4, 16), _moe(8, 2, 96, 1.2)),
        _layer("latent_attention", _latent(8, 32, 64, 32, 64, 48, 0.1, 200000.0), _dense(256, 1.0))]),
        seed=13, std=0.05, norm_std=0.1, page=16),
    # no attention at all: nothing is paged
    "b-e": dict(cfg=_model(150, 48, 1.5, 1e-6, [
        _layer("channel_delta", _delta(2, 1, 8, 8, 4, 4), _dense(64, 1.0)),
        _layer("lightning", _lightning(3, 8, 16, (0.9, 0.95, 0.5)), _moe(4, 2, 16, 1.0))]), seed=17, std=0.12, norm_std=0.2, page=16),
    # attention alone, of two sizes (two groups of pages): no state of fixed size, so equal prefixes share pages
    "b-f": dict(cfg=_model(180, 64, 0.7, 1e-6, [
        _layer("latent_attention", _latent(2, 16, 16, 16, 32, 24, 0.2, 1000.0), _dense(96, 2.0)),
        _layer("latent_attention", _latent(4, 8, 8, 8, 24, 16, 0.25, 1000.0), _moe(4, 2, 24, 1.0)),
        _layer("latent_attention", _latent(2, 16, 16, 16, 32, 24, 0.2, 1000.0), None)]), seed=19, std=0.12, norm_std=0.2, page=8),
}


def make_folder(path: str, name: str) -> str:
    spec = BESAVIK[name]
    write_model_folder(config_from_dict(spec["cfg"]), path, spec["seed"], spec["std"], spec["norm_std"], torch.bfloat16)
    return path


_plain: dict = {}


def plain_model(folder: str):
    if folder not in _plain:
        _plain[folder] = plain_besavik.read_model_folder(folder)
    return _plain[folder]


def plain_logits(folder: str, tokens) -> torch.Tensor:
    key = (folder, tuple(tokens))
    if key not in _plain:
        cfg, w = plain_model(folder)
        _plain[key] = plain_besavik.forward(cfg, w, list(tokens)).to(torch.float32)
    return _plain[key]


def vocab_of(name: str) -> int:
    return BESAVIK[name]["cfg"]["vocab"]


def make_replayer(folder, name, dtype, max_tokens, device="cuda:0", slots=4, poison=False):
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.engine.trace import TraceReplayer
    page = BESAVIK[name]["page"]
    unit = max(64, page)
    unit = -(-unit // page) * page
    num_pages = -(-max_tokens // unit) * (unit // page)
    loaded = load_model(folder, dtype, device, page, num_pages, slots, poison_cache=poison, check_device=(device != "cpu"))
    return TraceReplayer(folder, dtype, max_tokens, page_size=page, loaded=loaded)


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
    kw = dict(dtype=dtype, device=device, block_size=BESAVIK[name]["page"], max_model_len=160, max_num_seqs=4,
              max_num_batched_tokens=48)
    kw.update(engine_kwargs)
    ec = EngineConfig(**kw)
    loaded = load_model(folder, ec.dtype, ec.device, ec.block_size, ec.resolved_num_blocks(), ec.max_num_seqs,
                        ec.enable_prefix_cache, check_device=(device != "cpu"))
    return LLMEngine(loaded, ec)


def replay_cases(rep_factory, folder, name, dtype, what):
    """The ways of cutting requests into steps, each against the plain implementation: whole prompts; a prompt and
    then single tokens; from the first token one by one; portions of changing sizes down to two tokens; up to four
    live requests mixed, with pages and slots that come back and go out again."""
    from helpers import live_tokens_needed, mixed_steps, random_tokens, run_steps
    V = vocab_of(name)
    reqs = {"w0": random_tokens(V, 61, 1), "w1": random_tokens(V, 9, 2)}
    steps = [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}], "end": [r]} for r, t in reqs.items()]
    check_requests(run_steps(rep_factory(128), steps), folder, reqs, dtype, f"{what} whole")
    toks = random_tokens(V, 75, 3)
    steps = [{"entries": [{"id": "d", "tokens": toks[:35], "want": [0, 17, 34]}]}]
    steps += [{"entries": [{"id": "d", "tokens": [t], "want": [0]}]} for t in toks[35:]]
    check_requests(run_steps(rep_factory(128), steps), folder, {"d": toks}, dtype, f"{what} decode")
    steps = [{"entries": [{"id": "s", "tokens": [t], "want": [0]}]} for t in toks[:20]]
    check_requests(run_steps(rep_factory(64), steps), folder, {"s": toks[:20]}, dtype, f"{what} single tokens")
    toks = random_tokens(V, 90, 4)
    steps, p = [], 0
    for n in [2, 7, 3, 2, 16, 5, 2, 13, 9, 2, 11] + [1] * 18:
        steps.append({"entries": [{"id": "c", "tokens": toks[p:p + n], "want": list(range(n))}]})
        p += n
    assert p == len(toks)
    check_requests(run_steps(rep_factory(128), steps), folder, {"c": toks}, dtype, f"{what} portions")
    reqs = {f"m{i}": random_tokens(V, n, 20 + i) for i, n in enumerate([40, 64, 23, 90, 17, 55, 70, 33])}
    steps = mixed_steps(reqs, seed=7)
    rep = rep_factory(live_tokens_needed(steps, 64))
    check_requests(run_steps(rep, steps), folder, reqs, dtype, f"{what} mixed")
    assert rep.cache.pages_in_use() == 0 and rep.cache.slots.num_free == rep.cache.slots.num_slots
