"""Ganidra on the host side of the engine: configuration, registry, weights, the plan of layer runs, and
replay and generation on the CPU with the plain operations in the place of the kernels, against the plain
restatement of the design (tests/plain_ganidra.py).  The same traces run on the GPU in test_ganidra_gpu.py."""
import copy
import json
import os

import pytest
import torch

import ganidra_helpers as gh
import plain_ganidra
from helpers import random_tokens
from qwen_engine_b200.config import ConfigError, GanidraConfig
from qwen_engine_b200.registry import architecture_of, build_model, config_from_dict
from qwen_engine_b200.weights import SafetensorsSource, WeightError, check_against_manifest

F32 = torch.float32


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("ganidra")
    return {name: gh.make_folder(str(root / name), name) for name in ("g-a", "g-b", "g-c")}


def test_config_reads_its_own_keys_and_round_trips():
    raw = gh.GANIDRA["g-a"]["cfg"]
    assert architecture_of(raw).name == "Ganidra"
    cfg = config_from_dict(raw)
    assert isinstance(cfg, GanidraConfig)
    assert (cfg.vocab, cfg.width, cfg.embedding_scale, cfg.norm_eps) == (211, 64, 3.0, 1e-5)
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.layer_runs() == plain_ganidra.layer_order(raw)
    for name in gh.GANIDRA:
        raw = gh.GANIDRA[name]["cfg"]
        assert config_from_dict(raw).layer_runs() == plain_ganidra.layer_order(raw)


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="conv"), "not a mixer"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][1].update(mlp=dict(kind="routed", ff=8)), "feed-forward"),
    (lambda c: c.pop("norm"), "'norm' is missing"),
    (lambda c: c.update(loop=dict(start=2, stop=9, times=2)), "does not lie within"),
    (lambda c: c["layers"][0]["mixer"].update(tau=0), "positive"),
])
def test_config_refuses_what_it_cannot_run(change, text):
    raw = copy.deepcopy(gh.GANIDRA["g-a"]["cfg"])
    change(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_plan_gives_every_run_its_own_caches():
    model = build_model(config_from_dict(gh.GANIDRA["g-a"]["cfg"]))
    plan = model.layout.plan
    assert [e.layer for e in plan] == [0, 1, 0, 1, 2]
    assert [e.add_embedding for e in plan] == [False, False, True, False, False]
    slots = [s for e in plan for s in e.slots]
    assert sorted(slots) == list(range(len(slots)))            # no slot twice: each pass has its own state
    kinds = [type(s).__name__ for s in model.cache_specs()]
    assert kinds == ["FixedStateSpec", "PagedKVSpec", "FixedStateSpec", "FixedStateSpec", "PagedKVSpec", "FixedStateSpec",
                     "FixedStateSpec"]
    # keys of 16 and values of 32 share pages of the larger size; the window is the mixer's
    paged = model.cache_specs()[1]
    assert (paged.num_kv_heads, paged.head_dim, paged.window) == (2, 32, 9)


def test_tensor_names_and_the_rank_that_no_key_names(folders, tmp_path):
    folder = folders["g-a"]
    src = SafetensorsSource(folder)
    names = set(src.names())
    assert {"embed", "final.norm", "l0.norm1", "l0.mix.a2.b", "l1.mix.left.q.norm", "l1.mix.right.a1", "l1.mlp.gate",
            "l1.norm2"} <= names
    assert "l0.norm2" not in names and "l0.mlp.gate" not in names        # a layer without feed-forward has neither
    # without the 'rank' key the rank is whatever the file stores
    raw = copy.deepcopy(gh.GANIDRA["g-a"]["cfg"])
    for layer in raw["layers"]:
        for m in (layer["mixer"], layer["mixer"].get("right", {})):
            m.pop("rank", None)
    model = build_model(config_from_dict(raw))
    check_against_manifest(src, model.weight_manifest(), "folder")
    model.load_weights(src, F32, "cpu")
    assert model.blocks[0].mixer.rank == 4 and model.blocks[1].mixer.branches[1].rank == 3
    # a tensor of another width is still refused
    raw["width"] = 72
    with pytest.raises(WeightError, match="wrong shapes"):
        check_against_manifest(src, build_model(config_from_dict(raw)).weight_manifest(), "folder")


@pytest.mark.parametrize("name", ["g-a", "g-b", "g-c"])
def test_replay_on_the_host(folders, cpu_ops, name):
    folder = folders[name]
    gh.replay_cases(lambda n: gh.make_replayer(folder, name, F32, n, device="cpu", poison=True), folder, name, F32,
                    f"host {name}")


def test_keys_at_every_edge_of_the_window_on_the_host(folders, cpu_ops):
    """Every position of a prompt that is longer than the window and several pages, whole and from position
    0 token by token: the first tokens, pages' borders and the window's edge all lie among them."""
    name = "g-b"                                    # windows of 17 and 40 tokens, pages of 16
    folder = folders[name]
    toks = random_tokens(gh.vocab_of(name), 100, 31)
    from helpers import run_steps
    whole = [{"entries": [{"id": "a", "tokens": toks, "want": list(range(100))}], "end": ["a"]}]
    gh.check_requests(run_steps(gh.make_replayer(folder, name, F32, 128, device="cpu"), whole), folder, {"a": toks}, F32, "edges whole")
    single = [{"entries": [{"id": "a", "tokens": [t], "want": [0]}]} for t in toks]
    rep = gh.make_replayer(folder, name, F32, 128, device="cpu")
    gh.check_requests(run_steps(rep, single), folder, {"a": toks}, F32, "edges decoded")
    # the windowed groups gave back what every later query has passed
    held = {g.index: sum(p >= 0 for p in rep.live["a"].tables[g.index]) for g in rep.cache.paged_groups}
    assert max(held.values()) <= -(-40 // 16) + 1 and min(held.values()) <= -(-17 // 16) + 1


def test_greedy_generation_through_the_engine_on_the_host(folders, cpu_ops):
    from qwen_engine_b200.sampling.params import SamplingParams
    name = "g-a"
    folder = folders[name]
    cfg, w = gh.plain_model(folder)
    V = gh.vocab_of(name)
    prompts = [random_tokens(V, n, 40 + i) for i, n in enumerate([5, 19, 33, 2, 11, 26])]
    eng = gh.make_engine(folder, name, F32, device="cpu", max_num_seqs=3, max_num_batched_tokens=24, prefill_chunk_size=7)
    ids = [eng.add_request(p, SamplingParams(max_new_tokens=6, temperature=0.0)) for p in prompts]
    outs = {o.request_id: o for o in eng.serving()}
    for rid, p in zip(ids, prompts):
        assert list(outs[rid].output_token_ids) == plain_ganidra.greedy(cfg, w, p, 6), f"prompt of {len(p)} tokens"
    assert eng.cache.slots.num_free == eng.cache.slots.num_slots
