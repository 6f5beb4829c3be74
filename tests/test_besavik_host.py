"""Besavik on the host side of the engine: configuration, registry, weights and caches, and replay and generation on
the CPU with the plain operations in the place of the kernels, against the plain restatement of the design
(tests/plain_besavik.py).  The same traces run on the GPU in test_besavik_gpu.py."""
import copy

import pytest
import torch

import besavik_helpers as bh
import plain_besavik
from helpers import random_tokens
from qwen_engine_b200.config import BesavikConfig, ConfigError
from qwen_engine_b200.registry import architecture_of, build_model, config_from_dict
from qwen_engine_b200.weights import SafetensorsSource, WeightError, check_against_manifest

F32 = torch.float32


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("besavik")
    return {name: bh.make_folder(str(root / name), name) for name in ("b-a", "b-b", "b-c", "b-e", "b-f")}


def test_config_reads_its_own_keys_and_round_trips():
    raw = bh.BESAVIK["b-a"]["cfg"]
    assert architecture_of(raw).name == "Besavik"
    cfg = config_from_dict(raw)
    assert isinstance(cfg, BesavikConfig)
    assert (cfg.vocab, cfg.width, cfg.logit_scale, cfg.norm_eps) == (211, 64, 0.5, 1e-5)
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="gla"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][1].update(mlp=dict(kind="routed", ff=8)), "feed-forward"),
    (lambda c: c.pop("logit_scale"), "'logit_scale' is missing"),
    (lambda c: c["layers"][2]["mixer"].update(decay=[0.5]), "one number per head"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "even and at most"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "exceeds"),
])
def test_config_refuses_what_it_cannot_run(change, text):
    raw = copy.deepcopy(bh.BESAVIK["b-a"]["cfg"])
    change(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_caches_of_the_three_mixers():
    model = build_model(config_from_dict(bh.BESAVIK["b-a"]["cfg"]))
    kinds = [type(s).__name__ for s in model.cache_specs()]
    assert kinds == ["FixedStateSpec", "FixedStateSpec", "PagedKVSpec", "FixedStateSpec"]
    state, conv, latent, lightning = model.cache_specs()
    assert state.shape == (4, 12, 8) and conv.shape == (2, 2 * 2 * 8 + 4 * 12)      # taps - 1 inputs of q, k and v
    assert (latent.num_kv_heads, latent.head_dim, latent.window, latent.planes) == (1, 24 + 8, None, 1)
    assert lightning.shape == (2, 8, 16)
    assert model.attention_geometries == ((3, 1, 32, 0, False, 1),)


def test_tensor_names_and_the_ranks_that_no_key_names(folders):
    src = SafetensorsSource(folders["b-a"])
    names = set(src.names())
    assert {"embed", "embed.norm", "final.norm", "l0.norm1", "l0.mix.q.conv", "l0.mix.A_log", "l0.mix.dt_bias", "l0.mix.g2",
            "l0.mlp.e4.down", "l0.mlp.router", "l0.mlp.router.b", "l1.mix.dq.norm", "l1.mix.dkv", "l1.mix.uk", "l1.mlp.gate",
            "l2.mix.norm", "l2.mix.g"} <= names
    assert "l2.norm2" not in names and "l2.mlp.gate" not in names
    raw = copy.deepcopy(bh.BESAVIK["b-a"]["cfg"])
    raw["layers"][0]["mixer"].pop("rank")
    model = build_model(config_from_dict(raw))
    check_against_manifest(src, model.weight_manifest(), "folder")
    model.load_weights(src, F32, "cpu")
    assert model.blocks[0].mixer.decay_rank == 5 and model.blocks[0].mixer.gate_rank == 5
    raw["width"] = 72
    with pytest.raises(WeightError, match="wrong shapes"):
        check_against_manifest(src, build_model(config_from_dict(raw)).weight_manifest(), "folder")


@pytest.mark.parametrize("name", ["b-a", "b-b", "b-c", "b-e", "b-f"])
def test_replay_on_the_host(folders, cpu_ops, name):
    folder = folders[name]
    bh.replay_cases(lambda n: bh.make_replayer(folder, name, F32, n, device="cpu", poison=True), folder, name, F32,
                    f"host {name}")


def test_greedy_generation_through_the_engine_on_the_host(folders, cpu_ops):
    from qwen_engine_b200.sampling.params import SamplingParams
    name = "b-a"
    folder = folders[name]
    cfg, w = bh.plain_model(folder)
    V = bh.vocab_of(name)
    prompts = [random_tokens(V, n, 40 + i) for i, n in enumerate([5, 19, 33, 2, 11, 26])]
    eng = bh.make_engine(folder, name, F32, device="cpu", max_num_seqs=3, max_num_batched_tokens=24, prefill_chunk_size=7)
    ids = [eng.add_request(p, SamplingParams(max_new_tokens=6, temperature=0.0)) for p in prompts]
    outs = {o.request_id: o for o in eng.serving()}
    for rid, p in zip(ids, prompts):
        assert list(outs[rid].output_token_ids) == plain_besavik.greedy(cfg, w, p, 6), f"prompt of {len(p)} tokens"
    assert eng.cache.slots.num_free == eng.cache.slots.num_slots


def test_attention_alone_shares_the_pages_of_equal_prefixes(folders, cpu_ops):
    """A model without state of fixed size shares prefixes: a second request with the same first tokens takes the first
    one's pages (of both groups of pages) and its logits are the plain model's all the same."""
    from helpers import run_steps
    name = "b-f"
    folder = folders[name]
    V = bh.vocab_of(name)
    first = random_tokens(V, 40, 5)
    second = first[:24] + random_tokens(V, 10, 6)
    rep = bh.make_replayer(folder, name, F32, 192, device="cpu")
    assert rep.cache.prefix_cache and len(rep.cache.paged_groups) == 2
    steps = [{"entries": [{"id": "a", "tokens": first, "want": [39]}]},
             {"entries": [{"id": "b", "tokens": second, "want": [30, 33]}], "end": ["a", "b"]}]
    got = run_steps(rep, steps)
    assert rep.cache.prefix_hit_tokens == 24
    bh.check_requests(got, folder, {"a": first, "b": second}, F32, "shared prefix")
