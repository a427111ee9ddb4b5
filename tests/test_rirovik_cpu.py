"""The Rirovik architecture through the engine's host logic on the CPU (plain PyTorch kernels),
against the plain float64 model: configuration, checkpoint layout, shared cache layers, pages of
kept first tokens, every way of cutting requests into steps, and greedy generation through the
scheduler."""

import copy

import pytest
import torch

import plain_rirovik as pr
import traces
from conftest import RIROVIK_TINY
from plain_ops import PlainOps


def cpu_runner(folder, name, num_pages, max_num_seqs=4, max_len=512):
    from llmserve_b200.engine.runner import ModelRunner, load_model

    _, _, model = load_model(folder, "float32", "cpu", PlainOps(), max_len)
    return ModelRunner(model, page_tokens=RIROVIK_TINY[name]["page_tokens"], num_pages=num_pages,
                       max_model_len=max_len, max_num_seqs=max_num_seqs)


def test_config_round_trip_and_refusals():
    from llmserve_b200.config import ConfigError, architecture_for
    from llmserve_b200.config.rirovik import RirovikConfig

    for name in RIROVIK_TINY:
        d = RIROVIK_TINY[name]["config"]
        assert architecture_for(d).name == "Rirovik"
        cfg = RirovikConfig.from_dict(d)
        assert cfg.to_dict() == d and RirovikConfig.from_dict(cfg.to_dict()) == cfg
    d = RIROVIK_TINY["R1"]["config"]
    cfg = RirovikConfig.from_dict(d)
    assert cfg.layers[3].mixer.kv_from == 1 and cfg.layers[2].mlp is None and cfg.layers[1].mlp.shared_ff == 0
    assert cfg.layers[2].mixer.keep_first == 3 and cfg.layers[0].mixer.window == 0

    def broken(change):
        b = copy.deepcopy(d)
        change(b)
        with pytest.raises(ConfigError):
            RirovikConfig.from_dict(b)

    broken(lambda b: b["layers"][0].update(type="conv"))
    broken(lambda b: b["layers"][0]["mixer"].pop("scale"))
    broken(lambda b: b["layers"][0]["mixer"].update(sink=1))
    broken(lambda b: b["layers"][0]["mixer"].update(mask={"size": 4}))  # the causal kind has no window
    broken(lambda b: b["layers"][1]["mixer"].pop("mask"))  # the windowed kind needs one
    broken(lambda b: b["layers"][1]["mixer"]["rot"].update(dims=7))
    broken(lambda b: b["layers"][3]["mixer"].update(kv_from=3))  # not an earlier layer
    broken(lambda b: b["layers"][3]["mixer"].update(kv_from=2))  # not a latent layer
    broken(lambda b: b["layers"][3]["mixer"].update(kv_rank=48))  # another rank than the layer it reads
    broken(lambda b: b["layers"][3]["mixer"]["rot"].update(base=7.0))  # another rotation than the layer it reads
    broken(lambda b: b["layers"][2]["mixer"].update(kv_heads=3))
    broken(lambda b: b["layers"][0]["mlp"]["router"].update(top=6))
    broken(lambda b: b["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda b: b["embedding"].pop("scale"))
    broken(lambda b: b["norm"].pop("eps"))


def test_plan_shares_cache_layers_and_keeps_the_widest_window():
    from llmserve_b200.config.rirovik import RirovikConfig
    from llmserve_b200.models.rirovik import rirovik_plan

    plan = rirovik_plan(RirovikConfig.from_dict(RIROVIK_TINY["R1"]["config"]))
    assert [(e.layer, e.cache) for e in plan.run_order] == [(0, 0), (1, 1), (2, 2), (3, 1)]
    assert [getattr(l.mixer, "cache_window", None) for l in plan.layers] == [0, 33, None, 33]
    assert [l.mixer.window for l in plan.layers] == [0, 20, 12, 33]
    assert plan.layers[2].feed_forward is None and not plan.layers[3].mixer.own_latent
    assert plan.layers[2].mixer.keep_first == 3 and plan.layers[1].mixer.gate == "head" and plan.layers[0].mixer.gate == "none"
    assert plan.embed_scale == 2.5 and not plan.tie_head
    plan2 = rirovik_plan(RirovikConfig.from_dict(RIROVIK_TINY["R2"]["config"]))
    assert [(e.layer, e.cache) for e in plan2.run_order] == [(0, 0), (1, 1), (2, 2), (3, 3), (4, 1)]
    assert plan2.layers[1].mixer.cache_window == 0 and plan2.layers[4].mixer.window == 7  # the writer sees everything


def test_checkpoint_errors_are_reported_together(rirovik_dirs, tmp_path):
    from safetensors.torch import load_file, save_file

    from llmserve_b200.engine.runner import load_model
    from llmserve_b200.weights.loader import CheckpointError

    t = load_file(str(rirovik_dirs["R1"] / "model.safetensors"))
    assert "l3.mix.dkv" not in t and "l2.norm2" not in t and "l1.mlp.shared.up" not in t and "l0.mix.g" not in t
    assert t["l2.mix.g"].shape == (4 * 32, 96) and t["l1.mix.g"].shape == (2, 96) and t["head"].shape == (211, 96)
    del t["l0.mix.uq"]
    t["l1.mix.dkv"] = t["l1.mix.dkv"][:-1].contiguous()
    t["l3.mix.sink"] = torch.zeros(4)
    (tmp_path / "config.json").write_text((rirovik_dirs["R1"] / "config.json").read_text())
    save_file(t, str(tmp_path / "model.safetensors"))
    with pytest.raises(CheckpointError) as e:
        load_model(tmp_path, "float32", "cpu", PlainOps(), 64)
    msg = str(e.value)
    assert "l0.mix.uq" in msg and "l1.mix.dkv" in msg and "l3.mix.sink" in msg


def test_pages_of_kept_first_tokens_are_never_given_back():
    from llmserve_b200.cache import CacheManager, KVGroupSpec

    spec = KVGroupSpec((0,), 1, 16, window=10, page_tokens=4, keep_first=6)  # tokens 0..5: pages 0 and 1
    plain = KVGroupSpec((1,), 1, 16, window=10, page_tokens=4)
    m = CacheManager([spec, plain], [16, 16], 2)
    m.admit("a")
    for _ in range(10):
        m.allocate("a", 5)
        m.commit("a", 5)
        m.check_invariants()
    kept, windowed = m.block_table("a", 0), m.block_table("a", 1)
    assert kept[0] >= 0 and kept[1] >= 0 and kept[2] < 0  # the pages of the first six tokens stay
    assert windowed[0] < 0 and windowed[1] < 0
    first_needed = (50 - 10 + 1) // 4
    assert all(p < 0 for p in kept[2:first_needed]) and all(p >= 0 for p in kept[first_needed:])
    assert spec.live_tokens(1000, 1) == plain.live_tokens(1000, 1) + 8
    m.release("a")
    assert m.usage() == 0.0


LENGTHS = {"R1": [5, 70, 1, 33, 49, 90, 2], "R2": [2, 40, 9, 64, 17, 75], "R3": [3, 110, 18, 77]}


@pytest.fixture(scope="module")
def expected(rirovik_dirs):
    out = {}
    for name in RIROVIK_TINY:
        reqs = traces.make_requests(LENGTHS[name], RIROVIK_TINY[name]["config"]["vocab"], seed=5)
        out[name] = (reqs, {r: pr.model_logits(rirovik_dirs[name], t) for r, t in reqs.items()})
    return out


@pytest.mark.parametrize("name,mode", [("R1", "whole"), ("R1", "portions"), ("R1", "mixed"), ("R2", "decode_tail"),
                                       ("R2", "mixed"), ("R3", "portions")])
def test_every_way_of_cutting_matches_plain(rirovik_dirs, expected, name, mode):
    reqs, exp = expected[name]
    pool_tokens = traces.tokens_needed(reqs)
    runner = cpu_runner(rirovik_dirs[name], name, pool_tokens // RIROVIK_TINY[name]["page_tokens"])
    got = traces.replay(runner, getattr(traces, mode)(reqs))
    traces.compare(got, exp, atol=2e-4, rtol=5e-5)
    assert runner.manager.usage() == 0.0


def test_long_decoding_on_few_pages(rirovik_dirs):
    """200 tokens one by one from position 0 through windowed layers only (R2 without its causal
    layer would fit in a few pages; with it the causal group still needs them all): the windowed
    groups give pages back while the request lives, the kept first tokens' pages stay."""
    reqs = traces.make_requests([200], 130, seed=21)
    exp = {r: pr.model_logits(rirovik_dirs["R2"], t) for r, t in reqs.items()}
    runner = cpu_runner(rirovik_dirs["R2"], "R2", 25)
    got = traces.replay(runner, traces.decode_tail(reqs, tail=200))
    traces.compare(got, exp, atol=2e-4, rtol=5e-5)


def test_greedy_generation_through_the_scheduler(rirovik_dirs):
    from llmserve_b200 import LLM, SamplingParams

    prompts = [[5, 9, 100, 31, 7], list(range(40, 57)), [3] * 33, [100, 2]]
    m = LLM(str(rirovik_dirs["R1"]), dtype="float32", device="cpu", ops=PlainOps(), block_size=16, num_kv_blocks=24,
            max_model_len=128, max_num_seqs=3, max_num_batched_tokens=24)
    outs = m.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for o, p in zip(outs, prompts):
        assert o.outputs[0].token_ids == pr.greedy(rirovik_dirs["R1"], p, 8), p
