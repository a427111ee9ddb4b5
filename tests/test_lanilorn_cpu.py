"""The Lanilorn architecture through the engine's host logic on the CPU (plain PyTorch kernels),
against the plain float64 model: configuration, checkpoint layout, a size read from a tensor's
shape, every way of cutting requests into steps, long decoding and greedy generation through the
scheduler."""

import copy
import json

import pytest
import torch

import plain_lanilorn as pl
import traces
from conftest import LANILORN_TINY
from plain_ops import PlainOps


def cpu_runner(folder, name, num_pages, max_num_seqs=4, max_len=512):
    from llmserve_b200.engine.runner import ModelRunner, load_model

    _, _, model = load_model(folder, "float32", "cpu", PlainOps(), max_len)
    return ModelRunner(model, page_tokens=LANILORN_TINY[name]["page_tokens"], num_pages=num_pages,
                       max_model_len=max_len, max_num_seqs=max_num_seqs)


def test_config_round_trip_and_refusals():
    from llmserve_b200.config import ConfigError, architecture_for
    from llmserve_b200.config.lanilorn import LanilornConfig

    for name in LANILORN_TINY:
        d = LANILORN_TINY[name]["config"]
        assert architecture_for(d).name == "Lanilorn"
        cfg = LanilornConfig.from_dict(d)
        assert cfg.to_dict() == d and LanilornConfig.from_dict(cfg.to_dict()) == cfg
    d = LANILORN_TINY["L1"]["config"]
    cfg = LanilornConfig.from_dict(d)
    assert cfg.streams == 2 and cfg.layers[1].ff == 0 and cfg.layers[0].mixer.yarn.factor == 4.0
    assert cfg.layers[2].mixer.temp_every == 8 and cfg.layers[3].mixer.decay_rank == 4

    def broken(change):
        b = copy.deepcopy(d)
        change(b)
        with pytest.raises(ConfigError):
            LanilornConfig.from_dict(b)

    broken(lambda b: b["layers"][0].update(type="conv"))
    broken(lambda b: b["layers"][0]["mixer"].pop("scale"))
    broken(lambda b: b["layers"][0]["mixer"].update(vdim=8))  # the values are the keys
    broken(lambda b: b["layers"][0]["mixer"].update(sink=1))
    broken(lambda b: b["layers"][0]["mixer"]["rot"].update(dims=7))
    broken(lambda b: b["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"))
    broken(lambda b: b["layers"][0]["mixer"].update(kv_heads=3))
    broken(lambda b: b["layers"][2]["mixer"].pop("diff"))
    broken(lambda b: b["layers"][2]["mixer"]["q_temp"].update(every=0))
    broken(lambda b: b["layers"][1]["mixer"].update(tau=0.0))
    broken(lambda b: b["layers"][0]["mlp"].update(kind="moe"))
    broken(lambda b: b.pop("streams"))
    broken(lambda b: b.pop("logit_scale"))
    broken(lambda b: b["embedding"].pop("scale"))


def test_plan_is_streams_blocks_with_the_right_mixers():
    from llmserve_b200.config.lanilorn import LanilornConfig
    from llmserve_b200.models.lanilorn import lanilorn_plan

    plan = lanilorn_plan(LanilornConfig.from_dict(LANILORN_TINY["L1"]["config"]))
    assert [l.kind for l in plan.layers] == ["streams"] * 4 and plan.residual_streams == 2 and plan.tie_head
    assert [l.mixer.kind for l in plan.layers] == ["attention", "gated_linear_attention", "differential_attention",
                                                   "gated_linear_attention"]
    a = plan.layers[0].mixer
    assert a.values_are_keys and a.sinks and a.gate == "head" and a.qk_norm_scope == "row" and a.window == 10
    assert a.position.head_dim == 12 and a.position.scaling_type == "yarn"
    assert plan.layers[1].feed_forward is None and plan.layers[2].mixer.out_scale == pytest.approx(0.7)
    assert plan.layers[1].mixer.query_scale == 0.25 and plan.embed_scale == 1.5 and plan.logit_scale == 0.5
    assert not plan.final_norm.learned_read


def test_a_size_that_only_a_tensor_gives_is_read_from_the_folder(lanilorn_dirs, tmp_path):
    """The inner size of the decay matrices need not stand in config.json."""
    import shutil

    from llmserve_b200.config import ConfigError
    from llmserve_b200.config.lanilorn import LanilornConfig
    from llmserve_b200.engine.runner import load_model

    src = lanilorn_dirs["L1"]
    shutil.copy(src / "model.safetensors", tmp_path / "model.safetensors")
    d = json.loads((src / "config.json").read_text())
    for l in d["layers"]:
        l["mixer"].pop("decay_rank", None)
    (tmp_path / "config.json").write_text(json.dumps(d))
    cfg = LanilornConfig.from_pretrained(tmp_path)
    assert [l.mixer.decay_rank for l in cfg.layers if l.type == "gla"] == [8, 4]
    _, _, model = load_model(tmp_path, "float32", "cpu", PlainOps(), 64)
    assert model.blocks[3].mixer.decay_in_weight.shape == (4, 64)
    with pytest.raises(ValueError):  # without a folder nothing gives the size
        from llmserve_b200.models.lanilorn import lanilorn_plan

        lanilorn_plan(LanilornConfig.from_dict(d))
    assert ConfigError is not None


def test_checkpoint_errors_are_reported_together(lanilorn_dirs, tmp_path):
    from safetensors.torch import load_file, save_file

    from llmserve_b200.engine.runner import load_model
    from llmserve_b200.weights.loader import CheckpointError

    t = load_file(str(lanilorn_dirs["L1"] / "model.safetensors"))
    t.pop("l0.mix.sink")
    t["l1.norm2"] = torch.zeros(64)  # a layer without feed-forward has no second norm
    t["l2.hc1.mix"] = torch.zeros(3, 3)
    save_file(t, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text((lanilorn_dirs["L1"] / "config.json").read_text())
    with pytest.raises(CheckpointError) as e:
        load_model(tmp_path, "float32", "cpu", PlainOps(), 64)
    assert e.value.missing == ["l0.mix.sink"] and e.value.unexpected == ["l1.norm2"]
    assert [w[0] for w in e.value.wrong_shape] == ["l2.hc1.mix"]


def test_stretched_frequencies_against_the_formula_written_out():
    """The tables of the position part: pairs that turn fast keep their frequency, slow ones are
    stretched by the factor, the ones between are blended, and both tables carry the factor's magnitude."""
    from llmserve_b200.parts.base import BuildEnv
    from llmserve_b200.parts.positions import RotaryPositionEncoding, RotarySpec

    env = BuildEnv(ops=None, dtype=torch.float32, device=torch.device("cpu"), max_positions=50)
    for dims, base, sc in [(12, 10000.0, dict(factor=4.0, original=64, fast=16.0, slow=2.0)),
                           (32, 250.0, dict(factor=16.0, original=40, fast=4.0, slow=0.5)),
                           (6, 50.0, dict(factor=2.0, original=8, fast=1.0, slow=1.0))]:
        spec = RotarySpec(head_dim=dims, theta=base, scaling_type="yarn", factor=sc["factor"],
                          original_max_positions=sc["original"], yarn_fast=sc["fast"], yarn_slow=sc["slow"])
        cos, sin = RotaryPositionEncoding(spec, env).rotary_tables()
        f, mag = pl.yarn_frequencies(dims, base, sc)
        ang = torch.arange(50, dtype=torch.float64)[:, None] * f[None, :]
        assert torch.allclose(cos.double(), ang.cos() * mag, atol=1e-6) and torch.allclose(sin.double(), ang.sin() * mag, atol=1e-6)
        plain = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        assert (f <= plain + 1e-15).all() and (f >= plain / sc["factor"] - 1e-15).all() and mag > 1.0


LENGTHS = {"L1": [5, 70, 1, 33, 49, 126, 2], "L2": [2, 40, 9, 64, 17, 100], "L3": [3, 90, 18, 77]}


@pytest.fixture(scope="module")
def expected(lanilorn_dirs):
    out = {}
    for name in LANILORN_TINY:
        reqs = traces.make_requests(LENGTHS[name], LANILORN_TINY[name]["config"]["vocab"], seed=5)
        out[name] = (reqs, {r: pl.model_logits(lanilorn_dirs[name], t) for r, t in reqs.items()})
    return out


@pytest.mark.parametrize("name,mode", [("L1", "whole"), ("L1", "portions"), ("L1", "mixed"), ("L2", "decode_tail"),
                                       ("L2", "mixed"), ("L3", "portions"), ("L3", "mixed")])
def test_every_way_of_cutting_matches_plain(lanilorn_dirs, expected, name, mode):
    reqs, exp = expected[name]
    pool_tokens = traces.tokens_needed(reqs)
    runner = cpu_runner(lanilorn_dirs[name], name, pool_tokens // LANILORN_TINY[name]["page_tokens"])
    got = traces.replay(runner, getattr(traces, mode)(reqs))
    traces.compare(got, exp, atol=2e-4, rtol=5e-5)
    assert runner.manager.usage() == 0.0


def test_long_decoding_from_the_first_token(lanilorn_dirs):
    """150 tokens one by one from position 0: the windows pass over decoded tokens, the recurrent
    state is carried through every step."""
    reqs = traces.make_requests([150], 130, seed=21)
    exp = {r: pl.model_logits(lanilorn_dirs["L2"], t) for r, t in reqs.items()}
    runner = cpu_runner(lanilorn_dirs["L2"], "L2", 19)
    got = traces.replay(runner, traces.decode_tail(reqs, tail=150))
    traces.compare(got, exp, atol=2e-4, rtol=5e-5)


def test_greedy_generation_through_the_scheduler(lanilorn_dirs):
    from llmserve_b200 import LLM, SamplingParams

    prompts = [[5, 9, 100, 31, 7], list(range(40, 57)), [3] * 33, [100, 2]]
    m = LLM(str(lanilorn_dirs["L1"]), dtype="float32", device="cpu", ops=PlainOps(), block_size=16, num_kv_blocks=24,
            max_model_len=128, max_num_seqs=3, max_num_batched_tokens=24)
    outs = m.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for o, p in zip(outs, prompts):
        assert o.outputs[0].token_ids == pl.greedy(lanilorn_dirs["L1"], p, 8), p


def wanted_subsets(make_runner, folder, vocab):
    """Steps that want some rows, one row or none: the model's last norm then reads only those rows,
    and a step's last write into the streams is carried out without a read behind it."""
    from llmserve_b200.engine.batch import StepEntry

    reqs = traces.make_requests([41, 30], vocab, seed=13)
    exp = {r: pl.model_logits(folder, t) for r, t in reqs.items()}
    runner = make_runner()
    a, b = reqs["r0"], reqs["r1"]
    steps = [([("r0", a[:17], [3, 16]), ("r1", b[:9], [])], None),
             ([("r0", a[17:18], []), ("r1", b[9:22], [0, 12])], None),
             ([("r0", a[18:19], [0]), ("r1", b[22:23], [])], None),
             ([("r0", a[19:41], [21]), ("r1", b[23:30], [6, 2])], None)]
    at = {"r0": 0, "r1": 0}
    for entries, _ in steps:
        logits = runner.run([StepEntry(r, t, w) for r, t, w in entries]).float().cpu()
        row = 0
        for r, t, w in entries:
            for k in w:
                ref = exp[r][at[r] + k]
                assert (logits[row] - ref).abs().max().item() <= 2e-4 + 5e-5 * ref.abs().max().item(), (r, at[r] + k)
                row += 1
            at[r] += len(t)
        assert row == logits.shape[0]


@pytest.mark.parametrize("name", ["L1", "L2"])
def test_steps_that_want_some_rows_or_none(lanilorn_dirs, name):
    wanted_subsets(lambda: cpu_runner(lanilorn_dirs[name], name, 16), lanilorn_dirs[name], LANILORN_TINY[name]["config"]["vocab"])
