"""Shared fixtures: tiny random-weight Llama folders, written fresh into a temporary folder."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

# Tiny configurations that differ in every size and option.
TINY = {
    "A": dict(vocab_size=256, hidden_size=64, intermediate_size=160, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, rope_theta=10000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=256, seed=0,
              page_tokens=16),
    "B": dict(vocab_size=384, hidden_size=128, intermediate_size=352, num_hidden_layers=3,
              num_attention_heads=4, num_key_value_heads=1, head_dim=32, rope_theta=100000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=512, seed=2,
              page_tokens=8),
    # head size 64 (the tensor-core attention path), three query heads per key head, widths that
    # are no power of two, untied head, attention biases
    "C": dict(vocab_size=515, hidden_size=192, intermediate_size=272, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, rope_theta=50000.0,
              rms_norm_eps=3e-6, tie_word_embeddings=False, attention_bias=True,
              max_position_embeddings=1024, seed=7, page_tokens=32),
}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def tiny_config(name: str):
    from llmserve_b200.config import LlamaConfig

    d = {k: v for k, v in TINY[name].items() if k not in ("seed", "page_tokens")}
    return LlamaConfig.from_dict({"model_type": "llama", **d})


@pytest.fixture(scope="session")
def tiny_dirs(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (bfloat16 storage)."""
    from llmserve_b200.weights import write_random_model

    out = {}
    for name, spec in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny-{name}")
        write_random_model(d, tiny_config(name), spec["seed"])
        out[name] = d
    return out


@pytest.fixture(scope="session")
def sharp_dirs(tmp_path_factory):
    """Same shapes, weights scaled up so that logits are far from flat (argmax ties unlikely)."""
    from safetensors.torch import load_file, save_file

    from llmserve_b200.weights import write_random_model

    out = {}
    for name, spec in TINY.items():
        d = tmp_path_factory.mktemp(f"sharp-{name}")
        write_random_model(d, tiny_config(name), spec["seed"] + 100)
        f = d / "model.safetensors"
        t = load_file(str(f))
        t = {k: (v.float() * 6).to(v.dtype) if v.dim() > 1 else v for k, v in t.items()}
        save_file(t, str(f))
        out[name] = d
    return out


# ---- Gubotar: small configurations that differ in every size, option and in the order of layers.
def _ret(heads, dim, vdim, decay, rot, base, ff):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
                                            "rot": {"dims": rot, "base": base}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _par(heads, kv, dim, scale, chunk, rheads, rdim, rvdim, decay, ff):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale,
                               "mask": {"size": chunk}},
                      "right": {"heads": rheads, "dim": rdim, "vdim": rvdim, "decay": decay}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


GUBOTAR_TINY = {
    # retention first; partial rotation; value size unlike key size; a layer without feed-forward;
    # grouped key heads; a chunk that is no multiple of the page
    "G1": dict(seed=3, page_tokens=16, config={
        "architecture": "Gubotar", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
        "layers": [_ret(3, 16, 32, [0.9, 0.97, 0.995], 8, 10000.0, 160),
                   _par(4, 2, 16, 0.6, 24, 2, 24, 40, [0.8, 0.99], 0),
                   _ret(2, 48, 16, [0.999, 0.5], 48, 500.0, 64)]}),
    # a head size that is no multiple of 16; one key head; a chunk shorter than a page; one
    # linear-attention head; width and vocabulary that are no multiples of 8
    "G2": dict(seed=9, page_tokens=8, config={
        "architecture": "Gubotar", "vocab": 130, "width": 68, "norm": {"eps": 1e-6},
        "layers": [_par(2, 1, 40, 0.35, 7, 1, 20, 64, [0.95], 96),
                   _par(6, 6, 16, 0.5, 33, 4, 8, 8, [0.9, 0.99, 0.999, 0.3], 48)]}),
    # sizes that are multiples of nothing: width 70, head sizes 24, 10, 12 and 20, six rotated dims
    # of ten, four query heads on one key head, a chunk of one page, a single layer kind first
    "G3": dict(seed=14, page_tokens=16, config={
        "architecture": "Gubotar", "vocab": 97, "width": 70, "norm": {"eps": 1e-5},
        "layers": [_par(4, 1, 24, 0.4, 16, 3, 12, 20, [0.97, 0.9, 0.999], 50),
                   _ret(5, 10, 14, [0.9, 0.95, 0.99, 0.995, 0.999], 6, 777.0, 0),
                   _par(2, 2, 32, 0.2, 1, 2, 10, 36, [0.5, 0.9], 30)]}),
    # retention layers only: the model keeps no pages at all; two rotated dims of 32
    "G4": dict(seed=21, page_tokens=16, config={
        "architecture": "Gubotar", "vocab": 64, "width": 32, "norm": {"eps": 1e-6},
        "layers": [_ret(2, 16, 16, [0.9, 0.99], 16, 1e4, 48), _ret(1, 32, 8, [0.95], 2, 1e4, 0)]}),
}


def write_gubotar(folder, name, spread=True):
    """A random Gubotar folder. ``spread``: per-channel weights, temperatures and stored-around-zero
    norm weights are drawn wide, so that leaving one of them out changes the logits clearly."""
    from safetensors.torch import load_file, save_file

    from llmserve_b200.config.gubotar import GubotarConfig
    from llmserve_b200.weights import write_random_model

    spec = GUBOTAR_TINY[name]
    write_random_model(folder, GubotarConfig.from_dict(spec["config"]), spec["seed"])
    if spread:
        f = folder / "model.safetensors"
        t = load_file(str(f))
        g = torch.Generator().manual_seed(spec["seed"] + 1)
        for k, v in t.items():
            if v.dim() == 1 and not k.endswith("shift"):
                around = 0.0 if (k.endswith("norm1") or k.endswith("norm2") or k == "final.norm") else 1.0
                t[k] = (around + (torch.rand(v.shape, generator=g) - 0.5)).to(v.dtype)
            elif k == "embed":
                t[k] = (v.float() * 40).to(v.dtype)
        save_file(t, str(f))
    return folder


@pytest.fixture(scope="session")
def gubotar_dirs(tmp_path_factory):
    return {name: write_gubotar(tmp_path_factory.mktemp(f"gubotar-{name}"), name) for name in GUBOTAR_TINY}


# ---- Pazivik: small configurations that differ in every size, in the order of layers and in which
# optional thing is there.
def _lat(heads, dim, vdim, rank, scale, window, mlp, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _moe(experts, top, ff, shared):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def _dense(ff):
    return {"kind": "dense", "ff": ff}


PAZIVIK_TINY = {
    # a reader whose window is wider than its writer's; two experts per token; a latent rank that
    # is no multiple of 16; a layer without feed-forward; experts without a shared one
    "P1": dict(seed=4, page_tokens=16, config={
        "architecture": "Pazivik", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
        "embedding": {"bigram": {"buckets": 97, "mul_cur": 5, "mul_prev": 31}},
        "layers": [_lat(3, 16, 24, 32, 0.3, 20, _dense(160)),
                   _lat(2, 32, 8, 32, 0.2, 33, _moe(5, 2, 24, 40), kv_from=0),
                   _lat(4, 8, 16, 40, 0.5, 7, None),
                   _lat(1, 48, 20, 40, 0.15, 7, _moe(3, 1, 32, 0), kv_from=2)]}),
    # widths that are multiples of nothing; a window shorter than a page; a layer without a mask;
    # every expert chosen; one bucket; no soft cap; a reader that follows its writer at a distance
    "P2": dict(seed=11, page_tokens=8, config={
        "architecture": "Pazivik", "vocab": 130, "width": 70, "norm": {"eps": 1e-6},
        "embedding": {"bigram": {"buckets": 1, "mul_cur": 3, "mul_prev": 2}},
        "layers": [_lat(1, 24, 20, 16, 0.25, 5, _dense(50)),
                   _lat(5, 8, 12, 48, 0.4, 0, _moe(4, 4, 10, 16)),
                   _lat(2, 20, 6, 16, 0.3, 9, _dense(30), kv_from=0)]}),
    # the head and latent sizes of larger models; many experts; a window of exactly one page and
    # one of several pages; big multipliers of the bigram hash
    "P3": dict(seed=17, page_tokens=32, sharp=8, config={
        "architecture": "Pazivik", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "logit_softcap": 50.0,
        "embedding": {"bigram": {"buckets": 509, "mul_cur": 1000003, "mul_prev": 999983}},
        "layers": [_lat(8, 64, 32, 128, 0.125, 32, _moe(16, 3, 48, 64)),
                   _lat(4, 32, 64, 64, 0.18, 100, _dense(192)),
                   _lat(6, 16, 16, 64, 0.25, 64, _moe(2, 1, 64, 8), kv_from=1)]}),
    # a latent rank beyond the attention kernels' head sizes: keys and values are kept per head,
    # and the layer that reads another's latent rows is handed them within the step
    "P4": dict(seed=23, page_tokens=16, sharp=6, config={
        "architecture": "Pazivik", "vocab": 150, "width": 80, "norm": {"eps": 1e-5}, "logit_softcap": 15.0,
        "embedding": {"bigram": {"buckets": 53, "mul_cur": 11, "mul_prev": 7}},
        "layers": [_lat(2, 16, 24, 272, 0.25, 12, _dense(96)),
                   _lat(3, 8, 8, 272, 0.35, 30, _moe(3, 1, 16, 0), kv_from=0),
                   _lat(2, 24, 16, 48, 0.2, 9, None)]}),
}


def write_pazivik(folder, name):
    """A random Pazivik folder whose weights are drawn wide: attention is far from flat, sinks,
    norms and gates differ clearly from head to head, so that leaving one of them out, or reading
    a key too many, changes the logits clearly.

    No routing decision is a close call (a model computed in bfloat16 must pick the same experts
    as the float64 one): the last dims of the residual stream carry, for every token, one of
    evenly spaced levels per expert, in an order that depends on the token; no layer writes
    those dims, and each router row reads its expert's dim with weight one beside small random
    weights on all the others."""
    from safetensors.torch import load_file, save_file

    from llmserve_b200.config.pazivik import PazivikConfig
    from llmserve_b200.weights import write_random_model

    spec = PAZIVIK_TINY[name]
    write_random_model(folder, PazivikConfig.from_dict(spec["config"]), spec["seed"])
    f = folder / "model.safetensors"
    t = load_file(str(f))
    g = torch.Generator().manual_seed(spec["seed"] + 1)
    for k, v in t.items():
        if k.endswith("sink"):
            t[k] = (4 * (torch.rand(v.shape, generator=g) - 0.5)).to(v.dtype)
        elif v.dim() == 1:
            t[k] = (1.0 + (torch.rand(v.shape, generator=g) - 0.5)).to(v.dtype)
        elif k in ("embed", "bigram"):
            t[k] = (v.float() * 40).to(v.dtype)
        elif k.endswith("mix.q") or k.endswith("mix.uk"):
            t[k] = (v.float() * spec.get("sharp", 10)).to(v.dtype)  # wider heads need less to be sharp
        else:
            t[k] = (v.float() * 8).to(v.dtype)
    cfg = spec["config"]
    width = cfg["width"]
    moe = [(i, l["mlp"]["router"]["experts"]) for i, l in enumerate(cfg["layers"])
           if l["mlp"] is not None and l["mlp"]["kind"] == "moe"]
    most = max(e for _, e in moe)
    step = next(m for m in (3, 5, 7, 11) if all(most % q or m % q for q in (2, 3, 5, 7, 11)))
    dims = [width - 2 * most + 2 * e for e in range(most)]  # even entries: the sinusoid adds next to nothing there
    spacing = 1.5 if most <= 8 else 1.0
    tok = torch.arange(cfg["vocab"])[:, None]
    levels = spacing * (((tok * 7 + step * torch.arange(most)[None, :]) % most).float() - (most - 1) / 2)
    t["embed"][:, dims] = levels.to(t["embed"].dtype)
    t["bigram"][:, dims] = 0
    for k in t:
        if k.endswith("mix.o") or k.endswith("down"):
            t[k][dims, :] = 0
    for i, experts in moe:
        t[f"l{i}.norm2"][dims] = 1
        router = torch.randn(experts, width, generator=g) * 0.002
        router[torch.arange(experts), dims[:experts]] = 1.0
        t[f"l{i}.mlp.router"] = router.to(torch.bfloat16)
    save_file(t, str(f))
    return folder


@pytest.fixture(scope="session")
def pazivik_dirs(tmp_path_factory):
    return {name: write_pazivik(tmp_path_factory.mktemp(f"pazivik-{name}"), name) for name in PAZIVIK_TINY}


# ---- Rirovik: small configurations that differ in every size, in the kinds and order of layers
# and in which optional thing is there.
def _rlat(kind, heads, dim, rot_dim, vdim, rank, q_rank, scale, base, mlp, window=0, kv_from=None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank,
         "scale": scale, "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": kind, "mixer": m, "mlp": mlp}


def _ratt(heads, kv, dim, vdim, scale, window, keep, mlp):
    mask = {"size": window}
    if keep:
        mask["keep_first"] = keep
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                                           "mask": mask}, "mlp": mlp}


RIROVIK_TINY = {
    # values wider and narrower than keys; a reader whose window is wider than its writer's; a
    # layer without feed-forward; experts without a shared one; every expert chosen; one expert
    "R1": dict(seed=3, page_tokens=16, config={
        "architecture": "Rirovik", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
        "layers": [_rlat("latent_attention_2", 3, 16, 8, 24, 40, 24, 0.3, 10000.0, _moe(5, 2, 24, 40)),
                   _rlat("latent_attention", 2, 32, 16, 8, 32, 48, 0.2, 500.0, _moe(3, 1, 32, 0), window=20),
                   _ratt(4, 2, 16, 32, 0.4, 12, 3, None),
                   _rlat("latent_attention", 4, 8, 16, 16, 32, 16, 0.35, 500.0, _moe(4, 4, 16, 8), window=33, kv_from=1)]}),
    # widths that are multiples of nothing; a window shorter than a page and one of a single
    # token; more kept first tokens than the window holds; no kept tokens; one key/value head per
    # query head; a rotated part of which only some dims turn; a cache row that needs padding
    "R2": dict(seed=12, page_tokens=8, config={
        "architecture": "Rirovik", "vocab": 130, "width": 70, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
        "layers": [_ratt(3, 3, 24, 10, 0.25, 5, 9, _moe(4, 2, 10, 16)),
                   _rlat("latent_attention_2", 5, 8, 4, 12, 22, 10, 0.4, 100.0, _moe(2, 1, 30, 6), rot_dims=2),
                   _rlat("latent_attention", 1, 20, 6, 6, 18, 14, 0.3, 30.0, None, window=1),
                   _ratt(2, 1, 12, 12, 0.3, 40, 0, _moe(3, 3, 8, 0)),
                   _rlat("latent_attention", 2, 12, 4, 20, 22, 9, 0.3, 100.0, _moe(4, 2, 12, 12), window=7, kv_from=1,
                         rot_dims=2)]}),
    # the head and latent sizes of larger models (a cache row beyond 128 dims); many experts;
    # windows of exactly one page and of several; four query heads per key/value head
    "R3": dict(seed=19, page_tokens=32, sharp=5, config={
        "architecture": "Rirovik", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 11.3},
        "layers": [_rlat("latent_attention", 8, 64, 32, 64, 128, 96, 0.1, 20000.0, _moe(16, 3, 48, 64), window=32),
                   _ratt(8, 2, 64, 64, 0.125, 100, 4, _moe(2, 1, 64, 8)),
                   _rlat("latent_attention_2", 4, 32, 16, 48, 48, 64, 0.15, 1000000.0, _moe(6, 2, 40, 0))]}),
}


def write_rirovik(folder, name):
    """A random Rirovik folder whose weights are drawn wide: attention is far from flat, norms,
    biases and gates differ clearly from dim to dim and head to head, so that leaving one of them
    out, or reading a key too many, changes the logits clearly.

    No routing decision is a close call (a model computed in bfloat16 must pick the same experts
    as the float64 one): the last dims of the residual stream carry, for every token, one of
    evenly spaced levels per expert, in an order that depends on the token; no layer writes
    those dims (the norms behind the sublayers multiply them by 1 + (-1)), and each router row
    reads its expert's dim with weight one beside small random weights on all the others."""
    from safetensors.torch import load_file, save_file

    from llmserve_b200.config.rirovik import RirovikConfig
    from llmserve_b200.weights import write_random_model

    spec = RIROVIK_TINY[name]
    write_random_model(folder, RirovikConfig.from_dict(spec["config"]), spec["seed"])
    f = folder / "model.safetensors"
    t = load_file(str(f))
    g = torch.Generator().manual_seed(spec["seed"] + 1)
    for k, v in t.items():
        if k.endswith("dq.norm") or k.endswith("dkv.norm"):
            t[k] = (1.0 + (torch.rand(v.shape, generator=g) - 0.5)).to(v.dtype)
        elif v.dim() == 1:  # norm offsets, biases
            t[k] = (torch.rand(v.shape, generator=g) - 0.5).to(v.dtype)
        elif k == "embed":
            t[k] = (v.float() * 40 / spec["config"]["embedding"]["scale"]).to(v.dtype)
        elif k.endswith(("mix.uq", "mix.uk", "mix.q", "mix.k")):
            t[k] = (v.float() * spec.get("sharp", 10)).to(v.dtype)  # wider heads need less to be sharp
        else:
            t[k] = (v.float() * 8).to(v.dtype)
    cfg = spec["config"]
    width = cfg["width"]
    moe = [(i, l["mlp"]["router"]["experts"]) for i, l in enumerate(cfg["layers"]) if l["mlp"] is not None]
    most = max(e for _, e in moe)
    step = next(m for m in (3, 5, 7, 11) if all(most % q or m % q for q in (2, 3, 5, 7, 11)))
    dims = [width - most + e for e in range(most)]
    tok = torch.arange(cfg["vocab"])[:, None]
    levels = 1.5 * (((tok * 7 + step * torch.arange(most)[None, :]) % most).float() - (most - 1) / 2)
    t["embed"][:, dims] = (levels / cfg["embedding"]["scale"]).to(t["embed"].dtype)
    for i, l in enumerate(cfg["layers"]):
        t[f"l{i}.norm1b"][dims] = -1
        if l["mlp"] is not None:
            t[f"l{i}.norm2b"][dims] = -1
    for i, experts in moe:
        t[f"l{i}.norm2"][dims] = 0
        router = torch.randn(experts, width, generator=g) * 0.002
        router[torch.arange(experts), dims[:experts]] = 1.0
        t[f"l{i}.mlp.router"] = router.to(torch.bfloat16)
        t[f"l{i}.mlp.router.b"] = (0.2 * (torch.rand(experts, generator=g) - 0.5)).to(torch.bfloat16)
    save_file(t, str(f))
    return folder


@pytest.fixture(scope="session")
def rirovik_dirs(tmp_path_factory):
    return {name: write_rirovik(tmp_path_factory.mktemp(f"rirovik-{name}"), name) for name in RIROVIK_TINY}


# ----------------------------------------------------------------------------- Lanilorn
def _latt(heads, kv, dim, scale, mlp, window=0, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _ldiff(heads, kv, dim, vdim, scale, diff, mlp, q_temp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def _lgla(heads, dim, vdim, tau, rank, mlp):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


LANILORN_TINY = {
    # two streams; a window shorter than a page with a third of each head rotated under stretched
    # frequencies; grouped key heads in both attention kinds; a layer without feed-forward
    "L1": dict(seed=4, page_tokens=16, config={
        "architecture": "Lanilorn", "vocab": 157, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
        "logit_scale": 0.5, "streams": 2,
        "layers": [_latt(4, 2, 32, 0.2, _dense(96), window=10,
                         rot={"base": 10000.0, "dims": 12, "scaling": {"factor": 4.0, "fast": 16.0, "original": 64, "slow": 2.0}}),
                   _lgla(2, 16, 24, 8.0, 8, None),
                   _ldiff(4, 2, 16, 32, 0.3, 0.3, _dense(80), q_temp=(0.4, 8)),
                   _lgla(3, 32, 16, 2.0, 4, _dense(48))]}),
    # sizes that are multiples of nothing; four streams; pages of 8 tokens; whole heads rotated
    # without stretching; one key head per query head, and one for all; keys wider than values
    "L2": dict(seed=9, page_tokens=8, config={
        "architecture": "Lanilorn", "vocab": 130, "width": 72, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.7},
        "logit_scale": 3.0, "streams": 4,
        "layers": [_lgla(3, 20, 12, 16.0, 5, _dense(50)),
                   _latt(3, 3, 24, 0.25, None, window=21, rot={"base": 500.0, "dims": 24}),
                   _ldiff(3, 1, 40, 24, 0.15, 0.7, None, q_temp=(1.0, 3)),
                   _latt(2, 1, 18, 0.3, _dense(30), window=3, rot={"base": 50.0, "dims": 6}),
                   _ldiff(2, 2, 10, 50, 0.4, 0.2, _dense(64))]}),
    # one stream; attention that sees everything and has no rotation; a window of one token; no
    # query temperature; a root of one
    "L3": dict(seed=21, page_tokens=16, config={
        "architecture": "Lanilorn", "vocab": 99, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
        "logit_scale": 1.0, "streams": 1,
        "layers": [_latt(2, 2, 16, 0.3, _dense(64)),
                   _ldiff(2, 1, 16, 16, 0.25, 0.5, None),
                   _lgla(1, 48, 64, 1.0, 3, _dense(32)),
                   _latt(6, 2, 16, 0.3, None, window=1, rot={"base": 100.0, "dims": 16,
                         "scaling": {"factor": 16.0, "fast": 4.0, "original": 32, "slow": 0.5}})]}),
}


def write_lanilorn(folder, name):
    """A random model folder whose queries and keys are sharp and whose small tensors (norm weights,
    stream weights, scales per channel, sinks, decay biases, the weights of the second map) differ
    clearly from one another, so that leaving one of them out, a key too many or a lost state
    changes the logits clearly."""
    from safetensors.torch import load_file, save_file

    from llmserve_b200.config.lanilorn import LanilornConfig
    from llmserve_b200.weights import write_random_model

    spec = LANILORN_TINY[name]
    write_random_model(folder, LanilornConfig.from_dict(spec["config"]), spec["seed"])
    f = folder / "model.safetensors"
    t = load_file(str(f))
    g = torch.Generator().manual_seed(spec["seed"] + 1)
    n = spec["config"]["streams"]
    for k, v in t.items():
        r = torch.rand(v.shape, generator=g)
        if k.endswith(".mix") and v.dim() == 2 and ".hc" in k:
            t[k] = (torch.eye(n) * 0.8 + (r - 0.3) * 0.5).to(v.dtype)
        elif ".hc" in k:  # read and write weights
            t[k] = (0.4 + r).to(v.dtype) * (1 if k.endswith(".in") else -1)
        elif k.endswith(".sink"):
            t[k] = (4 * r - 1).to(v.dtype)
        elif k.endswith("a2.b"):
            t[k] = (5 * r - 1).to(v.dtype)
        elif k.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            t[k] = (0.6 * (r - 0.5)).to(v.dtype)
        elif v.dim() == 1:  # norm weights, scales per channel
            t[k] = (0.5 + r).to(v.dtype)
        elif k == "embed":
            t[k] = (v.float() * 40).to(v.dtype)
        elif k.endswith(("mix.q", "mix.k")):
            t[k] = (v.float() * spec.get("sharp", 10)).to(v.dtype)
        elif k.endswith(("mix.a1", "mix.a2")):
            t[k] = (v.float() * 25).to(v.dtype)
        else:
            t[k] = (v.float() * 8).to(v.dtype)
    save_file(t, str(f))
    return folder


@pytest.fixture(scope="session")
def lanilorn_dirs(tmp_path_factory):
    return {name: write_lanilorn(tmp_path_factory.mktemp(f"lanilorn-{name}"), name) for name in LANILORN_TINY}
