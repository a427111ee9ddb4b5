"""Typed configuration of the Lanilorn architecture, read from its ``config.json``.

The file names the architecture (``"architecture": "Lanilorn"``), ``vocab``, ``width``, the epsilon
of every norm (``norm.eps``), the factor on the embedded tokens (``embedding.scale``), the factor on
the logits (``logit_scale``), the number of residual streams (``streams``) and a list ``layers``.
Each entry has ``type`` (the mixer), the mixer's sizes under ``mixer`` and its feed-forward under
``mlp`` (null: none). The mixers:

* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim`` (the values are the keys as projected,
  so it equals ``dim``), ``scale``, optionally ``mask.size`` (a window) and ``rot`` (``base``,
  ``dims`` and optionally ``scaling`` with ``factor``, ``original``, ``fast``, ``slow``);
* ``attention_2`` (two softmax maps per head, the second subtracted): ``heads``, ``kv_heads``,
  ``dim``, ``vdim``, ``scale``, ``diff`` and optionally ``q_temp`` (``coef``, ``every``);
* ``gla`` (linear attention with a decay per key channel and token): ``heads``, ``dim``, ``vdim``,
  ``tau``.

The feed-forward is ``{"kind": "dense", "ff": n}``. Layers may differ in kind and in every size. A
required key that is absent is an error, and so is a key that this engine does not know, because
it would change the math silently.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .gubotar import _take
from .llama import ConfigError
from .pazivik import _take_some

MIXER_TYPES = ("attention", "attention_2", "gla")


@dataclass(frozen=True)
class YarnConfig:
    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self):
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class WindowedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int  # 0: every earlier token
    rot_dims: int  # 0: no rotation
    rot_base: float
    yarn: YarnConfig | None

    @classmethod
    def from_dict(cls, d, where):
        heads, kv, dim, vdim, scale, mask, rot = _take_some(
            d, ("heads", "kv_heads", "dim", "vdim", "scale"), ("mask", "rot"), where)
        if min(int(heads), int(kv), int(dim)) < 1 or int(heads) % int(kv):
            raise ConfigError(f"{where}: sizes must be positive and heads a multiple of kv_heads")
        if int(vdim) != int(dim):
            raise ConfigError(f"{where}: the values are the projected keys, so vdim must equal dim")
        window = 0
        if mask is not None:
            (window,) = _take(mask, ("size",), where + ".mask")
            if int(window) < 1:
                raise ConfigError(f"{where}.mask: size must be positive")
        dims, base, yarn = 0, 10000.0, None
        if rot is not None:
            base, dims, scaling = _take_some(rot, ("base", "dims"), ("scaling",), where + ".rot")
            if int(dims) % 2 or not 0 <= int(dims) <= int(dim) or float(base) <= 1.0:
                raise ConfigError(f"{where}.rot: dims must be even and at most dim, base above one")
            if scaling is not None:
                f, fast, orig, slow = _take(scaling, ("factor", "fast", "original", "slow"), where + ".rot.scaling")
                if float(f) <= 0 or float(orig) <= 0 or float(fast) <= 0 or float(slow) <= 0:
                    raise ConfigError(f"{where}.rot.scaling: every number must be positive")
                yarn = YarnConfig(float(f), float(orig), float(fast), float(slow))
        return cls(int(heads), int(kv), int(dim), int(vdim), float(scale), int(window), int(dims), float(base), yarn)

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.yarn is not None:
                d["rot"]["scaling"] = self.yarn.to_dict()
        return d


@dataclass(frozen=True)
class DifferentialAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    temp_coef: float
    temp_every: int  # 0: no query temperature

    @classmethod
    def from_dict(cls, d, where):
        heads, kv, dim, vdim, scale, diff, q_temp = _take_some(
            d, ("heads", "kv_heads", "dim", "vdim", "scale", "diff"), ("q_temp",), where)
        if min(int(heads), int(kv), int(dim), int(vdim)) < 1 or int(heads) % int(kv):
            raise ConfigError(f"{where}: sizes must be positive and heads a multiple of kv_heads")
        coef, every = 0.0, 0
        if q_temp is not None:
            coef, every = _take(q_temp, ("coef", "every"), where + ".q_temp")
            if int(every) < 1:
                raise ConfigError(f"{where}.q_temp: every must be positive")
        return cls(int(heads), int(kv), int(dim), int(vdim), float(scale), float(diff), float(coef), int(every))

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
             "scale": self.scale, "diff": self.diff}
        if self.temp_every:
            d["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
        return d


@dataclass(frozen=True)
class GatedLinearAttentionConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    # inner size of the two decay matrices. A file need not name it: a model folder gives it by
    # the shape of the layer's first decay matrix (``from_pretrained``); 0: not known.
    decay_rank: int = 0

    @classmethod
    def from_dict(cls, d, where):
        heads, dim, vdim, tau, rank = _take_some(d, ("heads", "dim", "vdim", "tau"), ("decay_rank",), where)
        if min(int(heads), int(dim), int(vdim)) < 1 or float(tau) <= 0 or int(rank or 0) < 0:
            raise ConfigError(f"{where}: sizes and tau must be positive")
        return cls(int(heads), int(dim), int(vdim), float(tau), int(rank or 0))

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.decay_rank:
            d["decay_rank"] = self.decay_rank
        return d


_MIXER_CONFIGS = {"attention": WindowedAttentionConfig, "attention_2": DifferentialAttentionConfig,
                  "gla": GatedLinearAttentionConfig}


@dataclass(frozen=True)
class LanilornLayerConfig:
    type: str
    mixer: Any
    ff: int  # 0: no feed-forward

    @classmethod
    def from_dict(cls, d, where):
        kind, mixer, mlp = _take(d, ("type", "mixer", "mlp"), where)
        if kind not in _MIXER_CONFIGS:
            raise ConfigError(f"{where}: layer type {kind!r} is not known (known: {MIXER_TYPES})")
        ff = 0
        if mlp is not None:
            mlp_kind, ff = _take(mlp, ("kind", "ff"), where + ".mlp")
            if mlp_kind != "dense" or int(ff) < 1:
                raise ConfigError(f"{where}.mlp: kind must be 'dense' and ff positive")
        return cls(kind, _MIXER_CONFIGS[kind].from_dict(mixer, where + ".mixer"), int(ff))

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": {"kind": "dense", "ff": self.ff} if self.ff else None}


@dataclass(frozen=True)
class LanilornConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embed_scale: float
    logit_scale: float
    streams: int
    layers: tuple[LanilornLayerConfig, ...]

    architecture = "Lanilorn"
    max_position_embeddings = 1 << 17  # rotation tables are made for as many positions as the engine runs
    tie_word_embeddings = True
    eos_token_ids: tuple[int, ...] = ()

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def num_parameters(self) -> int:
        from ..models.lanilorn import lanilorn_checkpoint_layout

        total = 0
        for entry in lanilorn_checkpoint_layout(self).entries:
            for src in entry.sources:
                n = 1
                for k in src.shape:
                    n *= k
                total += n
        return total

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "LanilornConfig":
        required = ("architecture", "embedding", "layers", "logit_scale", "norm", "streams", "vocab", "width")
        # keys beside these at the top describe the file, not the model (a name, a seed)
        arch, emb, layers, logit_scale, norm, streams, vocab, width = _take(
            {k: v for k, v in d.items() if k in required}, required, "config")
        if arch != cls.architecture:
            raise ConfigError(f"config: architecture {arch!r} is not {cls.architecture!r}")
        (eps,) = _take(norm, ("eps",), "config.norm")
        (scale,) = _take(emb, ("scale",), "config.embedding")
        if not layers:
            raise ConfigError("config: no layers")
        if int(streams) < 1 or int(vocab) < 1 or int(width) < 1:
            raise ConfigError("config: streams, vocab and width must be positive")
        out = tuple(LanilornLayerConfig.from_dict(l, f"config.layers[{i}]") for i, l in enumerate(layers))
        return cls(int(vocab), int(width), float(eps), float(scale), float(logit_scale), int(streams), out)

    @classmethod
    def from_pretrained(cls, path: str | Path) -> "LanilornConfig":
        """The folder's ``config.json``; a size that only a tensor's shape gives (the inner size
        of a ``gla`` layer's decay matrices) is read from the folder's safetensors headers."""
        d = json.loads((Path(path) / "config.json").read_text())
        layers = d.get("layers")
        open_ranks = [i for i, l in enumerate(layers if isinstance(layers, list) else [])
                      if isinstance(l, dict) and l.get("type") == "gla" and isinstance(l.get("mixer"), dict)
                      and not l["mixer"].get("decay_rank")]
        if open_ranks:
            from ..weights.loader import checkpoint_index

            index = checkpoint_index(path)
            for i in open_ranks:
                found = index.get(f"l{i}.mix.a1")
                if found is not None and len(found[1]) == 2:
                    layers[i] = dict(layers[i], mixer=dict(layers[i]["mixer"], decay_rank=int(found[1][0])))
        return cls.from_dict(d)

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "embedding": {"scale": self.embed_scale},
                "layers": [l.to_dict() for l in self.layers], "logit_scale": self.logit_scale,
                "norm": {"eps": self.norm_eps}, "streams": self.streams,
                "vocab": self.vocab_size, "width": self.hidden_size}
