"""Typed configuration of the Rirovik architecture, read from its ``config.json``.

The file names the architecture (``"architecture": "Rirovik"``), ``vocab``, ``width``, the epsilon
of every norm (``norm.eps``), the factor on the embedded tokens (``embedding.scale``) and a list
``layers``. Each entry has ``type`` (the mixer), the mixer's sizes under ``mixer`` and its
feed-forward under ``mlp`` (null: none). The mixers:

* ``latent_attention`` and ``latent_attention_2``: ``heads``, ``dim``, ``rot_dim``, ``vdim``,
  ``kv_rank``, ``q_rank``, ``scale``, ``rot`` (``base``, ``dims``); ``latent_attention`` also has
  ``mask.size`` (its window) and an output gate per head; ``latent_attention_2`` sees every
  earlier token and has no gate. Either may have ``kv_from``: the earlier layer whose cached rows
  it reads instead of making its own;
* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask`` (``size`` and,
  optionally, ``keep_first``; without ``mask`` every earlier token is seen).

The feed-forward is ``{"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}, "shared":
{"ff"}}`` (``shared`` may be absent or null). Layers may differ in kind and in every size. A key
that is absent is an error, and so is a key that this engine does not know, because it would
change the math silently.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .gubotar import _take
from .llama import ConfigError
from .pazivik import _take_some

LATENT_TYPES = ("latent_attention", "latent_attention_2")


def _mask(mask, where: str, optional: tuple[str, ...] = ()) -> list[int]:
    values = _take_some(mask, ("size",), optional, where + ".mask")
    out = [int(v or 0) for v in values]
    if out[0] < 1 or min(out) < 0:
        raise ConfigError(f"{where}.mask: size must be positive and nothing negative")
    return out


@dataclass(frozen=True)
class RirovikLatentConfig:
    heads: int
    dim: int  # query/key dims of a head that are not rotated
    rot_dim: int  # rotated dims of a head, and of the key part all heads share
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int  # how many of the rotated part's dims are turned
    window: int  # 0: every earlier token
    kv_from: int | None

    @classmethod
    def from_dict(cls, d, where, windowed: bool):
        required = ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot")
        optional = ("kv_from", "mask") if windowed else ("kv_from",)
        heads, dim, rot_dim, vdim, rank, q_rank, scale, rot, kv_from, *rest = _take_some(d, required, optional, where)
        mask = rest[0] if windowed else None
        base, dims = _take(rot, ("base", "dims"), where + ".rot")
        window = _mask(mask, where)[0] if mask is not None else 0
        if windowed and not window:
            raise ConfigError(f"{where}: a windowed layer needs mask.size")
        if min(int(heads), int(dim), int(vdim), int(rank), int(q_rank)) < 1 or int(rot_dim) < 0:
            raise ConfigError(f"{where}: sizes must be positive")
        if int(dims) % 2 or not 0 <= int(dims) <= int(rot_dim):
            raise ConfigError(f"{where}.rot: dims must be even and at most rot_dim")
        return cls(int(heads), int(dim), int(rot_dim), int(vdim), int(rank), int(q_rank), float(scale),
                   float(base), int(dims), window, None if kv_from is None else int(kv_from))

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
             "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale,
             "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class RirovikAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    keep_first: int

    @classmethod
    def from_dict(cls, d, where):
        heads, kv, dim, vdim, scale, mask = _take_some(d, ("heads", "kv_heads", "dim", "vdim", "scale"), ("mask",), where)
        window, keep = _mask(mask, where, ("keep_first",)) if mask is not None else (0, 0)
        if min(int(heads), int(kv), int(dim), int(vdim)) < 1 or int(heads) % int(kv):
            raise ConfigError(f"{where}: sizes must be positive and heads a multiple of kv_heads")
        return cls(int(heads), int(kv), int(dim), int(vdim), float(scale), window, keep)

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
            if self.keep_first:
                d["mask"]["keep_first"] = self.keep_first
        return d


@dataclass(frozen=True)
class RirovikMlpConfig:
    experts: int
    top: int
    ff: int
    shared_ff: int = 0  # 0: no shared expert

    @classmethod
    def from_dict(cls, d, where):
        kind, router, expert, shared = _take_some(d, ("kind", "router", "expert"), ("shared",), where)
        if kind != "moe":
            raise ConfigError(f"{where}: kind {kind!r} is not known (known: 'moe')")
        experts, top = _take(router, ("experts", "top"), where + ".router")
        (ff,) = _take(expert, ("ff",), where + ".expert")
        shared_ff = 0
        if shared is not None:
            (shared_ff,) = _take(shared, ("ff",), where + ".shared")
        if not 1 <= int(top) <= int(experts) or int(ff) < 1 or int(shared_ff) < 0:
            raise ConfigError(f"{where}: top must lie between 1 and experts, and sizes be positive")
        return cls(int(experts), int(top), int(ff), int(shared_ff))

    def to_dict(self):
        d = {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class RirovikLayerConfig:
    type: str
    mixer: Any  # RirovikLatentConfig | RirovikAttentionConfig
    mlp: RirovikMlpConfig | None

    @classmethod
    def from_dict(cls, d, where):
        kind, mixer, mlp = _take(d, ("type", "mixer", "mlp"), where)
        if kind in LATENT_TYPES:
            m = RirovikLatentConfig.from_dict(mixer, where + ".mixer", windowed=kind == "latent_attention")
        elif kind == "attention":
            m = RirovikAttentionConfig.from_dict(mixer, where + ".mixer")
        else:
            raise ConfigError(f"{where}: layer type {kind!r} is not known (known: {LATENT_TYPES + ('attention',)})")
        return cls(kind, m, None if mlp is None else RirovikMlpConfig.from_dict(mlp, where + ".mlp"))

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class RirovikConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embed_scale: float
    layers: tuple[RirovikLayerConfig, ...]

    architecture = "Rirovik"
    max_position_embeddings = 1 << 17  # rotation tables are made for as many positions as the engine runs
    tie_word_embeddings = False
    eos_token_ids: tuple[int, ...] = ()

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def num_parameters(self) -> int:
        from ..models.rirovik import rirovik_checkpoint_layout

        total = 0
        for entry in rirovik_checkpoint_layout(self).entries:
            for src in entry.sources:
                n = 1
                for k in src.shape:
                    n *= k
                total += n
        return total

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "RirovikConfig":
        required = ("architecture", "embedding", "layers", "norm", "vocab", "width")
        # keys beside these at the top describe the file, not the model (a name, a seed)
        arch, emb, layers, norm, vocab, width = _take({k: v for k, v in d.items() if k in required}, required, "config")
        if arch != cls.architecture:
            raise ConfigError(f"config: architecture {arch!r} is not {cls.architecture!r}")
        (eps,) = _take(norm, ("eps",), "config.norm")
        (scale,) = _take(emb, ("scale",), "config.embedding")
        if not layers:
            raise ConfigError("config: no layers")
        out = tuple(RirovikLayerConfig.from_dict(l, f"config.layers[{i}]") for i, l in enumerate(layers))
        for i, l in enumerate(out):
            j = getattr(l.mixer, "kv_from", None)
            if j is None:
                continue
            where = f"config.layers[{i}].mixer"
            if not 0 <= j < i or out[j].type not in LATENT_TYPES or out[j].mixer.kv_from is not None:
                raise ConfigError(f"{where}: kv_from must name an earlier latent layer with a latent of its own")
            a, b = out[j].mixer, l.mixer
            if (a.kv_rank, a.rot_dim, a.rot_dims, a.rot_base) != (b.kv_rank, b.rot_dim, b.rot_dims, b.rot_base):
                raise ConfigError(f"{where}: kv_rank, rot_dim or rot differ from layer {j}'s")
        return cls(int(vocab), int(width), float(eps), float(scale), out)

    @classmethod
    def from_pretrained(cls, path: str | Path) -> "RirovikConfig":
        return cls.from_dict(json.loads((Path(path) / "config.json").read_text()))

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "embedding": {"scale": self.embed_scale},
                "layers": [l.to_dict() for l in self.layers], "norm": {"eps": self.norm_eps},
                "vocab": self.vocab_size, "width": self.hidden_size}
