"""The Lanilorn architecture as data: which parts each layer has and where its tensors come from.

The embedded token is its row of the embedding table times a constant; the residual state is
several streams (``streams`` blocks: every sublayer reads a weighted sum of the streams through an
RMS norm and writes its result, scaled per channel, back into all of them). The mixer is one of

* ``attention``: grouped query heads whose values are the keys as projected; queries and keys
  normed over the whole projection, part of each head rotated (optionally with stretched slow
  frequencies), a sliding window, a sink per head in the softmax, a sigmoid gate per head;
* ``attention_2``: two softmax maps per head over the same values, the second subtracted with a
  learned weight, the difference divided by its root mean square; a query temperature that grows
  with the position; a sigmoid gate per head;
* ``gla``: linear attention with a decay per key channel made from the token through two small
  matrices, a norm per head and a SiLU gate.

The feed-forward is ``Wdown relu(Wup h)^2`` or absent. The model's last norm reads the sum of the
streams; the output projection is the embedding table, and the logits are multiplied by a constant.

Checkpoint tensors are named ``l<i>.<part>``; the matrices of one product are concatenated along
their rows (q | k | g; q | k | v | g).
"""

from __future__ import annotations

from ..config.lanilorn import LanilornConfig
from ..parts.attention import AttentionSpec
from ..parts.differential_attention import DifferentialAttentionSpec
from ..parts.feed_forward import MLPSpec
from ..parts.linear_attention import GatedLinearAttentionSpec
from ..parts.positions import NoPositionSpec, RotarySpec
from ..parts.streams import StreamsBlockSpec, StreamsRMSNormSpec
from .plan import CheckpointLayout, ModelPlan, ParamSource, RunEntry, Source


def _mixer_spec(l, w: int, eps: float):
    m = l.mixer
    if l.type == "attention":
        position = NoPositionSpec()
        if m.rot_dims:
            position = RotarySpec(head_dim=m.rot_dims, theta=m.rot_base)
            if m.yarn is not None:
                position = RotarySpec(
                    head_dim=m.rot_dims, theta=m.rot_base, scaling_type="yarn", factor=m.yarn.factor,
                    original_max_positions=m.yarn.original, yarn_fast=m.yarn.fast, yarn_slow=m.yarn.slow)
        return AttentionSpec(
            hidden_size=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
            position=position, window=m.window, qk_norm_eps=eps, qk_norm_scope="row", values_are_keys=True,
            gate="head", sinks=True)
    if l.type == "attention_2":
        return DifferentialAttentionSpec(
            hidden_size=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
            scale=m.scale, eps=eps, lam_offset=m.diff, out_scale=1.0 - m.diff, temp_coef=m.temp_coef,
            temp_every=m.temp_every)
    if m.decay_rank < 1:
        raise ValueError("gla: the inner size of the decay matrices is not known (it is read from the "
                         "checkpoint's tensor shapes, or given as mixer.decay_rank)")
    return GatedLinearAttentionSpec(
        hidden_size=w, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, decay_rank=m.decay_rank, tau=m.tau,
        eps=eps, query_scale=m.dim ** -0.5)


def lanilorn_plan(cfg: LanilornConfig) -> ModelPlan:
    w, eps, n = cfg.hidden_size, cfg.norm_eps, cfg.streams
    read_norm = StreamsRMSNormSpec(w, eps, n)
    layers = []
    for l in cfg.layers:
        ff = MLPSpec(w, l.ff, activation="relu2") if l.ff else None
        layers.append(StreamsBlockSpec(streams=n, norm_in=read_norm, mixer=_mixer_spec(l, w, eps),
                                       norm_post=read_norm if ff is not None else None, feed_forward=ff))
    return ModelPlan(
        vocab_size=cfg.vocab_size, hidden_size=w, layers=tuple(layers),
        run_order=tuple(RunEntry(i, i) for i in range(len(layers))),
        final_norm=StreamsRMSNormSpec(w, eps, n, learned_read=False), tie_head=True,
        embed_scale=cfg.embed_scale, logit_scale=cfg.logit_scale, residual_streams=n)


def lanilorn_checkpoint_layout(cfg: LanilornConfig) -> CheckpointLayout:
    w, n = cfg.hidden_size, cfg.streams
    entries = [
        ParamSource("embed.weight", (Source("embed", (cfg.vocab_size, w)),), "embedding"),
        ParamSource("final_norm.weight", (Source("final.norm", (w,)),), "scale"),
    ]
    for i, l in enumerate(cfg.layers):
        src, dst, m = f"l{i}.", f"layers.{i}.", l.mixer
        subs = [("1", "norm_in", "mixer_write")] + ([("2", "norm_post", "ff_write")] if l.ff else [])
        for q, norm, write in subs:
            entries += [
                ParamSource(f"{dst}{norm}.weight", (Source(f"{src}norm{q}", (w,)),), "scale"),
                ParamSource(f"{dst}{norm}.read", (Source(f"{src}hc{q}.in", (n,)),), "mix"),
                ParamSource(f"{dst}{write}.mix", (Source(f"{src}hc{q}.mix", (n, n)),), "mix"),
                ParamSource(f"{dst}{write}.out", (Source(f"{src}hc{q}.out", (n,)),), "scale"),
                ParamSource(f"{dst}{write}.scale", (Source(f"{src}ls{q}", (w,)),), "scale"),
            ]
        ms, md = src + "mix.", dst + "mixer."
        if l.type == "attention":
            q, k = m.heads * m.dim, m.kv_heads * m.dim
            entries += [
                ParamSource(md + "qkv.weight", (Source(ms + "q", (q, w)), Source(ms + "k", (k, w)),
                                                Source(ms + "g", (m.heads, w)))),
                ParamSource(md + "q_norm.weight", (Source(ms + "q.norm", (q,)),), "scale"),
                ParamSource(md + "k_norm.weight", (Source(ms + "k.norm", (k,)),), "scale"),
                ParamSource(md + "sinks", (Source(ms + "sink", (m.heads,)),), "scale"),
                ParamSource(md + "o.weight", (Source(ms + "o", (w, m.heads * m.vdim)),)),
            ]
        elif l.type == "attention_2":
            q, k, v = 2 * m.heads * m.dim, 2 * m.kv_heads * m.dim, m.kv_heads * m.vdim
            entries += [
                ParamSource(md + "qkv.weight", (Source(ms + "q", (q, w)), Source(ms + "k", (k, w)),
                                                Source(ms + "v", (v, w)), Source(ms + "g", (m.heads, w)))),
                ParamSource(md + "o.weight", (Source(ms + "o", (w, m.heads * m.vdim)),)),
            ]
            entries += [ParamSource(f"{md}lam.{a}{b}", (Source(f"{ms}l{a}{b}", (m.dim,)),), "offset")
                        for b in "12" for a in "qk"]
        else:
            qk, vg = m.heads * m.dim, m.heads * m.vdim
            entries += [
                ParamSource(md + "qkvg.weight", (Source(ms + "q", (qk, w)), Source(ms + "k", (qk, w)),
                                                 Source(ms + "v", (vg, w)), Source(ms + "g", (vg, w)))),
                ParamSource(md + "decay_in.weight", (Source(ms + "a1", (m.decay_rank, w)),)),
                ParamSource(md + "decay_out.weight", (Source(ms + "a2", (qk, m.decay_rank)),)),
                ParamSource(md + "decay_out.bias", (Source(ms + "a2.b", (qk,)),), "bias"),
                ParamSource(md + "norm.weight", (Source(ms + "norm", (m.vdim,)),), "scale"),
                ParamSource(md + "o.weight", (Source(ms + "o", (w, vg)),)),
            ]
        if l.ff:
            fs, fd = src + "mlp.", dst + "feed_forward."
            entries += [
                ParamSource(fd + "up.weight", (Source(fs + "up", (l.ff, w)),)),
                ParamSource(fd + "down.weight", (Source(fs + "down", (w, l.ff)),)),
            ]
    return CheckpointLayout(entries=tuple(entries))
