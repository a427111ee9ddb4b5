"""The Rirovik architecture as data: which parts each layer has and where its tensors come from.

The embedded token is its row of the embedding table times a constant. Every layer is a
``sandwich`` block (a norm before and after each sublayer, each multiplying by one plus its stored weight).
The mixer is one of

* latent attention with a query latent, a rotated key part that all heads share, a window and a
  sigmoid gate per head; such a layer may read the rows an earlier layer cached instead of
  making its own (the two then share a cache layer, which keeps the larger of their windows);
* the same without window and gate (every earlier token is seen);
* attention of grouped query heads with biases on q, k and v, q and k divided by their root mean
  square, no positions, a window that also keeps the sequence's first tokens, and a sigmoid gate
  per element of the heads' output.

The feed-forward is a set of routed experts (router with a bias, softmax over the chosen logits,
the weight on the expert's output, experts ``Wdown relu(Wup h)^2``) with a shared expert of the
same form. The output projection is a matrix of its own.

Checkpoint tensors are named ``l<i>.<part>``; the matrices of one product are concatenated along
their rows (dq | dkv | g; q | k | v | g; all experts' up; all experts' down).
"""

from __future__ import annotations

from ..config.rirovik import LATENT_TYPES, RirovikConfig
from ..parts.attention import AttentionSpec
from ..parts.blocks import SandwichBlockSpec
from ..parts.latent_attention import LatentAttentionSpec, needs_materialized_heads
from ..parts.moe import RoutedExpertsSpec
from ..parts.norms import RMSNormSpec
from ..parts.positions import NoPositionSpec
from .plan import CheckpointLayout, ModelPlan, ParamSource, RunEntry, Source


def _cache_of(cfg: RirovikConfig) -> list[int]:
    """Layer -> the layer whose cache it uses (itself, or the one it reads)."""
    return [i if getattr(l.mixer, "kv_from", None) is None else l.mixer.kv_from for i, l in enumerate(cfg.layers)]


def rirovik_plan(cfg: RirovikConfig) -> ModelPlan:
    w, eps = cfg.hidden_size, cfg.norm_eps
    norm = RMSNormSpec(w, eps, unit_offset=True)
    owner = _cache_of(cfg)
    # a shared cache layer keeps what its most far-sighted reader needs (0: everything)
    keep: dict[int, int] = {}
    for i, l in enumerate(cfg.layers):
        if l.type in LATENT_TYPES:
            win = l.mixer.window
            keep[owner[i]] = 0 if (win == 0 or keep.get(owner[i], win) == 0) else max(keep.get(owner[i], 0), win)
    layers = []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        if l.type in LATENT_TYPES:
            if needs_materialized_heads(m.kv_rank, m.rot_dim):
                raise NotImplementedError(
                    f"layer {i}: a cache row of kv_rank + rot_dim = {m.kv_rank + m.rot_dim} dims is beyond the "
                    "attention kernels' head sizes")
            mixer = LatentAttentionSpec(
                hidden_size=w, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, latent_rank=m.kv_rank,
                scale=m.scale, eps=eps, window=m.window, cache_window=keep[owner[i]], own_latent=m.kv_from is None,
                sinks=False, query_rank=m.q_rank, rope_dim=m.rot_dim, rope_rotated=m.rot_dims, rope_base=m.rot_base,
                gate="head" if l.type == "latent_attention" else "none")
        else:
            mixer = AttentionSpec(
                hidden_size=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
                position=NoPositionSpec(), bias=True, o_bias=False, window=m.window, qk_norm_eps=eps,
                qk_norm_weight=False, value_dim=m.vdim, keep_first=m.keep_first if m.window else 0, gate="element")
        ff = None
        if l.mlp is not None:
            ff = RoutedExpertsSpec(w, l.mlp.experts, l.mlp.top, l.mlp.ff, l.mlp.shared_ff, activation="relu2",
                                   router_bias=True, router_weights="softmax_of_chosen", weight_on="output",
                                   gated=False, shared_gate=False)
        layers.append(SandwichBlockSpec(norm_in=norm, mixer=mixer, norm_mixer_out=norm,
                                        norm_post=norm if ff is not None else None, feed_forward=ff,
                                        norm_ff_out=norm if ff is not None else None))
    users = sorted(set(owner))
    cache_id = {o: k for k, o in enumerate(users)}
    return ModelPlan(
        vocab_size=cfg.vocab_size, hidden_size=w, layers=tuple(layers),
        run_order=tuple(RunEntry(i, cache_id[owner[i]]) for i in range(len(layers))),
        final_norm=norm, tie_head=False, embed_scale=cfg.embed_scale)


def rirovik_checkpoint_layout(cfg: RirovikConfig) -> CheckpointLayout:
    w = cfg.hidden_size
    entries = [
        ParamSource("embed.weight", (Source("embed", (cfg.vocab_size, w)),), "embedding"),
        ParamSource("final_norm.weight", (Source("final.norm", (w,)),), "offset"),
        ParamSource("head.weight", (Source("head", (cfg.vocab_size, w)),)),
    ]
    ignored = []
    for i, l in enumerate(cfg.layers):
        src, dst, m = f"l{i}.", f"layers.{i}.", l.mixer
        entries += [
            ParamSource(dst + "norm_in.weight", (Source(src + "norm1", (w,)),), "offset"),
            ParamSource(dst + "norm_mixer_out.weight", (Source(src + "norm1b", (w,)),), "offset"),
        ]
        ms, md = src + "mix.", dst + "mixer."
        if l.type in LATENT_TYPES:
            rows = [Source(ms + "dq", (m.q_rank, w))]
            if m.kv_from is None:
                rows.append(Source(ms + "dkv", (m.kv_rank + m.rot_dim, w)))
                entries.append(ParamSource(md + "latent_norm.weight", (Source(ms + "dkv.norm", (m.kv_rank,)),), "scale"))
            if l.type == "latent_attention":
                rows.append(Source(ms + "g", (m.heads, w)))
            entries += [
                ParamSource(md + "in.weight", tuple(rows)),
                ParamSource(md + "q_norm.weight", (Source(ms + "dq.norm", (m.q_rank,)),), "scale"),
                ParamSource(md + "uq.weight", (Source(ms + "uq", (m.heads * (m.dim + m.rot_dim), m.q_rank)),)),
                ParamSource(md + "uk.weight", (Source(ms + "uk", (m.heads * m.dim, m.kv_rank)),)),
                ParamSource(md + "uv.weight", (Source(ms + "uv", (m.heads * m.vdim, m.kv_rank)),)),
                ParamSource(md + "o.weight", (Source(ms + "o", (w, m.heads * m.vdim)),)),
            ]
        else:
            q, k, v = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim
            entries += [
                ParamSource(md + "qkv.weight", (Source(ms + "q", (q, w)), Source(ms + "k", (k, w)),
                                                Source(ms + "v", (v, w)), Source(ms + "g", (m.heads * m.vdim, w)))),
                ParamSource(md + "qkv.bias", (Source(ms + "q.b", (q,)), Source(ms + "k.b", (k,)),
                                              Source(ms + "v.b", (v,))), "bias"),
                ParamSource(md + "o.weight", (Source(ms + "o", (w, m.heads * m.vdim)),)),
            ]
        if l.mlp is None:
            ignored += [src + "norm2", src + "norm2b"]  # a file may carry the unused norms of a layer without feed-forward
            continue
        entries += [
            ParamSource(dst + "norm_post.weight", (Source(src + "norm2", (w,)),), "offset"),
            ParamSource(dst + "norm_ff_out.weight", (Source(src + "norm2b", (w,)),), "offset"),
        ]
        fs, fd = src + "mlp.", dst + "feed_forward."
        E, ff = l.mlp.experts, l.mlp.ff
        entries += [
            ParamSource(fd + "router.weight", (Source(fs + "router", (E, w)),), "matrix32"),
            ParamSource(fd + "router.bias", (Source(fs + "router.b", (E,)),), "offset"),
            ParamSource(fd + "experts.up.weight", tuple(Source(f"{fs}e{e}.up", (ff, w)) for e in range(E))),
            ParamSource(fd + "experts.down.weight", tuple(Source(f"{fs}e{e}.down", (w, ff)) for e in range(E))),
        ]
        if l.mlp.shared_ff:
            entries += [
                ParamSource(fd + "shared.up.weight", (Source(fs + "shared.up", (l.mlp.shared_ff, w)),)),
                ParamSource(fd + "shared.down.weight", (Source(fs + "shared.down", (w, l.mlp.shared_ff)),)),
            ]
    return CheckpointLayout(entries=tuple(entries), ignored_names=tuple(ignored))
