"""Attention over a cached low-rank latent row per token, with a window and a sink per head.

Per token, with ``h`` the normed input, H heads of ``head_dim`` query/key dims and ``value_dim``
value dims, and a latent of ``latent_rank`` dims:

    q      = Wq h                                         [H, head_dim]
    c      = w_c * d / sqrt(mean(d^2) + eps),  d = Wd h   the cached latent row [latent_rank]
    k_j    = Wuk c_j,   v_j = Wuv c_j                      per head, never materialised
    s_j    = scale * q . k_j      for the keys j of the window (the last ``window`` positions,
                                  the query's own included; 0: all earlier ones)
    p_j    = exp(s_j) / (exp(sink) + sum_i exp(s_i))      sink: a learned number per head
    out    = Wo concat_heads(sum_j p_j v_j)

Only ``c`` is kept per token: one row of the cache serves as key and as value. The products with
``Wuk`` and ``Wuv`` are moved to the query's side, ``q . (Wuk c) = (Wuk^T q) . c`` and
``sum_j p_j Wuv c_j = Wuv (sum_j p_j c_j)``, so the attention kernels see H query heads of
``latent_rank`` dims on one shared key/value head. A latent rank that is no multiple of 16 is
padded with zeros when the weights are bound.

A layer with ``own_latent=False`` has no ``Wd``: it is bound to the cache layer of another layer
and reads the rows that layer wrote, with its own ``Wuk``, ``Wuv``, queries, window and sinks.
``cache_window`` is what the shared cache keeps (at least every reader's window).

Further options of the spec, all off by default (any of them takes the layer through
``_forward_rotary``):

* ``query_rank``: the queries are made from a latent of their own, ``q = Wuq (w_q * d_q / rms(d_q))``,
  ``d_q = Wdq h``;
* ``rope_dim``: beside its ``head_dim`` dims every query head has ``rope_dim`` more (laid out
  behind them), which meet one key part of ``rope_dim`` dims that all heads share: the last
  ``rope_dim`` rows of ``Wd``, not normed. Both are turned by the token's position first
  (``rope_rotated`` of the dims, neighbours ``(2i, 2i+1)`` as pairs, angle ``p * rope_base^(-2i /
  rope_rotated)``). The score is ``scale * (q . k_j + q_rope . k_rope_j)``. The cache row of a token
  is ``[c | k_rope (turned)]``; on the query's side ``[Wuk^T q | q_rope]`` meets it, and ``Wuv``
  has zero columns where the key part lies;
* ``gate="head"``: a factor per head on the heads' outputs, ``sigmoid(Wg x)[head]`` with ``x`` the
  mixer's input and one row of ``Wg`` per head.

The rows of the fused input matrix: the queries' (``Wq``, or ``Wdq`` with ``query_rank``), then
the latent's with the key part's behind them (a layer with a latent of its own), then the gate's.

``materialize=True`` is the other arrangement, for a latent rank beyond the attention kernels'
largest head size (:data:`MAX_KERNEL_DIM`): the layer keeps ``k_j`` and ``v_j`` themselves in
pages of its own (H key/value heads of ``max(head_dim, value_dim)`` dims, zero-padded), made from
the latent rows of this step's tokens. A layer without a latent of its own then takes those rows
from the layer that made them earlier in the same step (``latent_key`` names it).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import MIXERS, POSITION_ENCODINGS, Mixer, PagedKVNeed, ParamDecl, project_into
from .positions import RotarySpec


@dataclass(frozen=True)
class LatentAttentionSpec:
    hidden_size: int
    num_heads: int
    head_dim: int
    value_dim: int
    latent_rank: int
    scale: float
    eps: float  # of the latent row's norm
    window: int = 0  # 0: every earlier token
    cache_window: int = 0  # what the cache layer keeps: 0 or >= the window of every layer that reads it
    own_latent: bool = True
    sinks: bool = True
    materialize: bool = False  # keep keys and values per head instead of the latent row
    latent_key: int = 0  # materialize: under which name this step's latent rows are handed on
    query_rank: int = 0  # > 0: queries are made from a normed latent of this size
    rope_dim: int = 0  # > 0: rotated dims per query head, and of the key part all heads share
    rope_rotated: int = 0  # how many of them are turned (the first ones); the rest pass
    rope_base: float = 10000.0
    gate: str = "none"  # "head": a sigmoid gate per head on the heads' outputs
    kind: str = "latent_attention"


MAX_KERNEL_DIM = 256  # the attention kernels' largest head size


def needs_materialized_heads(latent_rank: int, rope_dim: int = 0) -> bool:
    """Whether a layer of this rank has to keep keys and values instead of latent rows."""
    row = latent_rank + rope_dim
    return row + (-row) % 16 > MAX_KERNEL_DIM


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    accepts_residual = True

    def __init__(self, spec: LatentAttentionSpec, env) -> None:
        super().__init__(spec, env)
        if spec.cache_window and (spec.window == 0 or spec.window > spec.cache_window):
            raise ValueError("latent_attention: the cache keeps fewer tokens than the window reads")
        self.q_size = spec.num_heads * (spec.head_dim + spec.rope_dim)
        self.rotary_path = bool(spec.query_rank or spec.rope_dim or spec.gate != "none")
        if spec.gate not in ("none", "head"):
            raise ValueError(f"latent_attention: gate {spec.gate!r} is not known")
        if spec.rope_rotated % 2 or not 0 <= spec.rope_rotated <= spec.rope_dim:
            raise ValueError("latent_attention: the turned dims are an even number of the rotated part's")
        if self.rotary_path and (spec.materialize or spec.sinks):
            raise NotImplementedError(
                "latent_attention: a query latent, a rotated key part or a gate together with sinks, or with a "
                f"cache row beyond {MAX_KERNEL_DIM} dims")
        self.rope_tables = None
        if spec.rope_rotated:
            self.rope_tables = POSITION_ENCODINGS.build(RotarySpec(spec.rope_rotated, spec.rope_base), env).rotary_tables()
        if spec.materialize:
            widest = max(spec.head_dim, spec.value_dim)
            self.kernel_dim = widest + (-widest) % 16
            self.pad = 0
            env.ops.check_attention_shape(self.kernel_dim, env.dtype, spec.num_heads, spec.num_heads)
            return
        self.pad = (-(spec.latent_rank + spec.rope_dim)) % 16
        self.kernel_dim = spec.latent_rank + spec.rope_dim + self.pad
        env.ops.check_attention_shape(self.kernel_dim, env.dtype, spec.num_heads, 1)

    def param_decls(self):
        s = self.spec
        rows = ((s.query_rank or self.q_size) + (s.latent_rank + s.rope_dim if s.own_latent else 0)
                + (s.num_heads if s.gate == "head" else 0))
        decls = {
            "in.weight": ParamDecl((rows, s.hidden_size), "matrix"),  # q rows, then the latent's, then the gate's
            "uk.weight": ParamDecl((s.num_heads * s.head_dim, s.latent_rank), "matrix"),
            "uv.weight": ParamDecl((s.num_heads * s.value_dim, s.latent_rank), "matrix"),
            "o.weight": ParamDecl((s.hidden_size, s.num_heads * s.value_dim), "matrix"),
        }
        if s.own_latent:
            decls["latent_norm.weight"] = ParamDecl((s.latent_rank,), "scale")
        if s.sinks:
            decls["sink"] = ParamDecl((s.num_heads,), "offset")
        if s.query_rank:
            decls["q_norm.weight"] = ParamDecl((s.query_rank,), "scale")
            decls["uq.weight"] = ParamDecl((self.q_size, s.query_rank), "matrix")
        return decls

    def bind(self, params):
        s = self.spec
        H, R = s.num_heads, s.latent_rank
        self.in_weight = params["in.weight"]
        self.o_weight = params["o.weight"]
        self.latent_norm_weight = params.get("latent_norm.weight")
        self.sink = params.get("sink")
        self.q_norm_weight = params.get("q_norm.weight")
        self.uq_weight = params.get("uq.weight")
        if self.rotary_path:
            # Wuk^T per head as [out, in] = [R, head_dim]: its product fills the first R dims of the
            # head's slot; Wuv [H, value_dim, slot] with zero columns behind the latent's R
            self.uk_t = params["uk.weight"].view(H, s.head_dim, R).transpose(1, 2).contiguous()
            self.uv = torch.nn.functional.pad(params["uv.weight"].view(H, s.value_dim, R),
                                              (0, self.kernel_dim - R)).contiguous()
            return
        if s.materialize:
            self._bind_materialized(params)
            return
        # the query side's products, per head as [out, in]: Wuk^T [H, R(+pad), head_dim] and
        # Wuv [H, value_dim, R(+pad)]
        uk_t = params["uk.weight"].view(H, s.head_dim, R).transpose(1, 2)
        uv = params["uv.weight"].view(H, s.value_dim, R)
        if self.pad:
            uk_t = torch.nn.functional.pad(uk_t, (0, 0, 0, self.pad))
            uv = torch.nn.functional.pad(uv, (0, self.pad))
        self.uk_t = uk_t.contiguous()
        self.uv = uv.contiguous()

    def _bind_materialized(self, params):
        """Every head's q, k and v rows padded with zero rows to the kernels' head size, and the
        output projection with zero columns to match."""
        s = self.spec
        H, D, V, Dk, R = s.num_heads, s.head_dim, s.value_dim, self.kernel_dim, s.latent_rank

        def pad_heads(w, d):  # [H * d, n] -> [H * Dk, n]
            out = w.new_zeros(H, Dk, w.shape[1])
            out[:, :d] = w.view(H, d, w.shape[1])
            return out.view(H * Dk, w.shape[1])

        w_in = params["in.weight"]
        q = pad_heads(w_in[: self.q_size], D)
        self.in_weight = torch.cat([q, w_in[self.q_size :]], 0).contiguous()
        self.kv_weight = torch.cat([pad_heads(params["uk.weight"], D), pad_heads(params["uv.weight"], V)], 0).contiguous()
        o = params["o.weight"].new_zeros(s.hidden_size, H, Dk)
        o[:, :, :V] = params["o.weight"].view(s.hidden_size, H, V)
        self.o_weight = o.view(s.hidden_size, H * Dk).contiguous()

    def cache_need(self):
        if self.spec.materialize:
            return PagedKVNeed(self.spec.num_heads, self.kernel_dim, self.spec.cache_window)
        return PagedKVNeed(1, self.kernel_dim, self.spec.cache_window, values=False)

    def reserve(self, max_seqs: int) -> None:
        if hasattr(self.ops, "reserve_attention_scratch"):
            self.ops.reserve_attention_scratch(self.kernel_dim, max_seqs, self.spec.num_heads)

    def plan_key(self):
        return ("attention", self.env.dtype, self.kernel_dim)

    def plan_step(self, host_step, group):
        return self.ops.attention_plan(host_step, self.env.dtype, self.kernel_dim)

    def plan_rows(self, single: int, portions: int, tokens: int) -> dict[str, int]:
        qt = self.ops.attention_q_tile(self.env.dtype, self.kernel_dim)
        return {"tiles": tokens // qt + portions, "decode_seqs": single}

    accepts_deferral = True

    def forward(self, h, step, cache, residual=None, may_defer=False):
        s, ops = self.spec, self.ops
        tables = step.block_tables[cache.group]
        if self.rotary_path:
            return self._forward_rotary(h, step, cache, tables, residual, may_defer)
        if s.materialize:
            return self._forward_materialized(h, step, cache, tables, residual, may_defer)
        # q | latent in the compute dtype (one rounding of the product, whatever the number of rows:
        # the per-head products that follow take operands of that dtype on every kernel)
        proj = ops.linear(h, self.in_weight, None, out_dtype=self.env.dtype)
        if s.own_latent:
            if not cache.writes:
                raise RuntimeError("a latent-attention layer with its own latent must fill its cache layer")
            ops.latent_write(proj, self.q_size, s.latent_rank, self.latent_norm_weight, s.eps, cache.k,
                             step.positions, step.token_seq, tables)
        q = ops.head_linear(proj, 0, self.uk_t, out_dtype=self.env.dtype)  # [T, H * rank]
        o = ops.paged_attention(
            q, num_heads=s.num_heads, num_kv_heads=1, head_dim=self.kernel_dim, scale=s.scale,
            window=s.window, k_pages=cache.k, v_pages=cache.v, block_tables=tables,
            page_tokens=cache.page_tokens, step=step, plan=step.plans[self.plan_key()], sinks=self.sink)
        o = ops.head_linear(o, 0, self.uv, out_dtype=self.env.dtype)  # [T, H * value_dim]
        return project_into(ops, o, self.o_weight, None, self.env.residual_dtype, residual, may_defer)

    def _forward_rotary(self, h, step, cache, tables, residual, may_defer):
        """Input product (its sums unrounded) -> norms of both latents, rotation of the key part,
        page write -> queries from their latent -> the query's side of the key product and the
        rotated query dims into one row per head -> attention over the cached rows -> the value
        product -> gate -> output projection."""
        s, ops, dt = self.spec, self.ops, self.env.dtype
        H, R, Dr = s.num_heads, s.latent_rank, s.rope_dim
        cos, sin = self.rope_tables if self.rope_tables is not None else (None, None)
        proj = ops.linear(h, self.in_weight, None, out_dtype=torch.float32)
        q_cols = s.query_rank or self.q_size
        gate_col0 = q_cols + (R + Dr if s.own_latent else 0)
        if s.own_latent and not cache.writes:
            raise RuntimeError("a latent-attention layer with its own latent must fill its cache layer")
        cq = None
        if s.query_rank or s.own_latent:
            cq = ops.latent_rope_write(
                proj, q_col0=0, q_weight=self.q_norm_weight, kv_col0=q_cols,
                kv_weight=self.latent_norm_weight if s.own_latent else None, rot_dim=Dr, rot=s.rope_rotated,
                eps=s.eps, cos=cos, sin=sin, pages=cache.k, positions=step.positions, token_seq=step.token_seq,
                block_tables=tables, out_dtype=dt)
        if s.query_rank:
            q = ops.linear(cq, self.uq_weight, None, out_dtype=dt)  # [T, H * (head_dim + rope_dim)]
        else:
            q = ops.cast(proj[:, : self.q_size].contiguous(), dt)
        qk = ops.head_linear(q, 0, self.uk_t, out_dtype=dt, a_head_cols=s.head_dim + Dr,
                             out_head_cols=self.kernel_dim)
        if self.kernel_dim > R:
            ops.latent_query_rope(q, qk, num_heads=H, head_dim=s.head_dim, rot_dim=Dr, rot=s.rope_rotated,
                                  cos=cos, sin=sin, positions=step.positions, rank=R)
        o = ops.paged_attention(
            qk, num_heads=H, num_kv_heads=1, head_dim=self.kernel_dim, scale=s.scale, window=s.window,
            k_pages=cache.k, v_pages=cache.v, block_tables=tables, page_tokens=cache.page_tokens, step=step,
            plan=step.plans[self.plan_key()])
        o = ops.head_linear(o, 0, self.uv, out_dtype=dt)  # [T, H * value_dim]
        if s.gate == "head":
            ops.sigmoid_gate_mul(o, proj, gate_col0, s.value_dim)
        return project_into(ops, o, self.o_weight, None, self.env.residual_dtype, residual, may_defer)

    def _forward_materialized(self, h, step, cache, tables, residual, may_defer):
        """Keys and values of this step's tokens are made from their latent rows and kept in this
        layer's own pages; the attention is the ordinary one over H key/value heads."""
        s, ops = self.spec, self.ops
        H, Dk = s.num_heads, self.kernel_dim
        proj = ops.linear(h, self.in_weight, None, out_dtype=torch.float32)  # q (padded per head) | latent
        handed = step.__dict__.setdefault("latent_rows", {})
        if s.own_latent:
            d = proj[:, H * Dk :].contiguous()
            handed[s.latent_key] = ops.add_rmsnorm(d, None, self.latent_norm_weight, s.eps, out_dtype=self.env.dtype)
        c = handed[s.latent_key]
        kv = ops.linear(c, self.kv_weight, None, out_dtype=torch.float32)
        qkv = torch.cat([proj[:, : H * Dk], kv], dim=1)
        q = ops.norm_rope_kv_write(
            qkv, num_heads=H, num_kv_heads=H, head_dim=Dk, values_are_keys=False, q_weight=None, k_weight=None,
            eps=0.0, positions=step.positions, token_seq=step.token_seq, cos=None, sin=None, k_pages=cache.k,
            v_pages=cache.v, block_tables=tables, page_tokens=cache.page_tokens, out_dtype=self.env.dtype)
        o = ops.paged_attention(
            q, num_heads=H, num_kv_heads=H, head_dim=Dk, scale=s.scale, window=s.window, k_pages=cache.k,
            v_pages=cache.v, block_tables=tables, page_tokens=cache.page_tokens, step=step,
            plan=step.plans[self.plan_key()], sinks=self.sink)
        return project_into(ops, o, self.o_weight, None, self.env.residual_dtype, residual, may_defer)
