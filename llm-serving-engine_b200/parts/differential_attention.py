"""Differential attention: two softmax maps per head over the same values, the second subtracted.

Per token, with H query heads, G key/value heads, query/key size ``d`` and value size ``dv``:

    q = h Wq^T  (H x 2 x d),  k = h Wk^T  (G x 2 x d),  v = h Wv^T  (G x dv)
    q <- q * (1 + coef * ln(floor((position + 1) / every) + 1))        if a query temperature is set
    a_m = softmax_j(scale * q_m . k_m,j) v_j     for the two maps m = 1, 2, causal, head h on group h // (H/G)
    o = a_1 - lam * a_2;   o <- o / sqrt(mean(o^2) + eps) * out_scale   over the head's dv values
    out = (o * sigmoid(h Wg^T)_h) Wo^T          one gate per head

``lam = exp(lq1 . lk1) - exp(lq2 . lk2) + lam_offset`` is one number of the layer, formed in
float32 when the weights are bound.

The paged attention kernels run it as ``2H`` query heads on ``2G`` key heads: the rows of ``Wq`` are
reordered when they are bound, so that the query heads of one (group, map) follow each other and
the kernels' rule "query head j reads key head j // (H/G)" pairs every map with its own keys; every
value head is written into the pages of both of its maps' key heads. Heads are filled up to the
kernels' head size by the kernel that writes them. The kernels hand the two maps' results on in
float32 in the bfloat16 path too: the difference of two nearly equal maps would otherwise carry
their rounding.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .attention import rows_to_whole_vectors
from .base import MIXERS, Mixer, PagedKVNeed, ParamDecl, project_into


@dataclass(frozen=True)
class DifferentialAttentionSpec:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    eps: float
    lam_offset: float  # added to the learned part of the second map's weight
    out_scale: float  # multiplies the normed difference
    temp_coef: float = 0.0
    temp_every: int = 0  # 0: no query temperature
    window: int = 0
    kind: str = "differential_attention"


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    def __init__(self, spec: DifferentialAttentionSpec, env) -> None:
        super().__init__(spec, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.group = spec.num_heads // spec.num_kv_heads
        widest = max(spec.head_dim, spec.value_dim)
        self.kernel_dim = widest + (-widest) % 16
        self.q_size = 2 * spec.num_heads * spec.head_dim
        self.k_size = 2 * spec.num_kv_heads * spec.head_dim
        self.v_size = spec.num_kv_heads * spec.value_dim
        env.ops.check_attention_shape(self.kernel_dim, env.dtype, 2 * spec.num_heads, 2 * spec.num_kv_heads)

    def param_decls(self):
        s = self.spec
        return {
            # rows: q (head by head, map 1 then map 2), k (the same), v, then one gate row per head
            "qkv.weight": ParamDecl((self.q_size + self.k_size + self.v_size + s.num_heads, s.hidden_size), "matrix"),
            "o.weight": ParamDecl((s.hidden_size, s.num_heads * s.value_dim), "matrix"),
            "lam.q1": ParamDecl((s.head_dim,), "offset"),
            "lam.k1": ParamDecl((s.head_dim,), "offset"),
            "lam.q2": ParamDecl((s.head_dim,), "offset"),
            "lam.k2": ParamDecl((s.head_dim,), "offset"),
        }

    def bind(self, params):
        s = self.spec
        w = params["qkv.weight"]
        # query rows from (group, head in group, map) to (group, map, head in group)
        q = w[: self.q_size].view(s.num_kv_heads, self.group, 2, s.head_dim, s.hidden_size)
        q = q.permute(0, 2, 1, 3, 4).reshape(self.q_size, s.hidden_size)
        self.qkv_weight = rows_to_whole_vectors(torch.cat([q, w[self.q_size:]], 0))
        self.o_weight = params["o.weight"]
        one = (params["lam.q1"].float() * params["lam.k1"].float()).sum().exp()
        two = (params["lam.q2"].float() * params["lam.k2"].float()).sum().exp()
        self.lam = float(one - two + torch.tensor(s.lam_offset, dtype=torch.float32))

    def cache_need(self):
        return PagedKVNeed(2 * self.spec.num_kv_heads, self.kernel_dim, self.spec.window)

    def reserve(self, max_seqs: int) -> None:
        if hasattr(self.ops, "reserve_attention_scratch"):
            self.ops.reserve_attention_scratch(self.kernel_dim, max_seqs, 2 * self.spec.num_heads)

    def plan_key(self):
        return ("attention", self.env.dtype, self.kernel_dim)

    def plan_step(self, host_step, group):
        return self.ops.attention_plan(host_step, self.env.dtype, self.kernel_dim)

    def plan_rows(self, single: int, portions: int, tokens: int) -> dict[str, int]:
        qt = self.ops.attention_q_tile(self.env.dtype, self.kernel_dim)
        return {"tiles": tokens // qt + portions, "decode_seqs": single}

    accepts_residual = True
    accepts_deferral = True

    def forward(self, h, step, cache, residual=None, may_defer=False):
        s, ops = self.spec, self.ops
        tables = step.block_tables[cache.group]
        qkv = ops.linear(h, self.qkv_weight, None, out_dtype=torch.float32)
        q = ops.qkv_norm_rope_write(
            qkv, num_heads=2 * s.num_heads, num_kv_heads=2 * s.num_kv_heads, num_value_heads=s.num_kv_heads,
            head_dim=s.head_dim, value_dim=s.value_dim, out_dim=self.kernel_dim,
            q_weight=None, k_weight=None, eps=0.0,
            temp_coef=s.temp_coef, temp_every=s.temp_every,
            positions=step.positions, token_seq=step.token_seq, cos=None, sin=None,
            k_pages=cache.k if cache.writes else None, v_pages=cache.v if cache.writes else None,
            block_tables=tables, page_tokens=cache.page_tokens, out_dtype=self.env.dtype)
        a = ops.paged_attention(
            q, num_heads=2 * s.num_heads, num_kv_heads=2 * s.num_kv_heads, head_dim=self.kernel_dim,
            scale=s.scale, window=s.window, k_pages=cache.k, v_pages=cache.v, block_tables=tables,
            page_tokens=cache.page_tokens, step=step, plan=step.plans[self.plan_key()],
            out_dtype=torch.float32)  # the maps are subtracted before anything is rounded
        o = ops.differential_combine(
            a, qkv, gate_col0=self.q_size + self.k_size + self.v_size, num_heads=s.num_heads, group=self.group,
            head_dim=self.kernel_dim, value_dim=s.value_dim, lam=self.lam, eps=s.eps, out_scale=s.out_scale,
            out_dtype=self.env.dtype)
        return project_into(ops, o, self.o_weight, None, self.env.residual_dtype, residual, may_defer)
