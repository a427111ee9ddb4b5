"""Linear attention: a recurrence over a matrix state, no softmax; with a fixed decay per head
(``decay_linear_attention``) or a decay per key channel made from the token (``gated_linear_attention``, below).

Per head, with ``q_t, k_t`` of ``key_dim`` values and ``v_t`` of ``value_dim``:

    S_t = decay * S_{t-1} + k_t v_t^T          S_{-1} = 0, float32, kept per request
    o_t = S_t^T q_t

Around it, chosen by the spec:

* ``activation``: ``silu`` applied to q, k and v as projected, or ``none``;
* rotary positions on the first ``position.head_dim`` dims of q and k (pairs ``(i, i + dims/2)``),
  or none; ``key_scale`` multiplies k after the rotation;
* ``out_norm``: ``heads`` divides each head's ``o`` by its root mean square (no weight); ``row``
  norms the concatenated heads together and multiplies by a weight;
* the result is multiplied by ``gate_activation(h Wg^T)`` (``silu`` or ``sigmoid``) and projected
  by ``Wo``.

One matrix product makes q | k | v | gate. Activations, rotation, the recurrence, the norm and the
gate run in float32 inside the kernels, whatever the compute dtype of the products is. The state
``[heads, value_dim, key_dim]`` (the transpose of S: a column of S is contiguous) is a
:class:`StateNeed`; a request's first token starts from zero whatever its slot held before.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from .base import MIXERS, POSITION_ENCODINGS, Mixer, ParamDecl, StateNeed, project_into


@dataclass(frozen=True)
class DecayLinearAttentionSpec:
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay: tuple[float, ...]
    eps: float
    activation: str = "none"  # of q, k and v: "none" or "silu"
    key_scale: float = 1.0
    position: Any = None  # a rotary spec whose head_dim is the number of rotated dims, or None
    out_norm: str = "heads"  # "heads": each head alone, no weight; "row": all heads, with a weight
    gate_activation: str = "silu"  # or "sigmoid"
    kind: str = "decay_linear_attention"


@MIXERS.register("decay_linear_attention")
class DecayLinearAttention(Mixer):
    keeps_running_state = True

    def __init__(self, spec: DecayLinearAttentionSpec, env) -> None:
        super().__init__(spec, env)
        if len(spec.decay) != spec.num_heads:
            raise ValueError("one decay per head is needed")
        if spec.activation not in ("none", "silu") or spec.gate_activation not in ("silu", "sigmoid"):
            raise ValueError("unknown activation")
        if spec.out_norm not in ("heads", "row"):
            raise ValueError("out_norm must be 'heads' or 'row'")
        self.rotary = None
        self.rot_dims = 0
        if spec.position is not None:
            self.rotary = POSITION_ENCODINGS.build(spec.position, env).rotary_tables()
            if self.rotary is not None:
                self.rot_dims = 2 * self.rotary[0].shape[1]
                if self.rot_dims > spec.key_dim:
                    raise ValueError("more rotated dims than the key size")
        self.decay = torch.tensor(spec.decay, dtype=torch.float64).to(torch.float32).to(env.device)
        self.qk = spec.num_heads * spec.key_dim
        self.vg = spec.num_heads * spec.value_dim

    def param_decls(self):
        s = self.spec
        decls = {
            "qkvg.weight": ParamDecl((2 * self.qk + 2 * self.vg, s.hidden_size), "matrix"),
            "o.weight": ParamDecl((s.hidden_size, self.vg), "matrix"),
        }
        if s.out_norm == "row":
            decls["norm.weight"] = ParamDecl((self.vg,), "scale")
        return decls

    def bind(self, params):
        self.qkvg_weight = params["qkvg.weight"]
        self.o_weight = params["o.weight"]
        self.norm_weight = params.get("norm.weight")

    def cache_need(self):
        s = self.spec
        return StateNeed((s.num_heads, s.value_dim, s.key_dim), torch.float32)

    accepts_deferral = True  # forward(..., may_defer=True) may return a product not yet converted

    def forward(self, h, step, cache, may_defer=False):
        s, ops = self.spec, self.ops
        proj = ops.linear(h, self.qkvg_weight, None, out_dtype=torch.float32)
        cos, sin = self.rotary if self.rotary is not None else (None, None)
        o = ops.decay_linear_attention(
            proj, num_heads=s.num_heads, key_dim=s.key_dim, value_dim=s.value_dim, decay=self.decay,
            state=cache.state, step=step, activation=s.activation, key_scale=s.key_scale,
            cos=cos, sin=sin)
        y = ops.gated_group_norm(
            o, proj, gate_offset=2 * self.qk + self.vg,
            group=s.value_dim if s.out_norm == "heads" else self.vg,
            weight=self.norm_weight, eps=s.eps, gate_activation=s.gate_activation,
            out_dtype=self.env.dtype)
        return project_into(ops, y, self.o_weight, None, self.env.residual_dtype, None, may_defer)


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Linear attention whose decay is made from the token itself, one number per key channel:

        alpha_t = sigmoid(z_t)^(1/tau),  z_t = A2 (A1 h_t) + b         (heads x key_dim values, float32)
        S_t = diag(alpha_t) S_{t-1} + k_t v_t^T,   o_t = S_t^T (query_scale * q_t)

    Each head's ``o`` is divided by its root mean square and multiplied by a weight of ``value_dim``
    values that all heads share; the concatenated heads are multiplied by ``silu(h Wg^T)`` (or
    its sigmoid) and projected by ``Wo``. ``decay_rank`` is the inner size of the two decay
    matrices."""

    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay_rank: int
    tau: float
    eps: float
    query_scale: float = 1.0
    gate_activation: str = "silu"
    kind: str = "gated_linear_attention"


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    keeps_running_state = True

    def __init__(self, spec: GatedLinearAttentionSpec, env) -> None:
        super().__init__(spec, env)
        if spec.gate_activation not in ("silu", "sigmoid"):
            raise ValueError("unknown activation")
        if spec.decay_rank < 1 or spec.tau <= 0:
            raise ValueError("gated linear attention: decay_rank and tau must be positive")
        self.qk = spec.num_heads * spec.key_dim
        self.vg = spec.num_heads * spec.value_dim

    def param_decls(self):
        s = self.spec
        return {
            "qkvg.weight": ParamDecl((2 * self.qk + 2 * self.vg, s.hidden_size), "matrix"),
            "decay_in.weight": ParamDecl((s.decay_rank, s.hidden_size), "matrix"),
            "decay_out.weight": ParamDecl((self.qk, s.decay_rank), "matrix"),
            "decay_out.bias": ParamDecl((self.qk,), "bias"),
            "norm.weight": ParamDecl((s.value_dim,), "scale"),
            "o.weight": ParamDecl((s.hidden_size, self.vg), "matrix"),
        }

    def bind(self, params):
        self.qkvg_weight = params["qkvg.weight"]
        self.decay_in_weight = params["decay_in.weight"]
        self.decay_out_weight = params["decay_out.weight"]
        self.decay_out_bias = params["decay_out.bias"]
        self.norm_weight = params["norm.weight"].repeat(self.spec.num_heads).contiguous()  # the same for every head
        self.o_weight = params["o.weight"]

    def cache_need(self):
        s = self.spec
        return StateNeed((s.num_heads, s.value_dim, s.key_dim), torch.float32)

    accepts_deferral = True

    def forward(self, h, step, cache, may_defer=False):
        s, ops = self.spec, self.ops
        proj = ops.linear(h, self.qkvg_weight, None, out_dtype=torch.float32)
        low = ops.linear(h, self.decay_in_weight, None, out_dtype=self.env.dtype)
        z = ops.linear(low, self.decay_out_weight, self.decay_out_bias, out_dtype=torch.float32)
        o = ops.decay_linear_attention(
            proj, num_heads=s.num_heads, key_dim=s.key_dim, value_dim=s.value_dim, decay=None,
            state=cache.state, step=step, activation="none", key_scale=1.0, cos=None, sin=None,
            decay_logits=z, decay_root=s.tau, query_scale=s.query_scale)
        y = ops.gated_group_norm(
            o, proj, gate_offset=2 * self.qk + self.vg, group=s.value_dim, weight=self.norm_weight,
            eps=s.eps, gate_activation=s.gate_activation, out_dtype=self.env.dtype)
        return project_into(ops, y, self.o_weight, None, self.env.residual_dtype, None, may_defer)
