"""Routed experts: each token runs through the ``top`` of ``num_experts`` small gated feed-forward
layers that a router picks for it, and through an optional shared expert.

    s      = sigmoid(Wr h)                    router scores, computed in 32-bit
    chosen = the ``top`` experts with the largest scores; their weights are the scores themselves
    y      = sum_{e chosen} expert_e(s_e * h)            the weight multiplies the expert's input
           + sigmoid(wg . h) * shared(h)                 if there is a shared expert
    expert(z) = Wdown (act(Wgate z) * (Wup z))

Options of the spec:

* ``router_bias``: a bias per expert is added to the router's logits;
* ``router_weights="softmax_of_chosen"``: the chosen experts' weights are the softmax over their
  logits alone (the choice itself is by the largest logits either way);
* ``weight_on="output"``: the weight multiplies the expert's output instead of its input (the two
  differ whenever the expert is not linear in its input);
* ``gated=False``: an expert is ``Wdown act(Wup z)`` with ``act`` a plain activation (``relu2``:
  the square of relu), and so is the shared expert;
* ``shared_gate=False``: the shared expert is added as it is, without a sigmoid gate.

The tokens' choices are sorted by expert on the device and the experts' products run as one
launch over tiles of rows that belong to one expert each, so nothing comes back to the host
between the router and the sum.
"""

from __future__ import annotations

from dataclasses import dataclass

from .base import FEED_FORWARDS, FeedForward, ParamDecl
from .feed_forward import PLAIN_ACTIVATIONS, MLPSpec, SwiGLUSpec


@dataclass(frozen=True)
class RoutedExpertsSpec:
    hidden_size: int
    num_experts: int
    top: int
    expert_size: int  # inner size of a routed expert
    shared_size: int = 0  # inner size of the shared expert; 0: none
    activation: str = "silu"
    router_bias: bool = False
    router_weights: str = "sigmoid"  # or "softmax_of_chosen"
    weight_on: str = "input"  # or "output"
    gated: bool = True
    shared_gate: bool = True
    kind: str = "routed_experts"


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    accepts_residual = True

    def __init__(self, spec: RoutedExpertsSpec, env) -> None:
        super().__init__(spec, env)
        if not 1 <= spec.top <= spec.num_experts:
            raise ValueError("routed_experts: top must lie between 1 and the number of experts")
        if spec.router_weights not in ("sigmoid", "softmax_of_chosen") or spec.weight_on not in ("input", "output"):
            raise ValueError("routed_experts: unknown kind of router weights or of their place")
        if not spec.gated and spec.activation not in PLAIN_ACTIVATIONS:
            raise ValueError(f"routed_experts: activation {spec.activation!r} is not known for ungated experts")
        self.children = {}
        if spec.shared_size:
            shared = (SwiGLUSpec(spec.hidden_size, spec.shared_size, activation=spec.activation) if spec.gated
                      else MLPSpec(spec.hidden_size, spec.shared_size, activation=spec.activation))
            self.children["shared"] = FEED_FORWARDS.build(shared, env)
        self.shared = self.children.get("shared")
        self.has_gate = self.shared is not None and spec.shared_gate

    def param_decls(self):
        s = self.spec
        decls = {
            # one more row with a shared expert: its gate
            "router.weight": ParamDecl((s.num_experts + (1 if self.has_gate else 0), s.hidden_size), "matrix32"),
            "experts.down.weight": ParamDecl((s.num_experts * s.hidden_size, s.expert_size), "matrix"),
        }
        if s.gated:
            decls["experts.gate_up.weight"] = ParamDecl((s.num_experts * 2 * s.expert_size, s.hidden_size), "matrix")
        else:
            decls["experts.up.weight"] = ParamDecl((s.num_experts * s.expert_size, s.hidden_size), "matrix")
        if s.router_bias:
            decls["router.bias"] = ParamDecl((s.num_experts,), "offset")
        if self.shared is not None:
            for name, decl in self.shared.param_decls().items():
                decls["shared." + name] = decl
        return decls

    def bind(self, params):
        s = self.spec
        self.router_weight = params["router.weight"]
        self.router_bias = params.get("router.bias")
        rows = 2 * s.expert_size if s.gated else s.expert_size
        self.gate_up_weight = params["experts.gate_up.weight" if s.gated else "experts.up.weight"].view(
            s.num_experts, rows, s.hidden_size)
        self.down_weight = params["experts.down.weight"].view(s.num_experts, s.hidden_size, s.expert_size)
        if self.shared is not None:
            self.shared.bind({k[len("shared."):]: v for k, v in params.items() if k.startswith("shared.")})

    def forward(self, h, step, residual=None, may_defer=False):
        s, ops = self.spec, self.ops
        if s.router_bias or s.router_weights != "sigmoid":
            idx, wts, gate = ops.moe_route(h, self.router_weight, s.num_experts, s.top, self.has_gate,
                                           bias=self.router_bias, weights=s.router_weights)
        else:
            idx, wts, gate = ops.moe_route(h, self.router_weight, s.num_experts, s.top, self.has_gate)
        plan = ops.moe_sort(idx, s.num_experts, self.env.dtype, width=_gcd8(s.hidden_size, s.expert_size))
        on_input = s.weight_on == "input"
        gu = ops.expert_linear(h, self.gate_up_weight, plan, top=s.top, wts=wts if on_input else None)
        if s.gated:
            a = ops.silu_mul(gu, out_dtype=self.env.dtype, activation=s.activation)
        else:
            a = ops.activation(gu, s.activation, self.env.dtype)
        y = ops.expert_linear(a, self.down_weight, plan)
        shared = self.shared.forward(h, step) if self.shared is not None else None
        if hasattr(shared, "resolve"):
            shared = shared.resolve()
        if on_input and self.has_gate == (shared is not None):
            return ops.moe_combine(y, plan, s.top, shared, gate, residual)
        return ops.moe_combine(y, plan, s.top, shared, gate, residual, wts=None if on_input else wts)


def _gcd8(*sizes: int) -> int:
    """8 if every size is a multiple of 8 (rows of whole 16-byte vectors in bfloat16), else 1."""
    return 8 if all(n % 8 == 0 for n in sizes) else 1
