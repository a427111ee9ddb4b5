"""Dense gated feed-forward (src/llmserve/models/transformer.py:62-71).

    gu = h @ Wgu^T          rows of Wgu: gate (first I rows), then up (last I rows)
    y  = (act(gate) * up) @ Wdown^T,     act = silu: g / (1 + exp(-g)), or
                                         gelu_tanh: 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))

No biases. The activation is computed in float32 (src/llmserve/kernels/csrc/fused_ops.cpp:75-91).

``mlp`` is the ungated form, ``y = Wdown act(Wup h)``, with ``act`` one of ``relu2`` (the square of
relu), ``relu``, ``gelu_tanh``, ``silu``.
"""

from __future__ import annotations

from dataclasses import dataclass

from .base import FEED_FORWARDS, FeedForward, ParamDecl, project_into


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"
    activation: str = "silu"  # or "gelu_tanh"


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def param_decls(self):
        s = self.spec
        return {
            "gate_up.weight": ParamDecl((2 * s.intermediate_size, s.hidden_size), "matrix"),
            "down.weight": ParamDecl((s.hidden_size, s.intermediate_size), "matrix"),
        }

    def __init__(self, spec: SwiGLUSpec, env) -> None:
        super().__init__(spec, env)
        if spec.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated feed-forward: activation {spec.activation!r} is not known")

    def bind(self, params):
        self.gate_up_weight = params["gate_up.weight"]
        self.down_weight = params["down.weight"]

    accepts_residual = True

    def forward(self, h, step, residual=None, may_defer=False):
        ops = self.ops
        if self.spec.activation == "silu":
            a = ops.gated_silu(h, self.gate_up_weight, None, out_dtype=self.env.dtype)
        else:
            a = ops.gated_silu(h, self.gate_up_weight, None, out_dtype=self.env.dtype,
                               activation=self.spec.activation)
        return project_into(ops, a, self.down_weight, None, self.env.residual_dtype, residual, may_defer)


PLAIN_ACTIVATIONS = ("relu2", "relu", "gelu_tanh", "silu")


@dataclass(frozen=True)
class MLPSpec:
    hidden_size: int
    intermediate_size: int
    activation: str = "relu2"
    kind: str = "mlp"


@FEED_FORWARDS.register("mlp")
class MLP(FeedForward):
    accepts_residual = True

    def __init__(self, spec: MLPSpec, env) -> None:
        super().__init__(spec, env)
        if spec.activation not in PLAIN_ACTIVATIONS:
            raise ValueError(f"feed-forward: activation {spec.activation!r} is not known")

    def param_decls(self):
        s = self.spec
        return {
            "up.weight": ParamDecl((s.intermediate_size, s.hidden_size), "matrix"),
            "down.weight": ParamDecl((s.hidden_size, s.intermediate_size), "matrix"),
        }

    def bind(self, params):
        self.up_weight = params["up.weight"]
        self.down_weight = params["down.weight"]

    def forward(self, h, step, residual=None, may_defer=False):
        a = self.ops.activated_linear(h, self.up_weight, self.spec.activation, self.env.dtype)
        return project_into(self.ops, a, self.down_weight, None, self.env.residual_dtype, residual, may_defer)
