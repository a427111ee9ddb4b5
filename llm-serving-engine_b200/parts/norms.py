"""Root-mean-square norm (src/llmserve/models/layers.py:11-21).

``y = x * rsqrt(mean(x^2) + eps) * w`` with the statistics, the scaling and the weight multiply in
float32; the result is rounded once to the compute dtype. The residual add that precedes the norm
in a pre-norm block is part of the same kernel (src/llmserve/kernels/csrc/fused_ops.cpp:52-73).

``unit_offset``: the stored weight lies around zero and the norm multiplies by ``1 + w``. The sum
is formed once, in float32, when the weight is bound; the kernels see an ordinary weight.
"""

from __future__ import annotations

from dataclasses import dataclass

from .base import NORMS, Norm, ParamDecl, PendingNormedBranch


@dataclass(frozen=True)
class RMSNormSpec:
    size: int
    eps: float
    unit_offset: bool = False  # multiply by 1 + w instead of w
    kind: str = "rmsnorm"


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    takes_pending_sums = True  # the kernel adds a product's pending sums as it reads the row

    def param_decls(self):
        return {"weight": ParamDecl((self.spec.size,), "offset" if self.spec.unit_offset else "scale")}

    def bind(self, params):
        w = params["weight"]
        self.weight = (w + 1.0) if self.spec.unit_offset else w

    def forward(self, x, residual=None, rows=None):
        if isinstance(residual, PendingNormedBranch):
            if rows is None:  # the branch's norm, the sum and this norm while the rows are held once
                return residual.norm.add_normed_then(x, residual.take(), self)
            residual = residual.resolve()  # only some rows are read here: the whole sum is formed first
        return self.ops.add_rmsnorm(
            x, residual, self.weight, self.spec.eps, out_dtype=self.env.dtype, rows=rows
        )

    def add_normed(self, x, branch, emit=True):
        """``x += norm(branch)``; returns the new ``x`` in the compute dtype if ``emit``."""
        return self.ops.rmsnorm_add(x, branch, self.weight, self.spec.eps,
                                    out_dtype=self.env.dtype if emit else None)

    def add_normed_then(self, x, branch, then):
        if not isinstance(then, RMSNorm):
            return super().add_normed_then(x, branch, then)
        return self.ops.rmsnorm_add(x, branch, self.weight, self.spec.eps, out_dtype=self.env.dtype,
                                    then_weight=then.weight, then_eps=then.spec.eps)
