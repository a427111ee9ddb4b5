"""Several residual streams (hyper-connections) instead of one.

The residual state of a token is ``n`` rows ``x_1 .. x_n`` of the model's width, all equal to the
embedded token at the start (``ModelPlan.residual_streams``; the tensor is ``[T, n * width]``
float32, a token's streams one after the other). A sublayer ``f`` with read weights ``r [n]``, mixing
weights ``M [n, n]`` (indexed from, to), write weights ``c [n]`` and a scale per channel ``g [width]``:

    u = sum_s r_s x_s;   y = g * f(norm(u));   x_t <- sum_s M[s, t] x_s + c_t y    (all t from the old x)

Three parts carry this:

* norm ``streams_rmsnorm``: reads ``u`` from the streams (with learned weights, or plainly their
  sum: what the model's last norm does) and norms it. Handed a :class:`PendingStreamsWrite` as its
  ``residual`` it carries that write out while it holds the token's rows (one launch for both);
* :class:`StreamsWrite`: the weights ``M``, ``c`` and ``g`` of one sublayer; ``pending(x, y)`` wraps
  the write that is still to be done;
* block ``streams``: ``norm_in -> mixer -> write``, then ``norm_post -> feed_forward -> write`` (the
  second half is optional). The block's last write is returned as pending, so that the next
  block's (or the model's) norm does it.

All of it is float32; only the normed rows are rounded to the compute dtype.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Norm, ParamDecl, Part


class PendingStreamsWrite:
    """A sublayer's result ``y`` that is still to be written into the streams ``x``. Exactly one of
    :meth:`take` (by the norm that reads ``x`` next) and :meth:`resolve` (written now) happens
    before anything else reads ``x``."""

    __slots__ = ("part", "x", "y")

    def __init__(self, part: "StreamsWrite", x, y) -> None:
        self.part, self.x, self.y = part, x, y

    def take(self):
        y, self.y = self.y, None
        return y

    def resolve(self) -> None:
        if self.y is not None:
            p = self.part
            p.ops.streams_write(self.x, self.take(), p.scale, p.mix, p.out, p.spec.streams)
        return None


@dataclass(frozen=True)
class StreamsWriteSpec:
    size: int
    streams: int
    layer_scale: bool = True  # a learned scale per channel on the sublayer's result
    kind: str = "streams_write"


class StreamsWrite(Part):
    kind = "streams_write"

    def param_decls(self):
        s = self.spec
        decls = {"mix": ParamDecl((s.streams, s.streams), "mix"), "out": ParamDecl((s.streams,), "scale")}
        if s.layer_scale:
            decls["scale"] = ParamDecl((s.size,), "scale")
        return decls

    def bind(self, params):
        self.mix = params["mix"]
        self.out = params["out"]
        self.scale = params.get("scale")

    def pending(self, x, y) -> PendingStreamsWrite:
        return PendingStreamsWrite(self, x, y)


@dataclass(frozen=True)
class StreamsRMSNormSpec:
    size: int
    eps: float
    streams: int
    learned_read: bool = True  # False: the streams are summed as they are
    kind: str = "streams_rmsnorm"


@NORMS.register("streams_rmsnorm")
class StreamsRMSNorm(Norm):
    takes_pending_sums = True  # a pending write into the streams is carried out by this norm's kernel

    def param_decls(self):
        s = self.spec
        decls = {"weight": ParamDecl((s.size,), "scale")}
        if s.learned_read:
            decls["read"] = ParamDecl((s.streams,), "mix")
        return decls

    def bind(self, params):
        self.weight = params["weight"]
        self.read = params.get("read")
        if self.read is None:
            self.read = torch.ones(self.spec.streams, dtype=torch.float32, device=self.env.device)

    def forward(self, x, residual=None, rows=None):
        s, write = self.spec, None
        if isinstance(residual, PendingStreamsWrite):
            if rows is None:
                write = residual
            else:  # only some rows are read here: the write is done for all of them first
                residual.resolve()
        elif residual is not None:
            raise TypeError("streams_rmsnorm: the only add it can carry out is a pending write into the streams")
        if write is None:
            return self.ops.streams_read_norm(x, self.read, self.weight, s.eps, s.streams,
                                              out_dtype=self.env.dtype, rows=rows)
        p = write.part
        return self.ops.streams_write(x, write.take(), p.scale, p.mix, p.out, s.streams, then_read=self.read,
                                      then_weight=self.weight, then_eps=s.eps, out_dtype=self.env.dtype)


@dataclass(frozen=True)
class StreamsBlockSpec:
    streams: int
    norm_in: Any  # a streams_rmsnorm spec
    mixer: Any
    norm_post: Any = None  # None together with feed_forward: the layer is its mixer alone
    feed_forward: Any = None
    layer_scale: bool = True
    kind: str = "streams"


@BLOCKS.register("streams")
class StreamsBlock(Block):
    def __init__(self, spec: StreamsBlockSpec, env) -> None:
        super().__init__(spec, env)
        write = StreamsWriteSpec(spec.norm_in.size, spec.streams, spec.layer_scale)
        self.children = {
            "norm_in": NORMS.build(spec.norm_in, env),
            "mixer": MIXERS.build(spec.mixer, env),
            "mixer_write": StreamsWrite(write, env),
        }
        if spec.feed_forward is not None:
            self.children["norm_post"] = NORMS.build(spec.norm_post, env)
            self.children["feed_forward"] = FEED_FORWARDS.build(spec.feed_forward, env)
            self.children["ff_write"] = StreamsWrite(write, env)
        for name, child in self.children.items():
            setattr(self, name, child)
        self.feed_forward = self.children.get("feed_forward")

    def forward(self, x, pending, step, cache):
        if pending is not None and not isinstance(pending, PendingStreamsWrite):
            raise TypeError("a streams block follows only blocks that leave their add as a pending streams write")
        h = self.norm_in.forward(x, pending)
        # a sublayer's output projection may come back as sums still to be taken: the write takes them
        if getattr(self.mixer, "accepts_deferral", False):
            y = self.mixer.forward(h, step, cache, may_defer=True)
        else:
            y = self.mixer.forward(h, step, cache)
        first = self.mixer_write.pending(x, y)
        if self.feed_forward is None:
            return x, first
        h = self.norm_post.forward(x, first)
        if getattr(self.feed_forward, "accepts_residual", False):
            f = self.feed_forward.forward(h, step, may_defer=True)
        else:
            f = self.feed_forward.forward(h, step)
        return x, self.ff_write.pending(x, f)
