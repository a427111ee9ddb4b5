"""Block arrangements.

``prenorm`` (src/llmserve/models/transformer.py:87-94, fused form :176-189):

    x <- x + mixer(norm_in(x));   x <- x + feed_forward(norm_post(x))     (the second half is optional)

The residual stream ``x`` is float32 and is updated in place; each add is carried out by the norm
that reads ``x`` next, so a block returns its feed-forward output as ``pending``: a tensor, None
(already added), or pending sums of the kernel set (see ``parts.base.settle``).

``branchnorm``: the norm stands on each branch's *output* and the branches read ``x`` itself:

    x <- x + norm_mixer(mixer(filter(x)));   x <- x + norm_ff(feed_forward(x))

``sandwich``: a norm before and a norm after each sublayer:

    x <- x + norm_mixer_out(mixer(norm_in(x)));   x <- x + norm_ff_out(feed_forward(norm_post(x)))

(the second half is optional).

``filter`` is an optional input filter of the mixer (a token shift, say); the feed-forward is
optional too. A filter that keeps something per request shares the block's cache layer with the
mixer: the mixer's needs come first, the filter's states after them.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import (BLOCKS, FEED_FORWARDS, INPUT_FILTERS, MIXERS, NORMS, Block, PendingNormedBranch, count_states,
                   flatten_needs, has_pages, settle)


@dataclass(frozen=True)
class PreNormBlockSpec:
    norm_in: Any
    mixer: Any
    norm_post: Any  # None together with feed_forward: the layer is its mixer alone
    feed_forward: Any
    kind: str = "prenorm"


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec: PreNormBlockSpec, env) -> None:
        super().__init__(spec, env)
        self.children = {
            "norm_in": NORMS.build(spec.norm_in, env),
            "mixer": MIXERS.build(spec.mixer, env),
        }
        if spec.feed_forward is not None:
            self.children["norm_post"] = NORMS.build(spec.norm_post, env)
            self.children["feed_forward"] = FEED_FORWARDS.build(spec.feed_forward, env)
        self.norm_in = self.children["norm_in"]
        self.mixer = self.children["mixer"]
        self.norm_post = self.children.get("norm_post")
        self.feed_forward = self.children.get("feed_forward")

    def forward(self, x, pending, step, cache):
        h = self.norm_in.forward(x, settle(pending, self.norm_in))
        if getattr(self.mixer, "accepts_residual", False):
            a = self.mixer.forward(h, step, cache, residual=x, may_defer=True)  # None: already added into x
        else:
            a = self.mixer.forward(h, step, cache)
        if self.feed_forward is None:
            return x, a
        h = self.norm_post.forward(x, settle(a, self.norm_post))
        if getattr(self.feed_forward, "accepts_residual", False):
            return x, self.feed_forward.forward(h, step, residual=x, may_defer=True)
        return x, self.feed_forward.forward(h, step)


@dataclass(frozen=True)
class BranchNormBlockSpec:
    mixer: Any
    norm_mixer: Any
    feed_forward: Any = None  # None: the layer has no feed-forward (and no norm for it)
    norm_ff: Any = None
    input_filter: Any = None
    kind: str = "branchnorm"


@BLOCKS.register("branchnorm")
class BranchNormBlock(Block):
    def __init__(self, spec: BranchNormBlockSpec, env) -> None:
        super().__init__(spec, env)
        self.children = {"mixer": MIXERS.build(spec.mixer, env), "norm_mixer": NORMS.build(spec.norm_mixer, env)}
        if spec.feed_forward is not None:
            self.children["feed_forward"] = FEED_FORWARDS.build(spec.feed_forward, env)
            self.children["norm_ff"] = NORMS.build(spec.norm_ff, env)
        if spec.input_filter is not None:
            self.children["filter"] = INPUT_FILTERS.build(spec.input_filter, env)
        self.mixer = self.children["mixer"]
        self.norm_mixer = self.children["norm_mixer"]
        self.feed_forward = self.children.get("feed_forward")
        self.norm_ff = self.children.get("norm_ff")
        self.filter = self.children.get("filter")
        need = self.mixer.cache_need()
        self._mixer_part = (has_pages(need), 0, count_states(need))
        self._filter_part = (False, count_states(need),
                             count_states(self.filter.cache_need()) if self.filter is not None else 0)

    def cache_need(self):
        needs = flatten_needs(self.mixer.cache_need())
        if self.filter is not None:
            needs += flatten_needs(self.filter.cache_need())
        return tuple(needs) if needs else None

    def forward(self, x, pending, step, cache):
        if pending is not None:  # a block of another arrangement came before: its add is done now
            pending = pending.resolve() if hasattr(pending, "resolve") else pending
            if pending is not None:
                x += pending
        if self.filter is not None:
            h = self.filter.forward(x, step, cache.part(*self._filter_part))
        else:
            h = self.ops.cast(x, self.env.dtype)
        if getattr(self.mixer, "accepts_deferral", False):
            a = self.mixer.forward(h, step, cache.part(*self._mixer_part), may_defer=True)
        else:
            a = self.mixer.forward(h, step, cache.part(*self._mixer_part))
        h = self.norm_mixer.add_normed(x, a, emit=self.feed_forward is not None)
        if self.feed_forward is not None:
            if getattr(self.feed_forward, "accepts_residual", False):
                f = self.feed_forward.forward(h, step, may_defer=True)
            else:
                f = self.feed_forward.forward(h, step)
            self.norm_ff.add_normed(x, f, emit=False)
        return x, None


@dataclass(frozen=True)
class SandwichBlockSpec:
    norm_in: Any
    mixer: Any
    norm_mixer_out: Any
    norm_post: Any = None  # None together with feed_forward and norm_ff_out: the layer is its mixer alone
    feed_forward: Any = None
    norm_ff_out: Any = None
    kind: str = "sandwich"


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    def __init__(self, spec: SandwichBlockSpec, env) -> None:
        super().__init__(spec, env)
        self.children = {
            "norm_in": NORMS.build(spec.norm_in, env),
            "mixer": MIXERS.build(spec.mixer, env),
            "norm_mixer_out": NORMS.build(spec.norm_mixer_out, env),
        }
        if spec.feed_forward is not None:
            self.children["norm_post"] = NORMS.build(spec.norm_post, env)
            self.children["feed_forward"] = FEED_FORWARDS.build(spec.feed_forward, env)
            self.children["norm_ff_out"] = NORMS.build(spec.norm_ff_out, env)
        for name, child in self.children.items():
            setattr(self, name, child)
        self.feed_forward = self.children.get("feed_forward")

    def forward(self, x, pending, step, cache):
        h = self.norm_in.forward(x, settle(pending, self.norm_in))
        if getattr(self.mixer, "accepts_deferral", False):
            a = self.mixer.forward(h, step, cache, may_defer=True)  # may be a product still lying as sums
        else:
            a = self.mixer.forward(h, step, cache)
        if self.feed_forward is None:
            return x, PendingNormedBranch(self.norm_mixer_out, x, a)  # the next norm adds it as it reads x
        # x += norm(a), and the next norm of the new x, in the norm's own way (one launch if it can)
        h = self.norm_mixer_out.add_normed_then(x, a, self.norm_post)
        if getattr(self.feed_forward, "accepts_residual", False):
            f = self.feed_forward.forward(h, step, may_defer=True)
        else:
            f = self.feed_forward.forward(h, step)
        return x, PendingNormedBranch(self.norm_ff_out, x, f)
