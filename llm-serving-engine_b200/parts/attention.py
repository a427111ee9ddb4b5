"""Causal self-attention over a paged key/value cache, with grouped query heads.

Per token (src/llmserve/models/transformer.py:37-59, src/llmserve/attention.py:231-307):

    qkv = h @ Wqkv^T (+ b)                      rows of Wqkv ordered q, then k, then v
    q, k = rotate(q, k; position)               if the position encoding has rotary tables
    cache[k, v at this token's slot] = k, v     before attention, so a portion attends to itself
    s_j = scale * q . k_j   for every key j of the same request with j <= position
                            (and j > position - window if the layer has a window)
    o = sum_j softmax(s)_j v_j                  query head h reads key/value head h // group
    out = o @ Wo^T (+ b)

``scale`` and ``window`` are parameters of the spec. Scores, softmax and the weighted sum run in
float32 inside the kernels.

Further options of the spec, all off by default:

* ``qk_norm_eps``: q and k are divided, head by head, by their root mean square and multiplied by
  a weight of ``head_dim`` values that all heads share (one for q, one for k), before any rotation;
* ``values_are_keys``: there is no value projection; the value of a token is its key as projected,
  before the norm and the rotation;
* ``head_temperature``: a learned number per query head multiplies its scores;
* ``distance_slopes``: ``slope_h * (i - j)`` is taken off the score of query i and key j;
* ``chunk``: query i reads key j only if ``i // chunk == j // chunk`` (positions count from the
  start of the sequence, however the prompt was cut);
* ``qk_norm_weight=False``: the q/k norm has no weight (a plain division by the root mean square);
* ``value_dim``: values have another size than queries and keys; the kernels then run on heads
  of the larger size, with zero rows and columns filling the smaller one up;
* ``keep_first``: with a window, the sequence's first ``keep_first`` keys stay visible to every
  later query beside its window, at their true positions; their pages are never given back;
* ``gate``: the heads' outputs are multiplied by ``sigmoid(Wg h)`` before the output projection,
  ``element`` by element (``Wg`` has as many rows as the concatenated heads) or ``head`` by head
  (one row per head); ``Wg`` reads the same ``h`` and its rows follow v's in the fused matrix;
* ``o_bias``: whether the output projection has a bias (None: as ``bias`` says);
* ``qk_norm_scope="row"``: the q/k norm runs over all of a token's query rows at once (and over
  all of its key rows), with weights of that size, instead of head by head;
* ``sinks``: a learned number per query head whose exponential joins the softmax's denominator
  without a key or a value.

A position encoding whose tables cover fewer dims than the head size rotates the first of each
head's dims (pairs ``(i, i + rotated/2)``) and passes the rest. That, and the norm over whole rows,
are served by the kernel set's ``qkv_norm_rope_write``, which also fills a head up to the kernels'
head size itself (the projection's rows are then left as they are).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from .base import MIXERS, POSITION_ENCODINGS, Mixer, PagedKVNeed, ParamDecl, project_into


def rows_to_whole_vectors(w, multiple: int = 8):
    """A fused projection matrix with zero rows behind its last, so that a row of the product is
    a whole number of 16-byte vectors whatever the number of gate rows is (the kernels that read
    the product then work on vectors; what lies behind the last head is never read)."""
    extra = (-w.shape[0]) % multiple
    if not extra:
        return w
    return torch.cat([w, w.new_zeros(extra, w.shape[1])], 0).contiguous()


@dataclass(frozen=True)
class AttentionSpec:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: Any  # a position-encoding spec
    bias: bool = False
    window: int = 0  # 0: every earlier token; w: the last w tokens, the query's own included
    qk_norm_eps: float | None = None
    values_are_keys: bool = False
    head_temperature: bool = False
    distance_slopes: tuple[float, ...] | None = None
    chunk: int = 0
    qk_norm_weight: bool = True
    value_dim: int | None = None  # None: head_dim
    keep_first: int = 0
    gate: str = "none"  # "element", "head"
    o_bias: bool | None = None  # None: as bias
    qk_norm_scope: str = "head"  # "row": one norm over all query rows of a token, one over all key rows
    sinks: bool = False
    kind: str = "attention"


@MIXERS.register("attention")
class PagedAttention(Mixer):
    def __init__(self, spec: AttentionSpec, env) -> None:
        super().__init__(spec, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.gate not in ("none", "element", "head"):
            raise ValueError(f"attention: gate {spec.gate!r} is not known")
        if spec.keep_first and (spec.window <= 0 or spec.chunk > 0):
            raise ValueError("attention: keep_first needs a window and no chunks")
        self.value_dim = spec.head_dim if spec.value_dim is None else spec.value_dim
        if spec.values_are_keys and self.value_dim != spec.head_dim:
            raise ValueError("attention: values that are keys have the keys' size")
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        self.position = POSITION_ENCODINGS.build(spec.position, env)
        self.rotary = self.position.rotary_tables()
        self.v_size = 0 if spec.values_are_keys else spec.num_kv_heads * self.value_dim
        self.gate_size = {"none": 0, "element": spec.num_heads * self.value_dim, "head": spec.num_heads}[spec.gate]
        self.o_bias_on = spec.bias if spec.o_bias is None else spec.o_bias
        if spec.qk_norm_scope not in ("head", "row"):
            raise ValueError(f"attention: qk_norm_scope {spec.qk_norm_scope!r} is not known")
        self.rot_dims = 2 * self.rotary[0].shape[1] if self.rotary is not None else 0
        if self.rot_dims > spec.head_dim:
            raise ValueError("attention: more rotated dims than the head size")
        # whole-row norms and partly rotated heads go through the kernel that prepares a token's rows at once
        self.by_rows = ((spec.qk_norm_scope == "row" and spec.qk_norm_eps is not None)
                        or (self.rotary is not None and self.rot_dims != spec.head_dim))
        if self.by_rows and (spec.bias or spec.gate == "element" or spec.keep_first):
            raise NotImplementedError("attention: whole-row norm or a partly rotated head with bias, element gate or kept keys")
        # the plain path (fused projection, rotation, cache write and attention) serves none of these
        self.extended = (spec.qk_norm_eps is not None or spec.values_are_keys or spec.head_temperature
                         or spec.distance_slopes is not None or spec.chunk > 0
                         or self.value_dim != spec.head_dim or spec.keep_first > 0 or spec.gate != "none"
                         or spec.sinks or self.by_rows)
        # The attention kernels take head sizes that are multiples of 16. With the score options on,
        # any other head size is padded with zeros up to the next one when the weights are bound:
        # zero dims change no dot product, the norm divides by the true size, and the padded dims
        # of the output (values are zero there) meet zero columns of the output projection.
        widest = max(spec.head_dim, self.value_dim)
        self.kernel_dim = widest + ((-widest) % 16 if self.extended else 0)
        self.pad = self.kernel_dim - spec.head_dim  # of a query or key head; a value head's may differ
        if self.pad and self.rotary is not None and not self.by_rows:
            raise NotImplementedError("a padded head size with rotary positions")
        self.slopes = None
        if spec.distance_slopes is not None:
            if len(spec.distance_slopes) != spec.num_heads:
                raise ValueError("one distance slope per query head is needed")
            self.slopes = torch.tensor(spec.distance_slopes, dtype=torch.float64).to(torch.float32).to(env.device)
        env.ops.check_attention_shape(self.kernel_dim, env.dtype, spec.num_heads, spec.num_kv_heads)

    def param_decls(self):
        s = self.spec
        decls = {
            # rows: q, k, v heads, then the gate's
            "qkv.weight": ParamDecl((self.q_size + self.kv_size + self.v_size + self.gate_size, s.hidden_size), "matrix"),
            "o.weight": ParamDecl((s.hidden_size, s.num_heads * self.value_dim), "matrix"),
        }
        if s.bias:
            decls["qkv.bias"] = ParamDecl((self.q_size + self.kv_size + self.v_size,), "bias")
        if self.o_bias_on:
            decls["o.bias"] = ParamDecl((s.hidden_size,), "bias")
        if s.qk_norm_eps is not None and s.qk_norm_weight:
            row = s.qk_norm_scope == "row"
            decls["q_norm.weight"] = ParamDecl((self.q_size if row else s.head_dim,), "scale")
            decls["k_norm.weight"] = ParamDecl((self.kv_size if row else s.head_dim,), "scale")
        if s.sinks:
            decls["sinks"] = ParamDecl((s.num_heads,), "scale")
        if s.head_temperature:
            decls["temperature"] = ParamDecl((s.num_heads,), "scale")
        return decls

    def bind(self, params):
        self.qkv_weight = params["qkv.weight"]
        self.o_weight = params["o.weight"]
        self.qkv_bias = params.get("qkv.bias")
        self.o_bias = params.get("o.bias")
        self.q_norm_weight = params.get("q_norm.weight")
        self.k_norm_weight = params.get("k_norm.weight")
        self.temperature = params.get("temperature")
        self.sinks = params.get("sinks")
        s = self.spec
        if s.qk_norm_eps is not None and not s.qk_norm_weight:  # the kernel's norm multiplies by a weight: ones
            row = s.qk_norm_scope == "row"
            self.q_norm_weight = torch.ones(self.q_size if row else s.head_dim, dtype=torch.float32, device=self.env.device)
            self.k_norm_weight = torch.ones(self.kv_size if row else s.head_dim, dtype=torch.float32, device=self.env.device)
        if self.by_rows:  # the kernel fills the heads up; only the output projection meets the padded heads
            self.qkv_weight = rows_to_whole_vectors(self.qkv_weight)
            if self.kernel_dim != self.value_dim:
                o = self.o_weight.new_zeros(s.hidden_size, s.num_heads, self.kernel_dim)
                o[:, :, :self.value_dim] = self.o_weight.view(s.hidden_size, s.num_heads, self.value_dim)
                self.o_weight = o.view(s.hidden_size, s.num_heads * self.kernel_dim).contiguous()
            return
        if self.gate_size and self.qkv_bias is not None:  # the gate has no bias
            self.qkv_bias = torch.cat([self.qkv_bias, self.qkv_bias.new_zeros(self.gate_size)])
        if self.kernel_dim != s.head_dim or self.kernel_dim != self.value_dim:
            self._pad_heads()

    def _pad_heads(self):
        """Every head's rows of q, k and v (and of a gate per element) filled up with zero rows to
        the kernels' head size, the output projection with zero columns to match."""
        s, D, V, Dp = self.spec, self.spec.head_dim, self.value_dim, self.kernel_dim
        H, G = s.num_heads, s.num_kv_heads
        parts = [(H, D), (G, D)] + ([] if s.values_are_keys else [(G, V)])
        if s.gate == "element":
            parts.append((H, V))

        def pad_rows(w):  # rows of the fused matrix (or entries of its bias), head by head
            out, at = [], 0
            for heads, d in parts:
                piece = w[at : at + heads * d]
                at += heads * d
                padded = w.new_zeros((heads, Dp) + tuple(w.shape[1:]))
                padded[:, :d] = piece.view((heads, d) + tuple(w.shape[1:]))
                out.append(padded.view((heads * Dp,) + tuple(w.shape[1:])))
            out.append(w[at:])  # a gate per head: one row each, as it is
            return torch.cat(out, 0).contiguous()

        self.qkv_weight = pad_rows(self.qkv_weight)
        if self.qkv_bias is not None:
            self.qkv_bias = pad_rows(self.qkv_bias)
        o = self.o_weight.new_zeros(s.hidden_size, H, Dp)
        o[:, :, :V] = self.o_weight.view(s.hidden_size, H, V)
        self.o_weight = o.view(s.hidden_size, H * Dp).contiguous()
        if self.q_norm_weight is not None:
            self.q_norm_weight = torch.nn.functional.pad(self.q_norm_weight, (0, Dp - D))
            self.k_norm_weight = torch.nn.functional.pad(self.k_norm_weight, (0, Dp - D))

    # what the cache manager has to keep for a layer of this kind
    def cache_need(self):
        s = self.spec
        return PagedKVNeed(s.num_kv_heads, self.kernel_dim, s.window, keep_first=s.keep_first)

    def reserve(self, max_seqs: int) -> None:
        """Allocate kernel scratch for up to ``max_seqs`` single-token sequences in a step."""
        if hasattr(self.ops, "reserve_attention_scratch"):
            self.ops.reserve_attention_scratch(self.kernel_dim, max_seqs, self.spec.num_heads)

    # work lists depend only on the batch, the kernels' tile size and the group's page size
    def plan_key(self):
        return ("attention", self.env.dtype, self.kernel_dim)

    def plan_step(self, host_step, group):
        return self.ops.attention_plan(host_step, self.env.dtype, self.kernel_dim)

    def plan_rows(self, single: int, portions: int, tokens: int) -> dict[str, int]:
        """Most rows of each work list for a step of ``single`` one-token sequences and ``portions``
        longer ones that hold ``tokens`` tokens together. A captured step has lists of exactly this
        many rows; a shorter list is filled up by repeating its last row (a tile that is computed
        twice writes the same values twice)."""
        qt = self.ops.attention_q_tile(self.env.dtype, self.kernel_dim)
        return {"tiles": tokens // qt + portions, "decode_seqs": single}

    accepts_residual = True
    accepts_deferral = True

    def forward(self, h, step, cache, residual=None, may_defer=False):
        s = self.spec
        ops = self.ops
        tables = step.block_tables[cache.group]
        cos, sin = self.rotary if self.rotary is not None else (None, None)
        if self.extended:
            o = self._extended(h, step, cache, tables, cos, sin)
            return project_into(ops, o, self.o_weight, self.o_bias, self.env.residual_dtype, residual, may_defer)
        o = ops.project_attend(
            h, self.qkv_weight, self.qkv_bias,
            num_heads=s.num_heads,
            num_kv_heads=s.num_kv_heads,
            head_dim=s.head_dim,
            scale=s.scale,
            window=s.window,
            positions=step.positions,
            token_seq=step.token_seq,
            cos=cos,
            sin=sin,
            k_pages=cache.k,
            v_pages=cache.v,
            writes=cache.writes,
            block_tables=tables,
            page_tokens=cache.page_tokens,
            step=step,
            plan=step.plans[self.plan_key()],
            out_dtype=self.env.dtype,
        )
        return project_into(ops, o, self.o_weight, self.o_bias, self.env.residual_dtype, residual, may_defer)

    def _extended(self, h, step, cache, tables, cos, sin):
        """Projection (its sums unrounded), norm / rotation / cache write, attention with the
        score options: three launches, and one more with an output gate."""
        s, ops = self.spec, self.ops
        qkv = ops.linear(h, self.qkv_weight, self.qkv_bias, out_dtype=torch.float32)
        if self.by_rows:
            return self._by_rows(qkv, step, cache, tables, cos, sin)
        q = ops.norm_rope_kv_write(
            qkv, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=self.kernel_dim,
            norm_dim=s.head_dim,
            values_are_keys=s.values_are_keys, q_weight=self.q_norm_weight, k_weight=self.k_norm_weight,
            eps=s.qk_norm_eps if s.qk_norm_eps is not None else 0.0,
            positions=step.positions, token_seq=step.token_seq, cos=cos, sin=sin,
            k_pages=cache.k if cache.writes else None, v_pages=cache.v if cache.writes else None,
            block_tables=tables, page_tokens=cache.page_tokens, out_dtype=self.env.dtype)
        o = ops.paged_attention(
            q, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=self.kernel_dim, scale=s.scale,
            window=s.window, k_pages=cache.k, v_pages=cache.v, block_tables=tables,
            page_tokens=cache.page_tokens, step=step, plan=step.plans[self.plan_key()],
            head_scale=self.temperature, slopes=self.slopes, chunk=s.chunk, keep_first=s.keep_first,
            sinks=self.sinks)
        if s.gate != "none":  # the gate's columns follow v's in the projection's rows
            col0 = (s.num_heads + s.num_kv_heads * (1 if s.values_are_keys else 2)) * self.kernel_dim
            ops.sigmoid_gate_mul(o, qkv, col0, 1 if s.gate == "element" else self.kernel_dim)
        return o

    def _by_rows(self, qkv, step, cache, tables, cos, sin):
        """The same three or four launches with the kernel that prepares all rows of a token."""
        s, ops = self.spec, self.ops
        normed = s.qk_norm_eps is not None
        q = ops.qkv_norm_rope_write(
            qkv, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads,
            num_value_heads=0 if s.values_are_keys else s.num_kv_heads, head_dim=s.head_dim,
            value_dim=self.value_dim, out_dim=self.kernel_dim,
            q_weight=self.q_norm_weight if normed else None, k_weight=self.k_norm_weight if normed else None,
            eps=s.qk_norm_eps or 0.0,
            positions=step.positions, token_seq=step.token_seq, cos=cos, sin=sin,
            k_pages=cache.k if cache.writes else None, v_pages=cache.v if cache.writes else None,
            block_tables=tables, page_tokens=cache.page_tokens, out_dtype=self.env.dtype)
        o = ops.paged_attention(
            q, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=self.kernel_dim, scale=s.scale,
            window=s.window, k_pages=cache.k, v_pages=cache.v, block_tables=tables,
            page_tokens=cache.page_tokens, step=step, plan=step.plans[self.plan_key()],
            head_scale=self.temperature, slopes=self.slopes, chunk=s.chunk, sinks=self.sinks)
        if s.gate == "head":  # one gate column per head, behind q, k (and v)
            col0 = self.q_size + self.kv_size + self.v_size
            ops.sigmoid_gate_mul(o, qkv, col0, self.kernel_dim)
        return o
