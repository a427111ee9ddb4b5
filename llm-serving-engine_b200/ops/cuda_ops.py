"""The kernel set of the product path: thin, checked calls into the sm_100a extension.

There is no other implementation behind these methods: if CUDA or the compiled extension is not
available, constructing :class:`CudaOps` raises.

Matrix products: float32 runs this package's own CUDA-core kernel (true 32-bit, no tensor-core
mode). bfloat16 products of up to 32 rows (decoding) run this package's tcgen05 kernel; with more
rows they go to cuBLAS through ``torch.mm`` with float32 accumulation, the same
library-for-linear-layers split as the reference (src/llmserve/models/layers.py:129-152).

The few-rows kernel shares a tile's K between blocks, which add their partial sums with integer
atomics into a buffer of 64-bit fixed-point numbers (value * 2^24). Such sums have the same bits
whatever the order of the additions was, so the bfloat16 path is reproducible from run to run.
The kernel that consumes the product (single-token attention, rotation and cache write, SiLU,
residual add and norm, or a plain conversion) reads the buffer, converts and leaves zeros behind. The buffers never leave
this class except as a :class:`PendingSums` that stands for "a product still to be added to the
residual stream".
"""

from __future__ import annotations

import numpy as np
import torch

from . import build

_DTYPES = (torch.float32, torch.bfloat16)


class PendingSums:
    """A product that is still to be added to the float32 tensor ``into`` (the residual stream).

    What a projection called with ``accumulate_into=x, may_defer=True`` may return instead of
    adding at once: the sums lie in a fixed-point buffer of the kernel set. Hand it, as the
    ``residual``, to the next ``add_rmsnorm`` on the same ``x`` (which adds it while it reads it
    anyway), or call :meth:`resolve` to have it added now. Exactly one of the two must happen
    before anything else reads ``x``.
    """

    __slots__ = ("ops", "sums", "into")

    def __init__(self, ops: "CudaOps", sums: torch.Tensor, into: torch.Tensor) -> None:
        self.ops, self.sums, self.into = ops, sums, into

    def resolve(self) -> None:
        """Add the sums to ``into`` now. Returns None: nothing is pending any more."""
        if self.sums is not None:
            self.ops.ext.fixed_to_float(self.sums, self.into, True)
            self.ops.launches += 1
            self.ops._sums_taken(self.sums)
            self.sums = None
        return None


class MoePlan:
    """What :meth:`CudaOps.moe_sort` leaves for the experts' products and the final sum: the int32
    work buffer (row ranges, the sorted order and its inverse, tiles), the number of choices, the
    number of experts and which kernel the tiles were cut for."""

    __slots__ = ("work", "n", "num_experts", "kind")

    def __init__(self, work, n, num_experts, kind) -> None:
        self.work, self.n, self.num_experts, self.kind = work, n, num_experts, kind


class DeferredProduct:
    """A few-rows product whose fixed-point sums nobody has taken yet. What ``linear`` may return
    to a caller that says ``may_defer=True`` without a tensor to add into: a kernel that reads the
    product once anyway (``rmsnorm_add``) takes the sums itself; :meth:`resolve` converts them to a
    float32 tensor for everybody else."""

    __slots__ = ("ops", "sums")

    def __init__(self, ops: "CudaOps", sums: torch.Tensor) -> None:
        self.ops, self.sums = ops, sums

    def resolve(self) -> torch.Tensor:
        out = torch.empty(self.sums.shape, dtype=torch.float32, device=self.sums.device)
        self.ops.ext.fixed_to_float(self.sums, out, False)
        self.ops.launches += 1
        self.ops._sums_taken(self.sums)
        self.sums = None
        return out


# Cost of a block of the single-token attention kernel in units of one key: its start (tables,
# queries, first tile) and end (partial results, counter), and what each further partition adds
# to the merge. From timings at 2118 keys of head size 64: a wave of blocks takes about 39 ns per
# key and 5 us besides.
_BLOCK_START_KEYS = 130
_MERGE_KEYS_PER_SPLIT = 4


def choose_decode_splits(pairs: int, max_ctx: int, num_sms: int, blocks_per_sm: int) -> int:
    """Context partitions per (sequence, key/value head) for ``pairs`` such pairs.

    The kernel runs one block per (partition, pair); ``blocks_per_sm * num_sms`` of them run at a
    time, a *wave*. One tile of keys is in flight per warp, so a block's speed is set by latency,
    not by how many blocks share the SM, and a wave that is part empty takes as long as a full
    one: 12 sequences x 32 heads cut in 3 make 1152 blocks for 1036 places and took 49 us where
    24 sequences took 79. So the number of partitions is the one that minimises
    ``waves * (keys per block + a block's fixed cost)``, among partitions of 128 keys or more
    (measured at one sequence of 2176 keys: 8 partitions 13.3 us, 16 10.9, 28 11.9, 34 12.1).
    The context is rounded up to a power of two first, so that the choice (which captured graphs
    are keyed on) does not flicker from step to step. Without a known occupancy: about six blocks
    per SM.
    """
    if pairs <= 0:
        return 1
    most = int(max(1, min((max_ctx + 127) // 128, 64)))
    if blocks_per_sm <= 0:
        want = max(1, (6 * num_sms + pairs - 1) // pairs)
        return int(min(want, most))
    wave = blocks_per_sm * num_sms
    ctx = 1 << max(0, int(max_ctx) - 1).bit_length()

    def cost(s: int) -> int:
        waves = -(-pairs * s // wave)
        return waves * (-(-ctx // s) + _BLOCK_START_KEYS + _MERGE_KEYS_PER_SPLIT * s)

    return min(range(1, most + 1), key=lambda s: (cost(s), s))


class CudaOps:
    name = "cuda-sm100a"
    defers_adds = True  # linear(..., accumulate_into=x, may_defer=True) may return PendingSums

    def __init__(self, device: torch.device | str = "cuda") -> None:
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise RuntimeError(
                "llmserve_b200 runs on a CUDA device only (built for sm_100a); no CPU fallback exists"
            )
        self.ext = build.load_core()
        self._attn_loaded: set[int] = set()
        self._scratch: torch.Tensor | None = None
        self.decode_blocks_per_sm = 0  # of the single-token attention kernel; 0: not asked yet
        self.fuse_rotation_into_attention = True  # single tokens: attention makes q, k, v from the product's sums
        self._takes_sums_known: dict[tuple, bool] = {}
        self._sample_scratch: torch.Tensor | None = None
        self._sample_rows = 0
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        # 0: fastest available; 1: CUDA cores; 2: mma.sync fed by plain loads; 3: single tokens fed by TMA
        self.attention_kernel = 0  # (tests compare them)
        self.use_skinny_gemm = True
        # rows up to which the own tcgen05 product runs (measured: above it the library is faster)
        self.skinny_max_rows = int(self.ext.gemm_bf16_skinny_max_rows())
        # Fixed-point sum buffers of the few-rows product, by shape. A buffer is zero whenever it
        # is not in _sums_live (the kernel that takes a product's sums leaves zeros behind).
        self._sums: dict[tuple[int, int], list[torch.Tensor]] = {}
        self._sums_live: set[int] = set()  # data_ptr of buffers whose sums have not been taken yet
        self._addmm_in_place: bool | None = None  # whether torch.addmm can add into a float32 tensor
        self.launches = 0  # kernels of this package enqueued (library matrix products not counted)

    # ------------------------------------------------------------------ capabilities
    def branch_dtype(self, dtype: torch.dtype) -> torch.dtype:
        """Dtype in which projections that feed the residual stream return their result."""
        return torch.float32

    def check_attention_shape(self, head_dim: int, dtype: torch.dtype, num_heads: int | None = None,
                              num_kv_heads: int | None = None) -> None:
        """Load the kernels of this head size. With the head counts given, also ask how many blocks
        of the single-token kernel an SM holds (the smallest answer over a model's layers is kept:
        :meth:`decode_splits` fills whole waves of that many blocks)."""
        if dtype not in _DTYPES:
            raise ValueError(f"attention kernels exist for float32 and bfloat16, not {dtype}")
        if head_dim not in self._attn_loaded:
            self.ext.load_attention_library(build.attention_library(head_dim), head_dim)
            self._attn_loaded.add(head_dim)
        if num_heads and num_kv_heads:
            n = int(self.ext.attention_decode_blocks_per_sm(head_dim, dtype == torch.bfloat16,
                                                            num_heads, num_kv_heads))
            if n > 0:
                self.decode_blocks_per_sm = min(self.decode_blocks_per_sm or n, n)

    def reserve_attention_scratch(self, head_dim: int, max_decode: int, num_heads: int,
                                  max_splits: int = 64) -> None:
        """Allocate the partial-result buffer of split-context attention once, at its largest."""
        need = int(self.ext.attention_scratch_floats(head_dim, max_decode, num_heads, max_splits))
        if self._scratch is None or self._scratch.numel() < need:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("attention scratch must be reserved before graph capture")
            # zeros: the buffer starts with completion counters that every launch leaves at zero
            self._scratch = torch.zeros(need, dtype=torch.float32, device=self.device)

    def check_kernel_errors(self) -> None:
        """Raise if a kernel recorded that one of its bounded waits ran out."""
        code = int(self.ext.kernel_error())
        if code:
            self.ext.clear_kernel_error()
            raise RuntimeError(f"a CUDA kernel of llmserve_b200 gave up waiting (code {code})")

    # ------------------------------------------------------------------ pointwise
    def embedding(self, token_ids, table):
        out = torch.empty(token_ids.shape[0], table.shape[1], dtype=torch.float32, device=table.device)
        self.ext.embedding(token_ids, table, out)
        self.launches += 1
        return out

    def add_rmsnorm(self, x, residual, weight, eps, out_dtype, rows=None):
        """``residual`` may be a :class:`PendingSums` for ``x``: its sums are added as they are read."""
        sums = None
        if isinstance(residual, PendingSums):
            if residual.into is not x:
                raise ValueError("these pending sums belong to another tensor")
            if rows is None and out_dtype == torch.bfloat16 and x.shape[1] % 4 == 0 and residual.sums is not None:
                sums, residual.sums = residual.sums, None
                residual = sums
            else:  # only some rows are read here, so the whole product is added first
                residual = residual.resolve()
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device)
        self.ext.add_rmsnorm(x, residual, weight, float(eps), out, rows)
        self.launches += 1
        if sums is not None:
            self._sums_taken(sums)
        return out

    # ------------------------------------------------------------------ fixed-point sums
    def _product_sums(self, a, w, bias) -> torch.Tensor:
        """``a @ w.T (+ bias)`` as fixed-point sums in a buffer that the caller must have taken
        (by a kernel that clears it) before the buffer of this shape is used again."""
        T, N = a.shape[0], w.shape[0]
        kept = self._sums.setdefault((T, N), [])  # usually one; two when branches of one shape are pending together
        buf = next((b for b in kept if b.data_ptr() not in self._sums_live), None)
        if buf is None:
            buf = torch.zeros(T, N, dtype=torch.int64, device=self.device)
            if not torch.cuda.is_current_stream_capturing():
                kept.append(buf)
        self._sums_live.add(buf.data_ptr())
        self.ext.gemm_bf16_skinny(a, w, bias, buf)
        self.launches += 1
        return buf

    def _sums_taken(self, buf: torch.Tensor) -> None:
        self._sums_live.discard(buf.data_ptr())

    _ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}

    def silu_mul(self, gu, out_dtype=None, activation="silu"):
        """``act(gate) * up`` of ``gu = [gate | up]``; ``activation``: silu or gelu_tanh."""
        out_dtype = out_dtype or gu.dtype
        out = torch.empty(gu.shape[0], gu.shape[1] // 2, dtype=out_dtype, device=gu.device)
        self.ext.silu_mul(gu, out, self._ACTIVATIONS[activation])
        self.launches += 1
        return out

    # ------------------------------------------------------------------ matrix products
    def _few_rows(self, a, w) -> bool:
        """Does the own tcgen05 kernel serve this product?"""
        return (self.use_skinny_gemm and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and a.shape[0] <= self.skinny_max_rows and a.shape[1] % 8 == 0)

    def linear(self, a, w, bias=None, out_dtype=None, accumulate_into=None, may_defer=False):
        """``a @ w.T (+ bias)`` as a new tensor of ``out_dtype`` (None: the compute dtype).

        With ``accumulate_into`` (a float32 tensor of the result's shape) the product may be
        added into that tensor instead; the return value is then None. A caller that passes
        ``may_defer=True`` may get a :class:`PendingSums` instead, which it has to hand on to
        whoever reads ``accumulate_into`` next.
        """
        if a.dtype == torch.float32:
            if w.dtype != torch.float32:
                raise TypeError("float32 activations need float32 weights")
            out = torch.empty(a.shape[0], w.shape[0], dtype=torch.float32, device=a.device)
            self.ext.gemm_f32(a, w, bias, out)
            self.launches += 1
            return out if out_dtype in (None, torch.float32) else out.to(out_dtype)
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise TypeError(f"linear: unsupported dtypes {a.dtype} x {w.dtype}")
        T = a.shape[0]
        N = w.shape[0]
        if self._few_rows(a, w):
            # few rows: the weights are streamed once through the tcgen05 kernel, work balanced
            # over all SMs, partial sums added as fixed-point numbers
            sums = self._product_sums(a, w, bias)
            if accumulate_into is not None:
                pending = PendingSums(self, sums, accumulate_into)
                return pending if may_defer else pending.resolve()
            if may_defer and out_dtype == torch.float32:
                return DeferredProduct(self, sums)
            out = torch.empty(T, N, dtype=out_dtype or torch.bfloat16, device=a.device)
            self.ext.fixed_to_float(sums, out, False)
            self.launches += 1
            self._sums_taken(sums)
            return out
        if accumulate_into is not None and bias is None and self._addmm_in_place is not False:
            # many rows: the library adds the product into the residual stream (beta = 1)
            try:
                torch.addmm(accumulate_into, a, w.t(), out_dtype=torch.float32, out=accumulate_into)
                self._addmm_in_place = True
                return None
            except (RuntimeError, TypeError):
                if self._addmm_in_place:
                    raise
                self._addmm_in_place = False  # this build of the library cannot; use the plain form
        if out_dtype == torch.float32:
            out = torch.mm(a, w.t(), out_dtype=torch.float32)
            if bias is not None:
                out += bias.float()
            return out
        if bias is not None:
            return torch.addmm(bias, a, w.t())  # bias added before the one rounding to bfloat16
        return torch.mm(a, w.t())

    def gated_silu(self, h, w, bias=None, out_dtype=None, activation="silu"):
        """``act(h @ gate.T) * (h @ up.T)`` for ``w = [gate rows; up rows]``. With few bfloat16
        rows the gate meets its activation as a float32 value (the activation kernel takes the
        product's fixed-point sums); otherwise as the product's rounded output."""
        out_dtype = out_dtype or h.dtype
        if self._few_rows(h, w) and out_dtype == torch.bfloat16 and w.shape[0] % 8 == 0:
            sums = self._product_sums(h, w, bias)
            out = self.silu_mul(sums, out_dtype=out_dtype, activation=activation)
            self._sums_taken(sums)
            return out
        return self.silu_mul(self.linear(h, w, bias), out_dtype=out_dtype, activation=activation)

    def project_rope_kv_write(self, h, w, bias, *, num_heads, num_kv_heads, head_dim, positions,
                              token_seq, cos, sin, k_pages, v_pages, block_tables, page_tokens,
                              out_dtype):
        """The fused q|k|v projection of ``h``, rotation of q and k, and the write of k and v into
        their pages; returns the rotated queries. With few bfloat16 rows q, k and v reach the
        rotation as float32 values (the rotation kernel takes the product's fixed-point sums)."""
        kw = dict(num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                  positions=positions, token_seq=token_seq, cos=cos, sin=sin, k_pages=k_pages,
                  v_pages=v_pages, block_tables=block_tables, page_tokens=page_tokens, out_dtype=out_dtype)
        if self._few_rows(h, w) and out_dtype == torch.bfloat16 and head_dim % 8 == 0:
            sums = self._product_sums(h, w, bias)
            q = self.rope_kv_write(sums, **kw)
            self._sums_taken(sums)
            return q
        return self.rope_kv_write(self.linear(h, w, bias), **kw)

    def project_attend(self, h, w, bias, *, num_heads, num_kv_heads, head_dim, scale, window, positions,
                       token_seq, cos, sin, k_pages, v_pages, writes, block_tables, page_tokens, step,
                       plan, out_dtype):
        """The fused q|k|v projection of ``h``, rotation, cache write (if ``writes``) and attention
        over the cache. For a step of few single tokens in bfloat16 this is two launches: the
        product leaves fixed-point sums, and the attention kernel makes its queries and this
        step's key and value from them (a single token's position is its context length - 1).
        Otherwise: projection, rotation + cache write, attention."""
        T = h.shape[0]
        n_dec = int(plan["decode_seqs"].shape[0])
        if (self.fuse_rotation_into_attention and writes and n_dec == T and int(plan["tiles"].shape[0]) == 0
                and self._few_rows(h, w) and out_dtype == torch.bfloat16 and self.attention_kernel in (0, 2)
                and self._takes_sums(head_dim, num_heads, num_kv_heads)):
            sums = self._product_sums(h, w, bias)
            out = torch.empty(T, num_heads * head_dim, dtype=out_dtype, device=h.device)
            splits = step.decode_splits if step.decode_splits else self.decode_splits(
                n_dec, num_kv_heads, step.max_decode_ctx)
            scratch = None
            if splits > 1:
                self.reserve_attention_scratch(head_dim, n_dec, num_heads, splits)
                scratch = self._scratch
            self.ext.paged_attention_from_sums(
                sums, out, k_pages, v_pages, num_heads, num_kv_heads, head_dim, float(scale), int(window),
                block_tables, step.ctx_lens, step.cu_q, plan["decode_seqs"], splits, scratch, cos, sin)
            self._sums_taken(sums)
            self.launches += 1
            return out
        q = self.project_rope_kv_write(
            h, w, bias, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
            positions=positions, token_seq=token_seq, cos=cos, sin=sin,
            k_pages=k_pages if writes else None, v_pages=v_pages if writes else None,
            block_tables=block_tables, page_tokens=page_tokens, out_dtype=out_dtype)
        return self.paged_attention(
            q, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, scale=scale, window=window,
            k_pages=k_pages, v_pages=v_pages, block_tables=block_tables, page_tokens=page_tokens,
            step=step, plan=plan)

    def _takes_sums(self, head_dim, num_heads, num_kv_heads) -> bool:
        key = (head_dim, num_heads, num_kv_heads)
        if key not in self._takes_sums_known:
            self._takes_sums_known[key] = bool(self.ext.attention_takes_sums(head_dim, True, num_heads, num_kv_heads))
        return self._takes_sums_known[key]

    # ------------------------------------------------------------------ attention
    def rope_kv_write(self, qkv, *, num_heads, num_kv_heads, head_dim, positions, token_seq,
                      cos, sin, k_pages, v_pages, block_tables, page_tokens, out_dtype):
        """Rotate q and k, write k and v into their pages; returns the rotated queries."""
        q = self.ext.rope_kv_write(qkv, num_heads, num_kv_heads, head_dim, positions, token_seq,
                                   cos, sin, k_pages, v_pages, block_tables, page_tokens,
                                   out_dtype == torch.bfloat16)
        self.launches += 1
        return q

    def attention_q_tile(self, dtype, head_dim):
        if head_dim not in self._attn_loaded:  # a caller that did not announce its head size first
            self.check_attention_shape(head_dim, dtype)
        return int(self.ext.attention_q_tile(head_dim, dtype == torch.bfloat16,
                                             self.attention_kernel))

    def attention_plan(self, host_step, dtype, head_dim):
        """Work lists for this step: tiles of the portions, and the single-token sequences."""
        qt = self.attention_q_tile(dtype, head_dim)
        tiles, decode = [], []
        for s, n in enumerate(host_step.q_lens.tolist()):
            if n == 1:
                decode.append(s)
            else:
                tiles.extend((s, q0) for q0 in range(0, n, qt))
        # longest contexts first: their tiles run longest
        tiles.sort(key=lambda t: -(int(host_step.ctx_lens[t[0]]) - int(host_step.q_lens[t[0]]) + t[1]))
        return {
            "tiles": np.asarray(tiles, dtype=np.int32).reshape(-1, 2),
            "decode_seqs": np.asarray(decode, dtype=np.int32),
        }

    def decode_splits(self, num_decode, num_kv_heads, max_ctx):
        """Context partitions per (sequence, head) for a step of single tokens."""
        return choose_decode_splits(num_decode * num_kv_heads, max_ctx, self.num_sms, self.decode_blocks_per_sm)

    def paged_attention(self, q, *, num_heads, num_kv_heads, head_dim, scale, window, k_pages,
                        v_pages, block_tables, page_tokens, step, plan, head_scale=None, slopes=None,
                        chunk=0, sinks=None, keep_first=0, out_dtype=None):
        """``head_scale`` / ``slopes`` (float32 ``[heads]``) and ``chunk``: a factor per head on the
        score, ``slope_h * (i - j)`` taken off it, and keys limited to the query's chunk. ``sinks``
        (float32 ``[heads]``): ``exp(sink_h)`` joins the softmax's denominator. ``keep_first``: with
        a window, the sequence's first ``keep_first`` keys stay visible beside the window's.
        ``out_dtype=torch.float32`` beside bfloat16 queries: the results are handed on unrounded."""
        out = torch.empty(q.shape[0], num_heads * head_dim, dtype=out_dtype or q.dtype, device=q.device)
        n_tiles = int(plan["tiles"].shape[0])
        n_dec = int(plan["decode_seqs"].shape[0])
        splits = step.decode_splits if step.decode_splits else self.decode_splits(
            n_dec, num_kv_heads, step.max_decode_ctx)
        scratch = None
        if n_dec and splits > 1:
            self.reserve_attention_scratch(head_dim, n_dec, num_heads, splits)
            scratch = self._scratch
        self.ext.paged_attention(
            q, out, k_pages, v_pages, num_heads, num_kv_heads, head_dim, float(scale),
            int(window), block_tables, step.ctx_lens, step.cu_q,
            plan["tiles"] if n_tiles else None, n_tiles,
            plan["decode_seqs"] if n_dec else None, n_dec, splits, scratch,
            self.attention_kernel, head_scale, slopes, int(chunk), sinks, int(keep_first) if window else 0,
        )
        self.launches += (1 if n_tiles else 0) + (1 if n_dec else 0)
        return out

    def norm_rope_kv_write(self, qkv, *, num_heads, num_kv_heads, head_dim, values_are_keys, q_weight,
                           k_weight, eps, positions, token_seq, cos, sin, k_pages, v_pages,
                           block_tables, page_tokens, out_dtype, norm_dim=None):
        """Head-wise RMS norm of q and k (if weights are given), rotation (if tables are given),
        key/value page write; returns the queries ``[T, heads * head_dim]`` in ``out_dtype``.
        ``qkv`` is the float32 projection (its rows may be wider than q, k and v: what lies behind
        them is not read); with ``values_are_keys`` it has no value heads and a
        token's value is its key as projected. ``norm_dim``: the number of dims the mean of the
        norm is taken over, when the trailing dims of a head are zero padding."""
        q = torch.empty(qkv.shape[0], num_heads * head_dim, dtype=out_dtype, device=qkv.device)
        self.ext.norm_rope_kv_write(qkv, q, num_heads, num_kv_heads, head_dim, bool(values_are_keys),
                                    q_weight, k_weight, float(eps), positions, token_seq, cos, sin,
                                    k_pages, v_pages, block_tables, int(page_tokens),
                                    int(norm_dim or head_dim))
        self.launches += 1
        return q

    # ------------------------------------------------------------------ embedding terms, latent attention
    def hashed_pair_add(self, x, table, state, step, *, buckets, mul_previous, mul_token):
        """``x[t] += table[(previous * mul_previous + token * mul_token) mod buckets]`` (row
        ``buckets`` at position 0); ``state`` (int32, one number per slot) hands the last token of
        a step to the request's next step."""
        self.ext.hashed_pair_add(x, table, state, step.token_ids, step.positions, step.token_seq, step.cu_q,
                                 step.state_slots, int(buckets), int(mul_previous), int(mul_token))
        self.launches += 1

    def sinusoid_add(self, x, positions, freq):
        """``x[t, 2i] += sin(p freq_i)``, ``x[t, 2i+1] += cos(p freq_i)``."""
        self.ext.sinusoid_add(x, positions, freq)
        self.launches += 1

    def latent_write(self, proj, col0, rank, weight, eps, pages, positions, token_seq, block_tables):
        """Columns ``col0 .. col0 + rank`` of each row of ``proj``, RMS-normed and weighted, into the
        token's place of ``pages`` ``[pages, 1, page_tokens, >= rank]`` (further dims are zeroed)."""
        self.ext.latent_write(proj, int(col0), int(rank), weight, float(eps), pages, positions, token_seq,
                              block_tables)
        self.launches += 1

    def _rows_kernel(self, a, w, rows: int, few: int) -> int:
        """Which kernel serves a product over gathered rows: 0 the CUDA cores (float32, or rows
        that are no whole 16-byte vectors), 2 the weight-streaming kernel for at most ``few`` rows,
        1 mma.sync tiles."""
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            return 0
        return 2 if rows <= few else 1

    def head_linear(self, a, col0, w, out_dtype, kind=None, a_head_cols=0, out_head_cols=0):
        """A product per head: ``out[t, h] = w[h] @ a[t, col0 + h*K : col0 + (h+1)*K]`` for ``w``
        ``[H, N, K]``; returns ``[T, H*N]``. ``kind`` forces a kernel (tests compare them).
        ``a_head_cols`` (default K): columns from one head to the next in ``a``, whose heads may
        carry more than the K columns that are read. ``out_head_cols`` (default N): the result is
        ``[T, H * out_head_cols]`` and a head's product fills the first N columns of its slot; the
        rest is left for the caller to fill."""
        out = torch.empty(a.shape[0], w.shape[0] * (out_head_cols or w.shape[1]), dtype=out_dtype, device=a.device)
        kind = self._rows_kernel(a, w, a.shape[0], self.skinny_max_rows) if kind is None else kind
        self.ext.head_linear(a, int(col0), w, out, int(kind), int(a_head_cols), int(out_head_cols))
        self.launches += 1
        return out

    def latent_rope_write(self, proj, *, q_col0=0, q_weight=None, kv_col0=0, kv_weight=None, rot_dim=0,
                          rot=0, eps, cos=None, sin=None, pages=None, positions, token_seq, block_tables,
                          out_dtype):
        """Of each row of ``proj``: the query latent (columns ``q_col0 ..``, as many as ``q_weight``
        has values) RMS-normed and returned ``[T, query rank]``; the key/value latent (columns
        ``kv_col0 ..``, as many as ``kv_weight`` has) RMS-normed and, behind it, the ``rot_dim``
        columns of the shared key part with their first ``rot`` dims turned by the token's position
        (neighbouring dims paired; ``cos``/``sin`` ``[positions, rot/2]``), written as one row of
        the token's page. Either side may be absent (its weight None)."""
        cq = None
        if q_weight is not None:
            cq = torch.empty(proj.shape[0], q_weight.numel(), dtype=out_dtype, device=proj.device)
        self.ext.latent_rope_write(proj, int(q_col0), q_weight, cq, int(kv_col0), kv_weight, int(rot_dim), int(rot),
                                   float(eps), cos, sin, pages if kv_weight is not None else None, positions,
                                   token_seq, block_tables)
        self.launches += 1
        return cq

    def latent_query_rope(self, q, out, *, num_heads, head_dim, rot_dim, rot, cos, sin, positions, rank):
        """``q [T, H * (head_dim + rot_dim)]``: every head's last ``rot_dim`` dims, turned by the
        position, go behind the ``rank`` dims of the head's slot in ``out [T, H * slot]``; what is
        left of the slot is zeroed."""
        self.ext.latent_query_rope(q, int(num_heads), int(head_dim), int(rot_dim), int(rot), cos, sin, positions,
                                   out, int(rank))
        self.launches += 1
        return out

    def sigmoid_gate_mul(self, o, g, col0, group):
        """``o[t, i] *= sigmoid(g[t, col0 + i // group])`` in place; returns ``o``."""
        self.ext.sigmoid_gate_mul(o, g, int(col0), int(group))
        self.launches += 1
        return o

    _PLAIN_ACTIVATIONS = {"relu2": 0, "relu": 1, "gelu_tanh": 2, "silu": 3}

    def activation(self, z, activation, out_dtype):
        """``act(z)`` element by element in ``out_dtype``; relu2 is the square of relu."""
        out = torch.empty(z.shape, dtype=out_dtype, device=z.device)
        self.ext.act_rows(z, out, self._PLAIN_ACTIVATIONS[activation])
        self.launches += 1
        return out

    def activated_linear(self, h, w, activation, out_dtype):
        """``act(h @ w.T)``. With few bfloat16 rows the activation meets the product as float32
        values (it takes the product's fixed-point sums)."""
        if self._few_rows(h, w) and out_dtype == torch.bfloat16:
            sums = self._product_sums(h, w, None)
            out = self.activation(sums, activation, out_dtype)
            self._sums_taken(sums)
            return out
        return self.activation(self.linear(h, w, None, out_dtype=torch.float32), activation, out_dtype)

    # ------------------------------------------------------------------ routed experts
    _ROUTER_WEIGHTS = {"sigmoid": 0, "softmax_of_chosen": 1}

    def moe_route(self, h, router, num_experts, top, has_gate, bias=None, weights="sigmoid"):
        """Router logits (+ ``bias``) in float32; returns (the ``top`` experts with the largest
        logits ``[T, top]`` int32, their weights ``[T, top]``, the shared expert's gate ``[T]`` or
        None). ``weights``: ``sigmoid`` of each chosen logit, or ``softmax_of_chosen``: the softmax
        over the chosen logits alone."""
        T = h.shape[0]
        idx = torch.empty(T, top, dtype=torch.int32, device=h.device)
        wts = torch.empty(T, top, dtype=torch.float32, device=h.device)
        gate = torch.empty(T, dtype=torch.float32, device=h.device) if has_gate else None
        self.ext.moe_route(h, router, int(num_experts), int(top), idx, wts, gate, bias, self._ROUTER_WEIGHTS[weights])
        self.launches += 1
        return idx, wts, gate

    def moe_sort(self, idx, num_experts, dtype, width=0, kind=None):
        """The choices sorted by expert, as row ranges and tiles for :meth:`expert_linear`: a plan
        that :meth:`moe_combine` reads too. ``dtype`` and ``width`` (of the experts' input) choose
        the kernel of the products: 0 the CUDA cores (float32), 2 the weight-streaming kernel (up
        to 48 choices: a few rows per expert; measured at 8 experts of 4096 x 2048, 2 per token:
        16 tokens 45 us against 55 us for the tiles, 32 tokens 72 against 58), 1 mma.sync tiles,
        3 tcgen05 tiles (more than 1024 choices, rows of whole 16-byte vectors); ``kind`` forces one."""
        n = idx.numel()
        if kind is None:
            if dtype != torch.bfloat16:
                kind = 0
            elif n <= 48:
                kind = 2
            else:
                kind = 3 if (n > 1024 and width % 8 == 0) else 1
        tile_rows = int(self.ext.moe_tile_rows(int(kind)))
        tiles = int(self.ext.moe_max_tiles(n, int(num_experts), tile_rows))
        work = torch.empty(num_experts + 1 + 2 * n + 2 * tiles + 1, dtype=torch.int32, device=idx.device)
        self.ext.moe_sort(idx, int(num_experts), work, tile_rows)
        self.launches += 1
        return MoePlan(work, n, int(num_experts), int(kind))

    def expert_linear(self, a, w, plan, top=0, wts=None):
        """float32 ``[n, N]``: sorted row r is ``w[its expert] @ a-row``. With ``top`` the a-row is
        gathered, ``a[choice // top] * wts[choice]``; without, ``a`` is already in sorted order."""
        out = torch.empty(plan.n, w.shape[1], dtype=torch.float32, device=a.device)
        kind, gathered = plan.kind, None
        if kind == 3 and (a.shape[1] % 8 or a.dtype != torch.bfloat16):
            raise ValueError("this plan's kernel takes bfloat16 rows of a multiple of 8 elements")
        if kind == 3 and top:
            gathered = torch.empty(plan.n, a.shape[1], dtype=a.dtype, device=a.device)
            self.launches += 1
        self.ext.expert_linear(a, w, out, plan.work, plan.n, int(top), wts, kind, gathered)
        self.launches += 1
        return out

    def moe_combine(self, y, plan, top, shared, gate, residual, wts=None):
        """Per token the sum of its experts' rows of ``y``, each times its weight if ``wts``
        ``[T, top]`` is given, (+ gate * shared; no gate: + shared): added into ``residual``
        (returns None) or returned."""
        work, num_experts = plan.work, plan.num_experts
        T = y.shape[0] // top
        out = residual if residual is not None else torch.empty(T, y.shape[1], dtype=torch.float32, device=y.device)
        self.ext.moe_combine(y, work, int(num_experts), int(top), shared, gate if shared is not None else None,
                             out, residual is not None, wts)
        self.launches += 1
        return None if residual is not None else out

    # ------------------------------------------------------------------ branch-norm blocks, state mixers
    def cast(self, x, dtype):
        """The float32 residual stream in the compute dtype (itself, if that is float32)."""
        if x.dtype == dtype:
            return x
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
        self.ext.cast_f32(x, out)
        self.launches += 1
        return out

    def token_shift(self, x, mix, state, step, out_dtype):
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        self.ext.token_shift(x, mix, state, out, step.token_seq, step.cu_q, step.ctx_lens, step.state_slots)
        self.launches += 1
        return out

    @staticmethod
    def _two_branches(branches, weights, coefficients):
        if not 1 <= len(branches) <= 2:
            raise NotImplementedError("the kernels norm and sum one or two branches")
        b = branches[1] if len(branches) == 2 else None
        wb = weights[1] if len(branches) == 2 else None
        cb = coefficients[1] if len(branches) == 2 else 0.0
        return branches[0], b, weights[0], wb, float(coefficients[0]), float(cb)

    def mix_normed(self, branches, weights, coefficients, eps):
        branches = [m.resolve() if isinstance(m, DeferredProduct) else m for m in branches]
        a, b, wa, wb, ca, cb = self._two_branches(branches, weights, coefficients)
        out = torch.empty_like(a)
        self.ext.mix_normed(a, b, wa, wb, ca, cb, float(eps), out)
        self.launches += 1
        return out

    def rmsnorm_add(self, x, branch, weight, eps, out_dtype=None, then_weight=None, then_eps=0.0):
        """``x += weight * y / rms(y)`` with ``y`` the branch (a float32 tensor, or a
        ``BranchMix`` whose members are normed and summed in the same launch); returns the new
        ``x`` in ``out_dtype`` unless that is None. With ``then_weight`` what is returned is the
        next norm of the new ``x``, ``then_weight * x / rms(x)`` (eps ``then_eps``), from the same
        launch."""
        if then_weight is not None and out_dtype is None:
            raise ValueError("the norm that follows needs an output dtype")
        out = None if out_dtype is None else torch.empty(x.shape, dtype=out_dtype, device=x.device)
        members = list(branch.branches) if hasattr(branch, "branches") else [branch]
        # products still lying as sums are taken by the kernel itself if all members are such
        # and their rows fit its shared memory; otherwise they are converted first
        deferred = [m for m in members if isinstance(m, DeferredProduct)]
        take = (len(deferred) == len(members) and all(m.sums is not None for m in deferred)
                and x.shape[1] * len(members) * 4 <= 48 * 1024)
        tensors = [(m.sums if take else m.resolve()) if isinstance(m, DeferredProduct) else m for m in members]
        if hasattr(branch, "branches"):
            a, b, wa, wb, ca, cb = self._two_branches(tensors, branch.weights, branch.coefficients)
            self.ext.rmsnorm_add(x, a, b, wa, wb, ca, cb, float(branch.eps), weight, float(eps), out,
                                 then_weight, float(then_eps))
        else:
            self.ext.rmsnorm_add(x, tensors[0], None, None, None, 1.0, 0.0, 0.0, weight, float(eps), out,
                                 then_weight, float(then_eps))
        self.launches += 1
        if take:
            for m in deferred:
                self._sums_taken(m.sums)
                m.sums = None
        return out

    def decay_linear_attention(self, proj, *, num_heads, key_dim, value_dim, decay, state, step,
                               activation, key_scale, cos, sin, decay_logits=None, decay_root=1.0,
                               query_scale=1.0):
        """Portions longer than the kernel's chunk run as chunks side by side (three launches and
        a scratch for the chunks' states); steps of single tokens and short portions are one launch.
        With ``decay_logits`` (float32 ``[T, heads * key_dim]``; ``decay`` is then None) the decay of
        key channel i at token t is ``sigmoid(z)^(1 / decay_root)``. ``query_scale`` multiplies q."""
        T = proj.shape[0]
        out = torch.empty(T, num_heads * value_dim, dtype=torch.float32, device=proj.device)
        L = self._la_chunk = getattr(self, "_la_chunk", None) or int(self.ext.linear_attention_chunk())
        host = getattr(step, "host", None)
        longest = int(host.q_lens.max()) if host is not None else T - (int(step.cu_q.shape[0]) - 2)
        max_chunks = max(1, -(-longest // L))
        scratch = None
        if max_chunks > 1:
            # a chunk's state, and with decays per channel the product of its decays behind them
            per_chunk = num_heads * (value_dim * key_dim + (key_dim if decay_logits is not None else 0))
            need = (T // L + int(step.cu_q.shape[0]) - 1) * per_chunk
            scratch = getattr(self, "_la_scratch", None)
            if scratch is None or scratch.numel() < need:
                if torch.cuda.is_current_stream_capturing():
                    raise RuntimeError("the linear-attention scratch must exist before graph capture")
                # a captured step keeps the address of the scratch it was recorded with: an
                # outgrown scratch is kept alive beside its successor
                self._la_outgrown = getattr(self, "_la_outgrown", []) + ([scratch] if scratch is not None else [])
                scratch = self._la_scratch = torch.empty(need, dtype=torch.float32, device=proj.device)
        self.ext.decay_linear_attention(proj, out, state, decay, step.cu_q, step.ctx_lens, step.state_slots,
                                        num_heads, key_dim, value_dim, cos, sin, activation == "silu",
                                        float(key_scale), max_chunks, scratch, decay_logits, float(decay_root),
                                        float(query_scale))
        self.launches += 3 if max_chunks > 1 else 1
        return out

    def gated_group_norm(self, o, proj, *, gate_offset, group, weight, eps, gate_activation, out_dtype):
        out = torch.empty(o.shape, dtype=out_dtype, device=o.device)
        self.ext.gated_group_norm(o, proj, int(gate_offset), int(group), weight, float(eps),
                                  gate_activation == "sigmoid", out)
        self.launches += 1
        return out

    # ------------------------------------------------------------------ residual streams
    def streams_spread(self, x, streams, scale=1.0):
        """``[T, W]`` float32 to ``[T, streams * W]``: every stream is ``x * scale``."""
        out = torch.empty(x.shape[0], streams * x.shape[1], dtype=torch.float32, device=x.device)
        self.ext.streams_spread(x, out, int(streams), float(scale))
        self.launches += 1
        return out

    def streams_read_norm(self, x, read, weight, eps, streams, out_dtype, rows=None):
        """``u = sum_s read[s] x_s`` of each token (or of the listed rows), RMS-normed with
        ``weight``, in ``out_dtype``."""
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty(n, x.shape[1] // streams, dtype=out_dtype, device=x.device)
        self.ext.streams_read_norm(x, read, weight, float(eps), out, int(streams), rows)
        self.launches += 1
        return out

    def streams_write(self, x, y, scale, mix, out, streams, then_read=None, then_weight=None, then_eps=0.0,
                      out_dtype=None):
        """``x_t <- sum_s mix[s, t] x_s + out[t] * scale * y`` for all streams of every token, in
        place. With ``then_read``: the same launch also returns the read and norm of the new
        streams (what the next sublayer reads). ``y``: a tensor ``[T, W]``, or a product whose
        sums have not been taken yet."""
        sums = None
        if isinstance(y, DeferredProduct):
            if y.sums is not None and (x.shape[1] // streams) % 4 == 0:
                sums, y.sums = y.sums, None
                y = sums
            else:
                y = y.resolve()
        h = None
        if then_read is not None:
            h = torch.empty(x.shape[0], x.shape[1] // streams, dtype=out_dtype, device=x.device)
        self.ext.streams_write(x, y, scale, mix, out, int(streams), then_read, then_weight, float(then_eps), h)
        self.launches += 1
        if sums is not None:
            self._sums_taken(sums)
        return h

    # ------------------------------------------------------------------ rows of q, k, v prepared a token at a time
    def qkv_norm_rope_write(self, qkv, *, num_heads, num_kv_heads, num_value_heads, head_dim, value_dim, out_dim,
                            q_weight, k_weight, eps, positions, token_seq, cos, sin, k_pages, v_pages,
                            block_tables, page_tokens, out_dtype, temp_coef=0.0, temp_every=0):
        """Of the float32 projection ``qkv`` (query heads, key heads, then ``num_value_heads`` value
        heads; 0: a key head's value is its key as projected): RMS norm over all of a token's
        query values and over all of its key values (if weights of those sizes are given), a query
        factor ``1 + temp_coef * ln((pos + 1) // temp_every + 1)``, rotation of the first dims of
        each head that the tables cover, heads filled up to ``out_dim`` with zeros, key/value page
        write (a value head goes to ``num_kv_heads / num_value_heads`` key heads' pages). Returns
        the queries ``[T, num_heads * out_dim]``."""
        q = torch.empty(qkv.shape[0], num_heads * out_dim, dtype=out_dtype, device=qkv.device)
        self.ext.qkv_norm_rope_write(qkv, q, int(num_heads), int(num_kv_heads), int(num_value_heads), int(head_dim),
                                     int(value_dim), int(out_dim), q_weight, k_weight, float(eps), float(temp_coef),
                                     int(temp_every), positions, token_seq, cos, sin, k_pages, v_pages,
                                     block_tables, int(page_tokens))
        self.launches += 1
        return q

    def differential_combine(self, a, proj, *, gate_col0, num_heads, group, head_dim, value_dim, lam, eps,
                             out_scale, out_dtype):
        """``a [T, 2 * heads * head_dim]`` (per key group: its heads' first maps, then their second
        ones) to ``[T, heads * value_dim]``: ``o = a1 - lam * a2``, divided by its root mean square,
        times ``out_scale`` and ``sigmoid(proj[t, gate_col0 + head])``."""
        out = torch.empty(a.shape[0], num_heads * value_dim, dtype=out_dtype, device=a.device)
        self.ext.differential_combine(a, proj, int(gate_col0), int(num_heads), int(group), int(head_dim),
                                      int(value_dim), float(lam), float(eps), float(out_scale), out)
        self.launches += 1
        return out

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature, top_k, top_p, min_p, seed, draw, kinds=3):
        """``kinds``: bit 0 = some row is greedy or cut by top-k / top-p / min-p, bit 1 = some row has
        a temperature and no cut; the kernel of a kind that is promised absent is not launched."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        rows = logits.shape[0]
        if self._sample_scratch is None or self._sample_rows < rows:
            if not torch.cuda.is_current_stream_capturing():
                # results of the blocks that share a row, and a counter per row (zero between launches)
                self._sample_rows = max(rows, 1024)
                self._sample_scratch = torch.zeros(int(self.ext.sample_scratch_ints(self._sample_rows)),
                                                   dtype=torch.int32, device=self.device)
        scratch = self._sample_scratch if self._sample_rows >= rows else None
        self.ext.sample(logits, temperature, top_k, top_p, min_p, seed, draw, out, scratch, kinds)
        self.launches += 1
        return out

    def logsumexp(self, logits):
        out = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
        self.ext.logsumexp(logits, out)
        self.launches += 1
        return out

    def apply_penalties(self, logits, row, token, count, presence, frequency, repetition):
        self.ext.apply_penalties(logits, row, token, count, presence, frequency, repetition)
        self.launches += 1

    def ban_tokens(self, logits, row, token):
        self.ext.ban_tokens(logits, row, token)
        self.launches += 1

    def token_state_add(self, state, slot, token, in_prompt):
        """Enter (slot, token) pairs into the penalties' token state ``[slots, vocab]`` (int32)."""
        self.ext.token_state_add(state, slot, token, in_prompt)
        self.launches += 1

    def apply_penalties_dense(self, logits, row, slot, presence, frequency, repetition, state):
        self.ext.apply_penalties_dense(logits, row, slot, presence, frequency, repetition, state)
        self.launches += 1


_instances: dict[str, CudaOps] = {}


def get_ops(device: torch.device | str = "cuda") -> CudaOps:
    key = str(torch.device(device))
    if key not in _instances:
        _instances[key] = CudaOps(device)
    return _instances[key]
