"""The Lanilorn parts on the GPU: each kernel against the plain float64 function of its mechanism,
then the model through the step function and through generation, against the plain model."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_lanilorn as pl
import traces
from conftest import LANILORN_TINY
from plain_ops import PlainOps

pytestmark = pytest.mark.gpu

F = torch.float64


@pytest.fixture(scope="module")
def ops():
    from llmserve_b200.ops import get_ops

    return get_ops("cuda")


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32).cuda()


def batch(q_lens, starts, slots):
    """The step arrays of a ragged batch (sequence i: q_lens[i] rows from position starts[i])."""
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    host = SimpleNamespace(q_lens=np.asarray(q_lens, dtype=np.int32),
                           ctx_lens=(np.asarray(starts) + np.asarray(q_lens)).astype(np.int32))
    return SimpleNamespace(
        cu_q=i32(cu), ctx_lens=i32(host.ctx_lens), state_slots=i32(slots),
        token_seq=i32(np.repeat(np.arange(len(q_lens)), q_lens)),
        positions=i32(np.concatenate([np.arange(s, s + n) for s, n in zip(starts, q_lens)])),
        host=host, decode_splits=0,
        max_decode_ctx=int(max([s + n for s, n in zip(starts, q_lens) if n == 1], default=0)))


def close(got, ref, tol, what=""):
    err = (got.double().cpu() - ref.double()).abs().max().item()
    bound = tol * max(1.0, ref.abs().max().item())
    assert err <= bound, f"{what}: {err:.3e} > {bound:.3e}"


# ----------------------------------------------------------------------------- residual streams
@pytest.mark.parametrize("T,W,S", [(5, 64, 2), (3, 75, 3), (9, 2048, 4), (2, 96, 1), (4, 50, 8), (3, 128, 12), (2, 33, 16)])
def test_streams_spread_read_and_write(ops, T, W, S):
    x0 = rnd(T, W, seed=1)
    x = ops.streams_spread(x0.cuda(), S, 1.75)
    assert torch.equal(x.cpu(), (x0 * 1.75).repeat(1, S))
    X = rnd(T, S, W, seed=2).to(F)
    read, w, mix, out, ls = (rnd(S, seed=3).to(F), 1 + rnd(W, seed=4).to(F), rnd(S, S, seed=5).to(F),
                             rnd(S, seed=6).to(F), 1 + rnd(W, seed=7).to(F))
    y = rnd(T, W, seed=8).to(F)
    f32 = lambda t: t.float().cuda().contiguous()
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 6e-3)):
        got = ops.streams_read_norm(f32(X.reshape(T, S * W)), f32(read), f32(w), 1e-5, S, dtype)
        close(got, pl.weighted_norm(pl.streams_read(X, read), w, 1e-5), tol, "read")
        rows = i32([T - 1, 0])
        got = ops.streams_read_norm(f32(X.reshape(T, S * W)), f32(read), f32(w), 1e-5, S, dtype, rows=rows)
        close(got, pl.weighted_norm(pl.streams_read(X, read), w, 1e-5)[[T - 1, 0]], tol, "read of some rows")
    new = pl.streams_write(X, y * ls, mix, out)
    xs = f32(X.reshape(T, S * W))
    assert ops.streams_write(xs, f32(y), f32(ls), f32(mix), f32(out), S) is None
    close(xs, new.reshape(T, S * W), 2e-6, "write")
    xs = f32(X.reshape(T, S * W))
    ops.streams_write(xs, f32(y), None, f32(mix), f32(out), S)  # without a scale per channel
    close(xs, pl.streams_write(X, y, mix, out).reshape(T, S * W), 2e-6, "write without scale")
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 6e-3)):
        xs = f32(X.reshape(T, S * W))
        h = ops.streams_write(xs, f32(y), f32(ls), f32(mix), f32(out), S, then_read=f32(read), then_weight=f32(w),
                              then_eps=1e-5, out_dtype=dtype)
        close(xs, new.reshape(T, S * W), 2e-6, "write before the read")
        close(h, pl.weighted_norm(pl.streams_read(new, read), w, 1e-5), tol, "the read that follows")


def test_streams_write_takes_a_products_sums(ops):
    """A few-rows product handed on as fixed-point sums is written into the streams by the same kernel."""
    from llmserve_b200.ops.cuda_ops import DeferredProduct

    T, W, S, K = 4, 64, 3, 128
    a, wt = rnd(T, K, seed=1).bfloat16().cuda(), rnd(W, K, seed=2, scale=0.1).bfloat16().cuda()
    y = ops.linear(a, wt, None, out_dtype=torch.float32, may_defer=True)
    if not isinstance(y, DeferredProduct):
        pytest.skip("this kernel set does not defer few-rows products")
    X = rnd(T, S, W, seed=3)
    mix, out = rnd(S, S, seed=4), rnd(S, seed=5)
    xs = X.reshape(T, S * W).cuda().contiguous()
    ops.streams_write(xs, y, None, mix.cuda(), out.cuda(), S)
    ref = pl.streams_write(X.to(F), a.cpu().to(F) @ wt.cpu().to(F).T, mix.to(F), out.to(F))
    close(xs, ref.reshape(T, S * W), 1e-5)
    again = ops.linear(a, wt, None, out_dtype=torch.float32)  # the buffer was left zero
    close(again, a.cpu().to(F) @ wt.cpu().to(F).T, 1e-5)


# ----------------------------------------------------------------------------- q, k, v rows of a token
def pages_for(n_seq, max_len, page_tokens, nk, Dp, dtype, seed=0, fill=float("nan")):
    """Shuffled block tables and pages filled with ``fill`` (NaN shows a row that should not have been written)."""
    per = -(-max_len // page_tokens)
    order = torch.randperm(n_seq * per + 3, generator=torch.Generator().manual_seed(seed))[: n_seq * per]
    tables = order.view(n_seq, per).to(torch.int32).cuda()
    k = torch.full((n_seq * per + 3, nk, page_tokens, Dp), fill, dtype=dtype).cuda()
    return tables, k, k.clone()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nk,nv,D,Dv,rot,temp,page_tokens", [
    (4, 2, 0, 32, 32, 12, None, 16),    # values are keys, part of the head rotated
    (3, 3, 0, 24, 24, 24, None, 8),     # a head size that is filled up, whole head rotated
    (8, 4, 2, 16, 40, 0, (0.5, 4), 16), # two maps per head: value heads repeated, a query temperature
    (2, 2, 1, 10, 50, 0, None, 8),
    (6, 1, 0, 18, 18, 6, (1.0, 1), 16),
])
def test_rows_are_normed_turned_filled_up_and_find_their_pages(ops, dtype, nq, nk, nv, D, Dv, rot, temp, page_tokens):
    q_lens, starts = [5, 1, 9], [0, 37, 14]
    b = batch(q_lens, starts, [0, 1, 2])
    T = sum(q_lens)
    Dp = max(D, Dv if nv else D)
    Dp += -Dp % 16
    width = (nq + nk) * D + nv * Dv + 5  # something behind the heads that is not read
    proj = rnd(T, width, seed=1)
    normed = nv == 0
    qw, kw = (0.5 + torch.rand(nq * D), 0.5 + torch.rand(nk * D)) if normed else (None, None)
    cos = sin = None
    if rot:
        f, mag = pl.yarn_frequencies(rot, 300.0, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0})
        ang = torch.arange(64, dtype=F)[:, None] * f[None, :]
        cos, sin = (ang.cos() * mag).float().cuda(), (ang.sin() * mag).float().cuda()
    tables, kp, vp = pages_for(3, 48, page_tokens, nk, Dp, dtype)
    got = ops.qkv_norm_rope_write(
        proj.cuda(), num_heads=nq, num_kv_heads=nk, num_value_heads=nv, head_dim=D, value_dim=Dv, out_dim=Dp,
        q_weight=qw.cuda() if normed else None, k_weight=kw.cuda() if normed else None, eps=1e-5,
        temp_coef=temp[0] if temp else 0.0, temp_every=temp[1] if temp else 0,
        positions=b.positions, token_seq=b.token_seq, cos=cos, sin=sin, k_pages=kp, v_pages=vp,
        block_tables=tables, page_tokens=page_tokens, out_dtype=dtype)
    pos = b.positions.cpu().long()
    p = proj.to(F)
    q, k = p[:, : nq * D], p[:, nq * D : (nq + nk) * D]
    v = k.view(T, nk, D) if nv == 0 else p[:, (nq + nk) * D : (nq + nk) * D + nv * Dv].view(T, nv, Dv).repeat_interleave(nk // nv, 1)
    if normed:
        q, k = pl.weighted_norm(q, qw.to(F), 1e-5), pl.weighted_norm(k, kw.to(F), 1e-5)
    if temp:
        q = q * (1.0 + temp[0] * torch.log(torch.floor((pos.to(F) + 1) / temp[1]) + 1.0))[:, None]
    q, k = q.view(T, nq, D), k.view(T, nk, D)
    if rot:
        sc = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
        q, k = pl.rotate_half_part(q, pos, rot, 300.0, sc), pl.rotate_half_part(k, pos, rot, 300.0, sc)
    tol = 3e-6 if dtype == torch.float32 else 5e-3
    fill = lambda x: torch.nn.functional.pad(x, (0, Dp - x.shape[-1]))
    close(got.view(T, nq, Dp), fill(q), tol, "queries")
    seq = b.token_seq.cpu().long()
    page = tables.cpu()[seq, pos // page_tokens].long()
    close(kp[page.cuda(), :, (pos % page_tokens).cuda()], fill(k), tol, "keys in their pages")
    close(vp[page.cuda(), :, (pos % page_tokens).cuda()], fill(v), tol, "values in their pages")
    written = torch.zeros(kp.shape[0], page_tokens, dtype=torch.bool)
    written[page, pos % page_tokens] = True
    assert torch.isnan(kp.float().cpu().permute(0, 2, 1, 3)[~written]).all(), "rows of other tokens were touched"
    # a layer that only reads writes no pages
    got2 = ops.qkv_norm_rope_write(
        proj.cuda(), num_heads=nq, num_kv_heads=nk, num_value_heads=nv, head_dim=D, value_dim=Dv, out_dim=Dp,
        q_weight=qw.cuda() if normed else None, k_weight=kw.cuda() if normed else None, eps=1e-5,
        temp_coef=temp[0] if temp else 0.0, temp_every=temp[1] if temp else 0,
        positions=b.positions, token_seq=b.token_seq, cos=cos, sin=sin, k_pages=None, v_pages=None,
        block_tables=tables, page_tokens=page_tokens, out_dtype=dtype)
    assert torch.equal(got2, got)


# ----------------------------------------------------------------------------- attention with sinks and a window, through the mixer's ops
def attend_paged(ops, dtype, H, G, D, page_tokens, window, n_rows, ctx, splits, sinks, q, k, v, scale, out_dtype=None):
    """One sequence of ``ctx`` tokens whose last ``n_rows`` are this step's queries."""
    b = batch([n_rows], [ctx - n_rows], [0])
    b.decode_splits = splits if n_rows == 1 else 0
    tables, kp, vp = pages_for(1, ctx, page_tokens, G, D, dtype, seed=3, fill=0.5)
    pos = torch.arange(ctx)
    page = tables.cpu()[0, pos // page_tokens].long().cuda()
    kp[page, :, (pos % page_tokens).cuda()] = k.to(dtype).cuda()
    vp[page, :, (pos % page_tokens).cuda()] = v.to(dtype).cuda()
    plan = {n: torch.from_numpy(a).cuda() for n, a in ops.attention_plan(b.host, dtype, D).items()}
    ops.check_attention_shape(D, dtype, H, G)
    return ops.paged_attention(
        q[ctx - n_rows:].reshape(n_rows, H * D).to(dtype).cuda().contiguous(), num_heads=H, num_kv_heads=G,
        head_dim=D, scale=scale, window=window, k_pages=kp, v_pages=vp, block_tables=tables, page_tokens=page_tokens,
        step=b, plan=plan, sinks=None if sinks is None else sinks.float().cuda(), out_dtype=out_dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_rows,splits", [(1, 1), (1, 3), (40, 0), (2, 0)])
@pytest.mark.parametrize("edge", ["inside", "outside", "far inside", "first"])
@pytest.mark.parametrize("D,window", [(32, 37), (64, 37), (64, 32)])  # 64: single tokens in bfloat16 run on the
# tensor-core kernel; a window of 37 ends in the middle of a page, one of 32 at a page's border
def test_a_planted_key_at_the_windows_edge_and_a_sink_that_counts(ops, dtype, n_rows, splits, edge, D, window):
    """One key matches the last query far better than all others. Just inside the window it takes
    the softmax's weight beside the sink; just outside it is not seen and the sink (which has no
    value) takes what random keys leave."""
    H, G, page_tokens, ctx = 4, 2, 16, 150 if window == 37 else 160
    q, k, v = rnd(ctx, H, D, seed=1, scale=0.3), rnd(ctx, G, D, seed=2, scale=0.3), rnd(ctx, G, D, seed=3)
    at = {"inside": ctx - window, "outside": ctx - window - 1, "far inside": ctx - 3, "first": 0}[edge]
    k[at] = 0
    k[at, :, 0] = 6.0
    q[-1] = 0
    q[-1, :, 0] = 6.0
    sinks = torch.tensor([3.0, -2.0, 8.0, 0.5])
    got = attend_paged(ops, dtype, H, G, D, page_tokens, window, n_rows, ctx, splits, sinks, q, k, v, 0.5)
    ref = pl.attend(q.to(F), k.to(F), v.to(F), 0.5, pl.causal(ctx, window), sinks.to(F))[ctx - n_rows:]
    close(got.view(n_rows, H, D), ref, 2e-5 if dtype == torch.float32 else 2e-2, edge)
    seen = edge in ("inside", "far inside")
    weight_on_planted = (ref[-1, 0] - v[at, 0].to(F)).abs().max().item() < 0.05
    assert weight_on_planted == seen
    if n_rows > 1:  # rows without a planted key share their weight with the sink
        without = pl.attend(q.to(F), k.to(F), v.to(F), 0.5, pl.causal(ctx, window), None)[ctx - n_rows:]
        assert (without - ref).abs().max().item() > 0.1, "the sink must matter in this test"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_rows,splits", [(1, 1), (1, 4), (64, 0)])
def test_a_far_key_among_hundreds_without_a_window(ops, dtype, n_rows, splits):
    H, G, D, ctx = 4, 4, 64, 700
    q, k, v = rnd(ctx, H, D, seed=1, scale=0.2), rnd(ctx, G, D, seed=2, scale=0.2), rnd(ctx, G, D, seed=3)
    k[5] = 0
    k[5, :, 3] = 7.0
    q[-1] = 0
    q[-1, :, 3] = 7.0
    got = attend_paged(ops, dtype, H, G, D, 16, 0, n_rows, ctx, splits, None, q, k, v, 0.4)
    ref = pl.attend(q.to(F), k.to(F), v.to(F), 0.4, pl.causal(ctx), None)[ctx - n_rows:]
    close(got.view(n_rows, H, D), ref, 2e-5 if dtype == torch.float32 else 2e-2)
    assert (ref[-1] - v[5].to(F)).abs().max().item() < 0.05


@pytest.mark.parametrize("n_rows,splits", [(1, 1), (1, 3), (50, 0), (2, 0)])
@pytest.mark.parametrize("H,G,D", [(4, 2, 64), (4, 4, 128), (12, 1, 64), (3, 3, 48), (2, 1, 160)])
def test_bfloat16_attention_hands_its_results_on_in_float32(ops, n_rows, splits, H, G, D):
    """Asked for a float32 out, every kernel that serves the call gives what it gives in
    bfloat16 before the last rounding: the two agree to that rounding, and the float32 one is the
    nearer to the plain result."""
    ctx = 200
    q, k, v = rnd(ctx, H, D, seed=1, scale=0.3), rnd(ctx, G, D, seed=2, scale=0.3), rnd(ctx, G, D, seed=3)
    args = (ops, torch.bfloat16, H, G, D, 16, 0, n_rows, ctx, splits, None, q, k, v, 0.3)
    wide = attend_paged(*args, out_dtype=torch.float32)
    narrow = attend_paged(*args)
    assert wide.dtype == torch.float32 and narrow.dtype == torch.bfloat16
    r = lambda t: t.bfloat16().to(F)  # the operands the bfloat16 kernels see
    ref = pl.attend(r(q), r(k), r(v), 0.3, pl.causal(ctx), None)[ctx - n_rows:].reshape(n_rows, H * D)
    close(narrow, wide.cpu(), 8e-3)
    assert (wide.double().cpu() - ref).abs().max() <= (narrow.double().cpu() - ref).abs().max() + 1e-6
    close(wide, ref, 6e-3)


# ----------------------------------------------------------------------------- the two maps combined
@pytest.mark.parametrize("dtype,a_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                           (torch.bfloat16, torch.float32)])  # maps in float32, result rounded once
@pytest.mark.parametrize("T,H,n,Dp,Dv", [(5, 4, 2, 32, 32), (3, 3, 3, 48, 24), (7, 2, 1, 64, 50), (2, 6, 2, 16, 10)])
def test_differential_combine(ops, dtype, a_dtype, T, H, n, Dp, Dv):
    a = rnd(T, 2 * H * Dp, seed=1).to(a_dtype)
    gate = rnd(T, 11 + H, seed=2)
    lam, eps, out_scale = 0.37, 1e-5, 0.6
    got = ops.differential_combine(a.cuda(), gate.cuda(), gate_col0=11, num_heads=H, group=n, head_dim=Dp,
                                   value_dim=Dv, lam=lam, eps=eps, out_scale=out_scale, out_dtype=dtype)
    maps = a.to(F).view(T, H // n, 2, n, Dp)[..., :Dv]
    o = (maps[:, :, 0] - lam * maps[:, :, 1]).reshape(T, H, Dv)
    ref = pl.unit_rms(o, eps) * out_scale * torch.sigmoid(gate[:, 11:].to(F))[:, :, None]
    close(got.view(T, H, Dv), ref, 3e-6 if dtype == torch.float32 else 8e-3)


def test_differential_attention_against_two_plain_softmaxes(ops):
    """The mixer's op sequence on one sequence, cut into a portion and single tokens, with grouped
    heads: every map must meet its own keys and both the same values."""
    from llmserve_b200.parts.base import BuildEnv
    from llmserve_b200.parts.differential_attention import DifferentialAttention, DifferentialAttentionSpec

    W, H, G, d, dv, n = 48, 4, 2, 16, 24, 21
    spec = DifferentialAttentionSpec(W, H, G, d, dv, scale=0.3, eps=1e-5, lam_offset=0.4, out_scale=0.6,
                                     temp_coef=0.5, temp_every=4)
    w = {"q": rnd(2 * H * d, W, seed=1), "k": rnd(2 * G * d, W, seed=2), "v": rnd(G * dv, W, seed=3),
         "g": rnd(H, W, seed=4), "o": rnd(W, H * dv, seed=5, scale=0.2),
         "lq1": rnd(d, seed=6, scale=0.3), "lk1": rnd(d, seed=7, scale=0.3), "lq2": rnd(d, seed=8, scale=0.3),
         "lk2": rnd(d, seed=9, scale=0.3)}
    h = rnd(n, W, seed=10, scale=0.5)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": 0.3, "diff": 0.4, "q_temp": {"coef": 0.5, "every": 4}}
    ref = pl.differential_attention(h.to(F), {k_: v_.to(F) for k_, v_ in w.items()}, "", m, 1e-5)
    for kernel_set, device in ((PlainOps(), "cpu"), (ops, "cuda")):
        env = BuildEnv(ops=kernel_set, dtype=torch.float32, device=torch.device(device), max_positions=64,
                       branch_dtype=torch.float32)
        part = DifferentialAttention(spec, env)
        part.bind({"qkv.weight": torch.cat([w["q"], w["k"], w["v"], w["g"]]).to(device), "o.weight": w["o"].to(device),
                   "lam.q1": w["lq1"].to(device), "lam.k1": w["lk1"].to(device), "lam.q2": w["lq2"].to(device),
                   "lam.k2": w["lk2"].to(device)})
        need = part.cache_need()
        pt = 8
        kp = torch.zeros(8, need.num_kv_heads, pt, need.head_dim, device=device)
        vp = torch.zeros_like(kp)
        tables = torch.tensor([[5, 2, 7, 1]], dtype=torch.int32, device=device)
        outs = []
        for a, b_ in ((0, 13), (13, 14), (14, n)):
            step = batch([b_ - a], [a], [0]) if device == "cuda" else None
            host = SimpleNamespace(q_lens=np.asarray([b_ - a], dtype=np.int32), ctx_lens=np.asarray([b_], dtype=np.int32))
            mk = (lambda x: i32(x)) if device == "cuda" else (lambda x: torch.tensor(np.asarray(x), dtype=torch.int32))
            step = SimpleNamespace(cu_q=mk([0, b_ - a]), ctx_lens=mk([b_]), token_seq=mk([0] * (b_ - a)),
                                   positions=mk(list(range(a, b_))), host=host, decode_splits=0,
                                   max_decode_ctx=b_ if b_ - a == 1 else 0, block_tables={0: tables})
            plan = kernel_set.attention_plan(host, torch.float32, need.head_dim)
            step.plans = {part.plan_key(): {k_: torch.from_numpy(v_).to(device) for k_, v_ in plan.items()}}
            cache = SimpleNamespace(k=kp, v=vp, writes=True, group=0, page_tokens=pt)
            outs.append(part.forward(h[a:b_].to(device), step, cache))
        close(torch.cat(outs), ref, 1e-5, device)


# ----------------------------------------------------------------------------- linear attention with a decay per channel and token
def plain_gla(proj, z, H, dk, dv, tau, qs, state0=None):
    """float64: returns outputs [n, H*dv] and the final state [H, dv, dk]."""
    n = proj.shape[0]
    p = proj.to(F)
    q = p[:, : H * dk].view(n, H, dk) * qs
    k = p[:, H * dk : 2 * H * dk].view(n, H, dk)
    v = p[:, 2 * H * dk : 2 * H * dk + H * dv].view(n, H, dv)
    alpha = (torch.sigmoid(z.to(F)) ** (1.0 / tau)).view(n, H, dk)
    S = torch.zeros(H, dk, dv, dtype=F) if state0 is None else state0.to(F).transpose(1, 2).clone()
    o = torch.zeros(n, H, dv, dtype=F)
    for t in range(n):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o.reshape(n, H * dv), S.transpose(1, 2)


@pytest.mark.parametrize("H,dk,dv,tau", [(2, 16, 24, 8.0), (3, 20, 12, 16.0), (1, 48, 64, 1.0), (4, 128, 128, 4.0),
                                         (2, 64, 40, 2.0)])
def test_gated_linear_attention_in_portions_chunks_and_single_tokens(ops, H, dk, dv, tau):
    """A ragged batch: a long portion that runs as several chunks side by side, a portion that
    goes on from a state, a sequence's first token, a single token behind a state; then the same
    sequences go on one token at a time. Slots hold garbage where a sequence starts."""
    L = int(ops.ext.linear_attention_chunk())
    q_lens, starts, slots = [3 * L + 7, 9, 1, 1, L + 1], [0, 5, 0, 30, 11], [3, 0, 4, 1, 2]
    b = batch(q_lens, starts, slots)
    T = sum(q_lens)
    width = 2 * H * dk + 2 * H * dv
    proj = rnd(T, width, seed=1, scale=0.5)
    z = rnd(T, H * dk + 3, seed=2, scale=2.0) + 2.0
    state = rnd(6, H, dv, dk, seed=3)
    state_dev = state.cuda().contiguous()
    qs = dk ** -0.5
    got = ops.decay_linear_attention(
        proj.cuda(), num_heads=H, key_dim=dk, value_dim=dv, decay=None, state=state_dev, step=b, activation="none",
        key_scale=1.0, cos=None, sin=None, decay_logits=z.cuda().contiguous(), decay_root=tau, query_scale=qs)
    at, finals = 0, []
    for n, s0, slot in zip(q_lens, starts, slots):
        ref, S = plain_gla(proj[at : at + n], z[at : at + n, : H * dk], H, dk, dv, tau, qs, state[slot] if s0 else None)
        close(got[at : at + n], ref, 2e-5, f"sequence of {n} from {s0}")
        close(state_dev[slot], S, 2e-5, "state left behind")
        finals.append(S)
        at += n
    assert torch.equal(state_dev[5].cpu(), state[5]), "a slot that no sequence uses was touched"
    # the plain kernel set agrees (it is the engine's CPU stand-in)
    cpu_state = state.clone()
    cb = SimpleNamespace(cu_q=b.cu_q.cpu(), ctx_lens=b.ctx_lens.cpu(), state_slots=b.state_slots.cpu(), positions=b.positions.cpu())
    ref_all = PlainOps().decay_linear_attention(
        proj, num_heads=H, key_dim=dk, value_dim=dv, decay=None, state=cpu_state, step=cb, activation="none",
        key_scale=1.0, cos=None, sin=None, decay_logits=z[:, : H * dk], decay_root=tau, query_scale=qs)
    close(got, ref_all, 3e-5)
    # every sequence goes on, one token each, for a few steps
    for step_no in range(3):
        nb = batch([1] * 5, [s + n + step_no for s, n in zip(starts, q_lens)], slots)
        p1, z1 = rnd(5, width, seed=10 + step_no, scale=0.5), rnd(5, H * dk, seed=20 + step_no, scale=2.0)
        got1 = ops.decay_linear_attention(
            p1.cuda(), num_heads=H, key_dim=dk, value_dim=dv, decay=None, state=state_dev, step=nb,
            activation="none", key_scale=1.0, cos=None, sin=None, decay_logits=z1.cuda(), decay_root=tau, query_scale=qs)
        for i in range(5):
            ref, finals[i] = plain_gla(p1[i : i + 1], z1[i : i + 1], H, dk, dv, tau, qs, finals[i])
            close(got1[i : i + 1], ref, 2e-5, "single token")


def test_a_decay_that_forgets_and_one_that_keeps(ops):
    """Channels whose logit is very negative forget the state at once; very positive ones keep it:
    with keys on single channels the output shows which tokens are still there."""
    H, dk, dv, n = 1, 16, 16, 70
    proj = torch.zeros(n, 2 * dk + 2 * dv)
    proj[:, 0:2] = 1.0                      # every query reads channels 0 and 1
    proj[0, dk + 0] = 1.0                   # token 0 writes channel 0 ...
    proj[0, dk + 1] = 1.0                   # ... and channel 1
    proj[0, 2 * dk : 2 * dk + dv] = torch.arange(dv) + 1.0
    z = torch.zeros(n, dk)
    z[:, 0] = 30.0                          # channel 0 keeps
    z[:, 1] = -30.0                         # channel 1 forgets: alpha = sigmoid(-30)^(1/2)
    b = batch([n], [0], [0])
    state = torch.zeros(1, H, dv, dk).cuda()
    got = ops.decay_linear_attention(proj.cuda(), num_heads=H, key_dim=dk, value_dim=dv, decay=None, state=state,
                                     step=b, activation="none", key_scale=1.0, cos=None, sin=None,
                                     decay_logits=z.cuda(), decay_root=2.0, query_scale=1.0)
    v0 = torch.arange(dv) + 1.0
    close(got[0], 2 * v0, 1e-6)          # both channels hold token 0 at its own step
    close(got[1], v0, 1e-5)              # one step later only the kept channel does
    close(got[n - 1], v0, 1e-5)          # and still does after a chunk border


# ----------------------------------------------------------------------------- the model
def gpu_runner(folder, name, num_pages, dtype, max_num_seqs=4, max_len=512):
    from llmserve_b200.engine.runner import ModelRunner, load_model
    from llmserve_b200.ops import get_ops

    _, _, model = load_model(folder, dtype, "cuda", get_ops("cuda"), max_len)
    return ModelRunner(model, page_tokens=LANILORN_TINY[name]["page_tokens"], num_pages=num_pages,
                       max_model_len=max_len, max_num_seqs=max_num_seqs, max_num_batched_tokens=max_len)


LENGTHS = {"L1": [5, 70, 1, 33, 49, 126, 2], "L2": [2, 40, 9, 64, 17, 100], "L3": [3, 150, 18, 77, 230]}
TOL = {"float32": (2e-4, 5e-5), "bfloat16": (0.0, 0.03)}  # (absolute, relative to the largest logit)


@pytest.fixture(scope="module")
def expected(lanilorn_dirs):
    out = {}
    for name in LANILORN_TINY:
        reqs = traces.make_requests(LENGTHS[name], LANILORN_TINY[name]["config"]["vocab"], seed=5)
        out[name] = (reqs, {r: pl.model_logits(lanilorn_dirs[name], t) for r, t in reqs.items()})
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["L1", "L2", "L3"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_plain(lanilorn_dirs, expected, name, mode, dtype):
    reqs, exp = expected[name]
    pool_tokens = traces.tokens_needed(reqs)
    runner = gpu_runner(lanilorn_dirs[name], name, pool_tokens // LANILORN_TINY[name]["page_tokens"], dtype)
    got = traces.replay(runner, getattr(traces, mode)(reqs))
    atol, rtol = TOL[dtype]
    traces.compare(got, exp, atol=atol, rtol=rtol)
    assert runner.manager.usage() == 0.0
    runner.check_kernels()


@pytest.mark.parametrize("name", ["L1", "L2", "L3"])
def test_layers_one_by_one_in_float32(lanilorn_dirs, name):
    """The sum of the streams after every layer against the plain model's."""
    folder = lanilorn_dirs[name]
    tokens = traces.make_requests([90], LANILORN_TINY[name]["config"]["vocab"], seed=2)["r0"]
    cfg, w = pl.load(folder)
    _, after = pl.forward(tokens, w, cfg, return_layers=True)
    runner = gpu_runner(folder, name, 16, "float32")
    model, seen, n = runner.model, [], cfg["streams"]
    for block in model.blocks:
        inner = block.forward

        def spy(x, pending, step, cache, inner=inner):
            x, pending = inner(x, pending, step, cache)
            assert pending.resolve() is None  # the layer's last write, left for the next norm: done now
            seen.append(x.view(x.shape[0], n, -1).sum(1))
            return x, None

        block.forward = spy
    from llmserve_b200.engine.batch import StepEntry

    runner.run([StepEntry("a", tokens, [0])])
    assert len(seen) == len(cfg["layers"])
    for i, x in enumerate(seen):
        close(x, after[i], 2e-5, f"after layer {i}")


def test_float32_logits_do_not_depend_on_the_cut(lanilorn_dirs, expected):
    reqs, _ = expected["L1"]
    pool = traces.tokens_needed(reqs) // 16
    a = traces.replay(gpu_runner(lanilorn_dirs["L1"], "L1", pool, "float32"), traces.whole(reqs))
    b = traces.replay(gpu_runner(lanilorn_dirs["L1"], "L1", pool, "float32"), traces.mixed(reqs, seed=4))
    scale = max(v.abs().max().item() for v in a.values())
    assert max((a[k] - b[k]).abs().max().item() for k in a) <= 2e-5 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(lanilorn_dirs, dtype):
    """300 tokens one by one from position 0: every window passes over decoded tokens, pages that a
    window has left are given back while the request lives, the state is carried through every step."""
    reqs = traces.make_requests([300], 130, seed=21)
    exp = {r: pl.model_logits(lanilorn_dirs["L2"], t) for r, t in reqs.items()}
    runner = gpu_runner(lanilorn_dirs["L2"], "L2", 38, dtype)
    got = traces.replay(runner, traces.decode_tail(reqs, tail=300))
    atol, rtol = TOL[dtype]
    traces.compare(got, exp, atol=atol, rtol=rtol)
    assert any(spec.window > 0 for spec in runner.manager.groups) and runner.manager.usage() == 0.0


def test_slots_and_pages_used_again(lanilorn_dirs):
    """One state slot and just enough pages: every request runs on what the one before it left."""
    reqs = traces.make_requests([40, 37, 64, 3], 157, seed=8)
    exp = {r: pl.model_logits(lanilorn_dirs["L1"], t) for r, t in reqs.items()}
    runner = gpu_runner(lanilorn_dirs["L1"], "L1", 4, "float32", max_num_seqs=1)
    traces.compare(traces.replay(runner, traces.portions(reqs)), exp, atol=2e-4, rtol=2e-5)


# ----------------------------------------------------------------------------- generation
PROMPTS = [[5, 9, 90, 31, 7], list(range(40, 57)), [3] * 33, [90, 2], list(range(70))]


def llm(folder, name, dtype, **kw):
    from llmserve_b200 import LLM

    d = dict(dtype=dtype, block_size=LANILORN_TINY[name]["page_tokens"], num_kv_blocks=64, max_model_len=256,
             max_num_seqs=8)
    d.update(kw)
    return LLM(str(folder), **d)


def greedy(n):
    from llmserve_b200 import SamplingParams

    return SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)


@pytest.mark.parametrize("name", ["L1", "L2"])
@pytest.mark.parametrize("kw", [dict(cuda_graphs=False), dict(cuda_graphs=True),
                                dict(cuda_graphs=True, max_num_batched_tokens=24),
                                dict(cuda_graphs=True, num_kv_blocks=14, max_num_batched_tokens=16)])
def test_greedy_float32_equals_plain_greedy(lanilorn_dirs, name, kw):
    """Through the entry point: the scheduler's batches, captured steps (single tokens and padded
    steps with portions), preemption by recomputation."""
    m = llm(lanilorn_dirs[name], name, "float32", **kw)
    outs = m.generate(PROMPTS, greedy(12))
    for o, p in zip(outs, PROMPTS):
        assert o.outputs[0].token_ids == pl.greedy(lanilorn_dirs[name], p, 12), (kw, p)


def test_greedy_bfloat16_picks_tokens_the_plain_model_also_ranks_first(lanilorn_dirs):
    outs = llm(lanilorn_dirs["L1"], "L1", "bfloat16", cuda_graphs=True).generate(PROMPTS, greedy(10))
    for o, p in zip(outs, PROMPTS):
        gen = o.outputs[0].token_ids
        logits = pl.model_logits(lanilorn_dirs["L1"], p + gen)[len(p) - 1 : -1]
        for t, row in zip(gen, logits):
            assert float(row.max() - row[t]) <= 0.03 * float(row.abs().max())


def wanted_subsets(make_runner, folder, vocab):
    """Steps that want some rows, one row or none: the model's last norm then reads only those rows,
    and a step's last write into the streams is carried out without a read behind it."""
    from llmserve_b200.engine.batch import StepEntry

    reqs = traces.make_requests([41, 30], vocab, seed=13)
    exp = {r: pl.model_logits(folder, t) for r, t in reqs.items()}
    runner = make_runner()
    a, b = reqs["r0"], reqs["r1"]
    steps = [([("r0", a[:17], [3, 16]), ("r1", b[:9], [])], None),
             ([("r0", a[17:18], []), ("r1", b[9:22], [0, 12])], None),
             ([("r0", a[18:19], [0]), ("r1", b[22:23], [])], None),
             ([("r0", a[19:41], [21]), ("r1", b[23:30], [6, 2])], None)]
    at = {"r0": 0, "r1": 0}
    for entries, _ in steps:
        logits = runner.run([StepEntry(r, t, w) for r, t, w in entries]).float().cpu()
        row = 0
        for r, t, w in entries:
            for k in w:
                ref = exp[r][at[r] + k]
                assert (logits[row] - ref).abs().max().item() <= 2e-4 + 5e-5 * ref.abs().max().item(), (r, at[r] + k)
                row += 1
            at[r] += len(t)
        assert row == logits.shape[0]


@pytest.mark.parametrize("name", ["L1", "L2"])
def test_steps_that_want_some_rows_or_none(lanilorn_dirs, name):
    wanted_subsets(lambda: gpu_runner(lanilorn_dirs[name], name, 16, "float32"), lanilorn_dirs[name], LANILORN_TINY[name]["config"]["vocab"])
