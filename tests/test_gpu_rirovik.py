"""The Rirovik parts on the GPU: each kernel against the plain float64 function of its mechanism,
then the model through the step function and through generation, against the plain model."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_rirovik as pr
import traces
from conftest import RIROVIK_TINY

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


def tables(rot, base, n):
    ang = torch.arange(n, dtype=F)[:, None] * base ** (-2.0 * torch.arange(rot // 2, dtype=F) / rot)[None, :]
    return ang.cos().float().cuda(), ang.sin().float().cuda()


# ----------------------------------------------------------------------------- latent rows with a rotated part
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Rq,R,Dr,rot,page_tokens", [(24, 40, 8, 8, 16), (10, 22, 4, 2, 8), (96, 128, 32, 32, 32),
                                                     (0, 18, 6, 6, 4), (14, 0, 0, 0, 8), (33, 7, 10, 0, 16)])
def test_latent_rows_are_normed_turned_and_find_their_page(ops, dtype, Rq, R, Dr, rot, page_tokens):
    """Two sequences whose tokens cross page borders, in shuffled pages; the query latent beside
    the key/value latent and the key part; only the first ``rot`` dims of the key part turn."""
    q_lens, starts = [13, 1], [5, 3 * page_tokens - 1]
    st = batch(q_lens, starts, [0, 1])
    T = sum(q_lens)
    extra = 5  # columns behind the key part (a gate's)
    proj = rnd(T, Rq + R + Dr + extra, seed=R + Rq, scale=2.0)
    qw, kw = 1 + rnd(max(Rq, 1), seed=1, scale=0.3)[:Rq], 1 + rnd(max(R, 1), seed=2, scale=0.3)[:R]
    Rp = R + Dr + (-(R + Dr)) % 16
    n_pages = 4 + 2 * (3 + 16 // page_tokens)
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3))
    bt = order[: 2 * (n_pages // 2)].view(2, -1)
    pages = torch.full((n_pages, 1, page_tokens, max(Rp, 16)), 7.0, dtype=dtype).cuda()
    cos, sin = tables(rot, 300.0, 200) if rot else (None, None)
    cq = ops.latent_rope_write(
        proj.cuda(), q_col0=0, q_weight=qw.cuda() if Rq else None, kv_col0=Rq, kv_weight=kw.cuda() if R else None,
        rot_dim=Dr, rot=rot, eps=1e-5, cos=cos, sin=sin, pages=pages, positions=st.positions, token_seq=st.token_seq,
        block_tables=i32(bt.tolist()), out_dtype=dtype)
    tol = 2e-6 if dtype == torch.float32 else 5e-3
    if Rq:
        close(cq, pr.plain_norm(proj[:, :Rq].to(F), qw.to(F), 1e-5), tol, "query latent")
    else:
        assert cq is None
    if not R:
        assert float((pages.float() - 7.0).abs().max()) == 0.0
        return
    pos = st.positions.cpu().tolist()
    seq = st.token_seq.cpu().tolist()
    for t in range(T):
        c = pr.plain_norm(proj[t : t + 1, Rq : Rq + R].to(F), kw.to(F), 1e-5)[0]
        full = torch.zeros(pos[t] + 1, Dr, dtype=F)
        full[pos[t]] = proj[t, Rq + R : Rq + R + Dr].to(F)
        kr = pr.rotate_pairs(full, rot, 300.0)[pos[t]] if rot else full[pos[t]]
        row = pages[bt[seq[t], pos[t] // page_tokens], 0, pos[t] % page_tokens].float().cpu()
        close(row[:R], c, tol, f"latent of token {t}")
        close(row[R : R + Dr], kr, tol, f"key part of token {t}")
        assert float(row[R + Dr :].abs().max() if Rp > R + Dr else 0.0) == 0.0
    written = {(int(bt[seq[t], pos[t] // page_tokens]), pos[t] % page_tokens) for t in range(T)}
    for p in range(n_pages):
        for o in range(page_tokens):
            if (p, o) not in written:
                assert float((pages[p, 0, o].float() - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,D,Dr,rot,R", [(1, 3, 16, 8, 8, 40), (37, 5, 8, 4, 2, 22), (130, 8, 64, 32, 32, 128),
                                            (70, 2, 20, 6, 6, 18), (9, 4, 24, 0, 0, 17), (5, 6, 16, 16, 8, 24), (3, 2, 8, 8, 0, 16)])
def test_the_querys_side_scores_like_keys_per_head(ops, dtype, T, H, D, Dr, rot, R):
    """``[Wuk^T q | turned q_rot] . [c | k_rot]`` equals ``q . (Wuk c) + turned q_rot . k_rot``; the
    padding of a head's slot is zero whatever the buffer held."""
    q = rnd(T, H * (D + Dr), seed=T).to(dtype)
    uk = rnd(H * D, R, seed=2, scale=0.3).to(dtype)
    uk_t = uk.view(H, D, R).transpose(1, 2).contiguous()
    Rp = R + Dr + (-(R + Dr)) % 16
    positions = torch.arange(3, 3 + T)
    cos, sin = tables(rot, 50.0, T + 3) if rot else (None, None)
    for kind in ([0] if dtype == torch.float32 else [0, 1, 2]):
        out = ops.head_linear(q.cuda(), 0, uk_t.cuda(), out_dtype=dtype, kind=kind, a_head_cols=D + Dr, out_head_cols=Rp)
        assert out.shape == (T, H * Rp)
        out.view(T, H, Rp)[:, :, R:] = 5.0
        ops.latent_query_rope(q.cuda(), out, num_heads=H, head_dim=D, rot_dim=Dr, rot=rot, cos=cos, sin=sin,
                              positions=i32(positions), rank=R)
        got = out.view(T, H, Rp).float().cpu()
        qq = q.to(F).view(T, H, D + Dr)
        ref_lat = torch.einsum("thd,hdr->thr", qq[..., :D], uk.to(F).view(H, D, R))
        full = torch.zeros(T + 3, H, Dr, dtype=F)
        full[3:] = qq[..., D:]
        ref_rot = pr.rotate_pairs(full, rot, 50.0)[3:] if rot else full[3:]
        tol = 3e-6 if dtype == torch.float32 else 1e-2
        close(got[..., :R], ref_lat, tol, f"kernel {kind}: latent side")
        if Dr:
            close(got[..., R : R + Dr], ref_rot, tol, f"kernel {kind}: rotated dims")
        if Rp > R + Dr:
            assert float(got[..., R + Dr :].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,N,group,col0,extra", [(1, 16, 1, 0, 0), (33, 24, 8, 5, 3), (200, 96, 32, 40, 0), (7, 30, 30, 2, 9),
                                                  (5, 20, 3, 1, 2), (3, 9, 2, 0, 0)])
def test_sigmoid_gate(ops, dtype, gdtype, T, N, group, col0, extra):
    if dtype == torch.float32 and gdtype == torch.bfloat16:
        pytest.skip("a float32 step keeps its gate in float32")
    o = rnd(T, N, seed=1).to(dtype)
    g = rnd(T, col0 + -(-N // group) + extra, seed=2, scale=3.0).to(gdtype)
    got = ops.sigmoid_gate_mul(o.clone().cuda(), g.cuda(), col0, group)
    cols = col0 + torch.arange(N) // group
    close(got, o.to(F) * torch.sigmoid(g.to(F)[:, cols]), 2e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("H", [70, 96, 131, 2052, 4100])
@pytest.mark.parametrize("emit", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sums", [False, True])
def test_a_branchs_norm_the_sum_and_the_next_norm_in_one_launch(ops, H, emit, sums):
    """x += w1 * b / rms(b); h = w2 * x / rms(x): x against the plain sum, h against the plain
    norm of it. ``sums``: the branch is a few-rows product that still lies as sums."""
    T, e1, e2 = 6, 1e-5, 3e-6
    x, w1, w2 = rnd(T, H, seed=1), 1 + rnd(H, seed=4, scale=0.4), 1 + rnd(H, seed=5, scale=0.4)
    if sums:
        a, m = rnd(T, 64, seed=6).to(torch.bfloat16), rnd(H, 64, seed=7, scale=0.3).to(torch.bfloat16)
        branch = ops.linear(a.cuda(), m.cuda(), None, out_dtype=torch.float32, may_defer=True)
        b = a.to(F) @ m.to(F).T
        if H <= 2048:
            assert hasattr(branch, "resolve"), "the product was expected to stay as sums"
    else:
        b = rnd(T, H, seed=2, scale=5.0).to(F)
        branch = b.float().cuda()
    ref_x = x.to(F) + pr.unit_rms(b, e1) * w1.to(F)
    ref_h = pr.unit_rms(ref_x, e2) * w2.to(F)
    gx = x.clone().cuda()
    h = ops.rmsnorm_add(gx, branch, w1.cuda(), e1, out_dtype=emit, then_weight=w2.cuda(), then_eps=e2)
    assert h.dtype == emit
    close(gx, ref_x, 3e-6 if not sums else 2e-5, "x")
    close(h, ref_h, (3e-6 if not sums else 2e-5) if emit == torch.float32 else 5e-3, "the next norm")
    gx2 = x.clone().cuda()  # the unfused pair gives the same x
    ops.rmsnorm_add(gx2, b.float().cuda(), w1.cuda(), e1)
    close(gx2, ref_x, 3e-6 if not sums else 2e-5, "x, unfused")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_plain_activations(ops, dtype):
    for shape in ((11, 52), (7, 9)):  # whole 16-byte vectors, and not
        z = rnd(*shape, seed=1, scale=2.0)
        refs = {"relu2": torch.relu(z.to(F)) ** 2, "relu": torch.relu(z.to(F)), "gelu_tanh": pr.gelu_tanh(z.to(F)),
                "silu": z.to(F) * torch.sigmoid(z.to(F))}
        for name, ref in refs.items():
            close(ops.activation(z.cuda(), name, dtype), ref, 2e-6 if dtype == torch.float32 else 5e-3, name)
    if dtype == torch.bfloat16:  # few rows: the activation takes the product's sums and meets them unrounded
        h, w = rnd(5, 64, seed=2).to(dtype), rnd(40, 64, seed=3, scale=0.3).to(dtype)
        got = ops.activated_linear(h.cuda(), w.cuda(), "relu2", dtype)
        close(got, torch.relu(h.to(F) @ w.to(F).T) ** 2, 5e-3)
        again = ops.activated_linear(h.cuda(), w.cuda(), "relu2", dtype)  # the sums were left zero
        assert torch.equal(got, again)


# ----------------------------------------------------------------------------- attention: kept first keys, edges, far keys
def attention_case(ops, dtype, H, G, D, page_tokens, ctx, n_rows, window, keep, scale, seed, sharp_key=None, splits=0,
                   latent=False):
    """One sequence of ``ctx`` keys in shuffled pages; the last ``n_rows`` are this step's queries
    (one row: the single-token kernel, cut into ``splits`` partitions if given). With ``sharp_key``
    the last query of every head is made to single out that key, whose value row carries a large
    planted number: the output shows it if and only if the key is read. ``latent``: one row per
    token that is key and value alike."""
    k = rnd(ctx, G, D, seed=seed)
    v = k if latent else rnd(ctx, G, D, seed=seed + 2)
    q = rnd(n_rows, H, D, seed=seed + 1)
    if sharp_key is not None:
        k[sharp_key] = 0
        k[sharp_key, :, 0] = 50.0
        v[sharp_key, :, 1] = 1000.0
        q[-1] = 0
        q[-1, :, 0] = 40.0 / (50.0 * scale)  # score 40 against scores near 0
    pages_needed = -(-ctx // page_tokens)
    order = torch.randperm(pages_needed + 3, generator=torch.Generator().manual_seed(seed))[:pages_needed]
    kp = torch.full((pages_needed + 4, G, page_tokens, D), float("nan"), dtype=dtype)
    vp = kp.clone()
    for j in range(ctx):
        kp[order[j // page_tokens], :, j % page_tokens] = k[j].to(dtype)
        vp[order[j // page_tokens], :, j % page_tokens] = v[j].to(dtype)
    st = batch([n_rows], [ctx - n_rows], [0])
    st.decode_splits = splits
    plan = {name: torch.tensor(a).cuda() for name, a in ops.attention_plan(st.host, dtype, D).items()}
    kp = kp.cuda()
    got = ops.paged_attention(
        q.reshape(n_rows, H * D).to(dtype).cuda(), num_heads=H, num_kv_heads=G, head_dim=D, scale=scale,
        window=window, k_pages=kp, v_pages=kp if latent else vp.cuda(), block_tables=i32(order[None].tolist()),
        page_tokens=page_tokens, step=st, plan=plan, keep_first=keep)
    kk, vv, qq = k.to(dtype).to(F), v.to(dtype).to(F), q.to(dtype).to(F)
    seen = pr.visible(ctx, window, keep)[ctx - n_rows :]
    ref = torch.zeros(n_rows, H, D, dtype=F)
    for h in range(H):
        g = h // (H // G)
        ref[:, h] = pr.masked_softmax(qq[:, h] @ kk[:, g].T * scale, seen) @ vv[:, g]
    return got.float().view(n_rows, H, D), ref


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,page_tokens,window,keep", [(4, 1, 48, 16, 90, 7), (6, 3, 32, 8, 5, 9), (8, 2, 64, 32, 100, 4),
                                                           (2, 2, 16, 16, 40, 0), (3, 1, 160, 16, 33, 70), (5, 5, 128, 16, 64, 1)])
@pytest.mark.parametrize("n_rows,splits", [(150, 0), (2, 0), (1, 1), (1, 3)])
def test_a_window_that_keeps_the_first_keys(ops, dtype, H, G, D, page_tokens, window, keep, n_rows, splits):
    ops.check_attention_shape(D, dtype, H, G)
    got, ref = attention_case(ops, dtype, H, G, D, page_tokens, ctx=300, n_rows=n_rows, window=window, keep=keep,
                              scale=1.5 / D ** 0.5, seed=H + D, splits=splits)
    close(got, ref, 2e-5 if dtype == torch.float32 else 2e-2)


EDGES = {"last kept": 6, "first not kept": 7, "just outside the window": 437 - 101, "just inside the window": 437 - 100,
         "far inside": 437 - 50, "the very first": 0}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_rows,splits", [(40, 0), (2, 0), (1, 1), (1, 4)])
@pytest.mark.parametrize("edge", list(EDGES))
def test_a_key_at_an_edge(ops, dtype, n_rows, splits, edge):
    """The last query's window of 100 reaches back to key ctx - 100, in the middle of a page; seven
    first keys are kept, which end in the middle of the first page."""
    ctx = 437
    ops.check_attention_shape(80, dtype, 6, 2)
    got, ref = attention_case(ops, dtype, 6, 2, 80, 16, ctx=ctx, n_rows=n_rows, window=100, keep=7, scale=0.1, seed=7,
                              sharp_key=EDGES[edge], splits=splits)
    close(got, ref, 3e-5 if dtype == torch.float32 else 2e-2)
    seen = ref[-1].abs().max() > 500  # the planted value is 1000
    assert bool(seen) == (edge not in ("first not kept", "just outside the window"))
    assert bool(got[-1].abs().max() > 500) == bool(seen)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_rows,splits", [(70, 0), (1, 1), (1, 5)])
@pytest.mark.parametrize("Rp", [48, 80, 160])
def test_a_far_key_among_hundreds_without_a_window(ops, dtype, n_rows, splits, Rp):
    """Latent rows that are keys and values alike, every earlier token visible: key 3 of 900."""
    ops.check_attention_shape(Rp, dtype, 4, 1)
    got, ref = attention_case(ops, dtype, 4, 1, Rp, 16, ctx=900, n_rows=n_rows, window=0, keep=0, scale=0.1, seed=11,
                              sharp_key=3, splits=splits, latent=True)
    close(got, ref, 3e-5 if dtype == torch.float32 else 2e-2)
    assert float(got[-1].abs().max()) > 500


# ----------------------------------------------------------------------------- routed experts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,E,top,ff,shared", [(1, 70, 4, 4, 10, True), (37, 96, 5, 2, 24, False),
                                                 (150, 128, 16, 3, 48, True), (9, 64, 40, 1, 33, True),
                                                 (300, 32, 3, 1, 8, False), (700, 192, 6, 2, 136, True)])
def test_routed_experts_against_the_plain_sum(ops, dtype, T, W, E, top, ff, shared):
    """Biased router, softmax over the chosen logits, ungated experts with the square of relu, the
    weight on the expert's output, a shared expert added as it is: against the plain function."""
    h = rnd(T, W, seed=T).to(dtype)
    w = {"router": rnd(E, W, seed=1, scale=0.3), "router.b": rnd(E, seed=6)}
    for e in range(E):
        w[f"e{e}.up"] = rnd(ff, W, seed=10 + e, scale=0.2).to(dtype)
        w[f"e{e}.down"] = rnd(W, ff, seed=100 + e, scale=0.2).to(dtype)
    up = torch.stack([w[f"e{e}.up"] for e in range(E)])
    down = torch.stack([w[f"e{e}.down"] for e in range(E)])
    shared_out = rnd(T, W, seed=4) if shared else None
    ref_idx, ref_w = pr.route(h.to(F), w, "", top)
    mlp = {"router": {"experts": E, "top": top}}
    ref = pr.moe(h.to(F), w, "", mlp) + (shared_out.to(F) if shared else 0.0)
    idx, wts, gate = ops.moe_route(h.cuda(), w["router"].cuda(), E, top, False, bias=w["router.b"].cuda(),
                                   weights="softmax_of_chosen")
    assert gate is None and torch.equal(idx.cpu().long(), ref_idx)
    close(wts, ref_w, 2e-6)
    close(wts.sum(-1), torch.ones(T, dtype=F), 1e-6)
    kinds = [None, 0] if dtype == torch.float32 else [None, 0, 1, 2] + ([3] if W % 8 == 0 and ff % 8 == 0 else [])
    for kind in kinds:  # every kernel of the experts' products gives the same sum
        plan = ops.moe_sort(idx, E, dtype, width=8 if W % 8 == 0 and ff % 8 == 0 else 1, kind=kind)
        u = ops.expert_linear(h.cuda(), up.cuda(), plan, top=top, wts=None)
        a = ops.activation(u, "relu2", dtype)
        y = ops.expert_linear(a, down.cuda(), plan)
        got = ops.moe_combine(y, plan, top, None if not shared else shared_out.cuda(), None, None, wts=wts)
        close(got, ref, 2e-5 if dtype == torch.float32 else 2e-2, f"kernel {kind}")
    ops.check_kernel_errors()


def test_router_ties_and_the_two_kinds_of_weights(ops):
    h = torch.zeros(3, 16)
    h[1, 0] = 1.0
    router = torch.zeros(6, 16)
    router[4, 0] = 2.0
    bias = torch.tensor([0.0, 0.0, 1.0, 0.0, 0.0, 0.0])
    idx, wts, _ = ops.moe_route(h.cuda(), router.cuda(), 6, 3, False, bias=bias.cuda(), weights="softmax_of_chosen")
    assert idx.cpu().tolist() == [[2, 0, 1], [4, 2, 0], [2, 0, 1]]
    e = torch.tensor([1.0, 0.0, 0.0]).exp()
    close(wts[0], e / e.sum(), 1e-6)
    e = torch.tensor([2.0, 1.0, 0.0]).exp()
    close(wts[1], e / e.sum(), 1e-6)
    idx, wts, _ = ops.moe_route(h.cuda(), router.cuda(), 6, 3, False, bias=bias.cuda())  # sigmoid of each
    assert idx.cpu().tolist() == [[2, 0, 1], [4, 2, 0], [2, 0, 1]]
    close(wts[0], torch.sigmoid(torch.tensor([1.0, 0.0, 0.0])), 1e-6)
    idx, wts, _ = ops.moe_route(h.cuda(), router.cuda(), 6, 1, False, weights="softmax_of_chosen")  # one expert: weight 1
    assert wts.cpu().flatten().tolist() == [1.0, 1.0, 1.0] and idx.cpu().flatten().tolist() == [0, 4, 0]


# ----------------------------------------------------------------------------- the model
def gpu_runner(folder, name, num_pages, dtype, max_num_seqs=4, max_len=512):
    from llmserve_b200.engine.runner import ModelRunner, load_model
    from llmserve_b200.ops import get_ops

    _, _, model = load_model(folder, dtype, "cuda", get_ops("cuda"), max_len)
    return ModelRunner(model, page_tokens=RIROVIK_TINY[name]["page_tokens"], num_pages=num_pages,
                       max_model_len=max_len, max_num_seqs=max_num_seqs, max_num_batched_tokens=max_len)


LENGTHS = {"R1": [5, 70, 1, 33, 49, 126, 2], "R2": [2, 40, 9, 64, 17, 100], "R3": [3, 150, 18, 77, 230]}
TOL = {"float32": (2e-4, 5e-5), "bfloat16": (0.0, 0.03)}  # (absolute, relative to the largest logit)


@pytest.fixture(scope="module")
def expected(rirovik_dirs):
    out = {}
    for name in RIROVIK_TINY:
        reqs = traces.make_requests(LENGTHS[name], RIROVIK_TINY[name]["config"]["vocab"], seed=5)
        out[name] = (reqs, {r: pr.model_logits(rirovik_dirs[name], t) for r, t in reqs.items()})
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["R1", "R2", "R3"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_plain(rirovik_dirs, expected, name, mode, dtype):
    reqs, exp = expected[name]
    pool_tokens = traces.tokens_needed(reqs)
    runner = gpu_runner(rirovik_dirs[name], name, pool_tokens // RIROVIK_TINY[name]["page_tokens"], dtype)
    got = traces.replay(runner, getattr(traces, mode)(reqs))
    atol, rtol = TOL[dtype]
    traces.compare(got, exp, atol=atol, rtol=rtol)
    assert runner.manager.usage() == 0.0
    runner.check_kernels()


@pytest.mark.parametrize("name", ["R1", "R2"])
def test_layers_one_by_one_in_float32(rirovik_dirs, name):
    """The residual stream after every layer against the plain model's."""
    folder = rirovik_dirs[name]
    tokens = traces.make_requests([60], RIROVIK_TINY[name]["config"]["vocab"], seed=2)["r0"]
    cfg, w = pr.load(folder)
    _, after = pr.forward(tokens, w, cfg, return_layers=True)
    runner = gpu_runner(folder, name, 16, "float32")
    model, seen = runner.model, []
    for block in model.blocks:
        inner = block.forward

        def spy(x, pending, step, cache, inner=inner):
            x, pending = inner(x, pending, step, cache)
            if pending is not None:  # the layer's last sum, left for the next norm: formed now
                assert pending.resolve() is None
            seen.append(x.clone())
            return x, None

        block.forward = spy
    from llmserve_b200.engine.batch import StepEntry

    runner.run([StepEntry("a", tokens, [0])])
    assert len(seen) == len(cfg["layers"])
    for i, x in enumerate(seen):
        close(x, after[i], 2e-5, f"after layer {i}")


def test_float32_logits_do_not_depend_on_the_cut(rirovik_dirs, expected):
    """Every kernel of the float32 path computes a row from that row's sequence alone and in a
    fixed order (attention's context partitions and tiles aside), so the mixed schedule gives the
    whole prompts' logits to the last bits."""
    reqs, _ = expected["R1"]
    pool = traces.tokens_needed(reqs) // 16
    a = traces.replay(gpu_runner(rirovik_dirs["R1"], "R1", pool, "float32"), traces.whole(reqs))
    b = traces.replay(gpu_runner(rirovik_dirs["R1"], "R1", pool, "float32"), traces.mixed(reqs, seed=4))
    scale = max(v.abs().max().item() for v in a.values())
    assert max((a[k] - b[k]).abs().max().item() for k in a) <= 4e-6 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(rirovik_dirs, dtype):
    """300 tokens one by one from position 0: every window passes over decoded tokens, pages that a
    window has left are given back while the request lives, and the kept first tokens stay."""
    reqs = traces.make_requests([300], 130, seed=21)
    exp = {r: pr.model_logits(rirovik_dirs["R2"], t) for r, t in reqs.items()}
    runner = gpu_runner(rirovik_dirs["R2"], "R2", 38, dtype)  # 304 tokens of room: the causal layer needs them
    got = traces.replay(runner, traces.decode_tail(reqs, tail=300))
    atol, rtol = TOL[dtype]
    traces.compare(got, exp, atol=atol, rtol=rtol)
    windowed = [g for g, spec in enumerate(runner.manager.groups) if spec.window > 0]
    assert windowed and runner.manager.usage() == 0.0


def test_slots_and_pages_used_again(rirovik_dirs):
    """One state slot and just enough pages: every request runs on what the one before it left."""
    reqs = traces.make_requests([40, 37, 64, 3], 211, seed=8)
    exp = {r: pr.model_logits(rirovik_dirs["R1"], t) for r, t in reqs.items()}
    runner = gpu_runner(rirovik_dirs["R1"], "R1", 4, "float32", max_num_seqs=1)
    traces.compare(traces.replay(runner, traces.portions(reqs)), exp, atol=2e-4, rtol=2e-5)


# ----------------------------------------------------------------------------- generation
PROMPTS = [[5, 9, 100, 31, 7], list(range(40, 57)), [3] * 33, [100, 2], list(range(70))]


def llm(folder, name, dtype, **kw):
    from llmserve_b200 import LLM

    d = dict(dtype=dtype, block_size=RIROVIK_TINY[name]["page_tokens"], num_kv_blocks=64, max_model_len=256,
             max_num_seqs=8)
    d.update(kw)
    return LLM(str(folder), **d)


def greedy(n):
    from llmserve_b200 import SamplingParams

    return SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)


@pytest.mark.parametrize("name", ["R1", "R2"])
@pytest.mark.parametrize("kw", [dict(cuda_graphs=False), dict(cuda_graphs=True),
                                dict(cuda_graphs=True, max_num_batched_tokens=24),
                                dict(cuda_graphs=True, num_kv_blocks=14, max_num_batched_tokens=16)])
def test_greedy_float32_equals_plain_greedy(rirovik_dirs, name, kw):
    """Through the entry point: the scheduler's batches, captured steps (single tokens and padded
    steps with portions), preemption by recomputation."""
    m = llm(rirovik_dirs[name], name, "float32", **kw)
    outs = m.generate(PROMPTS, greedy(12))
    for o, p in zip(outs, PROMPTS):
        assert o.outputs[0].token_ids == pr.greedy(rirovik_dirs[name], p, 12), (kw, p)


def test_greedy_bfloat16_picks_tokens_the_plain_model_also_ranks_first(rirovik_dirs):
    outs = llm(rirovik_dirs["R1"], "R1", "bfloat16", cuda_graphs=True).generate(PROMPTS, greedy(10))
    for o, p in zip(outs, PROMPTS):
        gen = o.outputs[0].token_ids
        logits = pr.model_logits(rirovik_dirs["R1"], p + gen)[len(p) - 1 : -1]
        for t, row in zip(gen, logits):
            assert float(row.max() - row[t]) <= 0.03 * float(row.abs().max())
