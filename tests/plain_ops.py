"""Plain PyTorch versions of the engine's kernels, one function per kernel, float32 arithmetic.

Two uses, both in tests only: each CUDA kernel is compared with its function here, and the
engine's host-side logic (runner, cache, scheduler) is exercised on the CPU with this object in
place of the CUDA kernel set. The product path never imports this file.
"""

from __future__ import annotations

import numpy as np
import torch


def philox4x32_10(c, k0, k1):
    """Philox4x32-10 on numpy uint32 arrays c[4]; returns 4 arrays."""
    c = [np.asarray(x, dtype=np.uint64) for x in c]
    k0 = np.uint64(k0)
    k1 = np.uint64(k1)
    m0, m1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = m0 * c[0]
        p1 = m1 * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = [(hi1 ^ c[1] ^ k0) & mask, lo1, (hi0 ^ c[3] ^ k1) & mask, lo0]
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return c


class PlainOps:
    name = "plain-torch"

    def __init__(self, q_tile: int = 32) -> None:
        self.q_tile = q_tile
        self.launches = 0
        self.accumulate = True  # add into the residual stream where a part offers it

    # ------------------------------------------------------------------ capabilities
    def branch_dtype(self, dtype):
        return torch.float32

    def check_attention_shape(self, head_dim, dtype, num_heads=None, num_kv_heads=None):
        if head_dim % 16:
            raise ValueError("head size must be a multiple of 16")

    # ------------------------------------------------------------------ pointwise
    def embedding(self, token_ids, table):
        return table[token_ids.long()].float()

    def add_rmsnorm(self, x, residual, weight, eps, out_dtype, rows=None):
        if rows is not None:
            v = x[rows.long()]
            if residual is not None:
                v = v + residual[rows.long()].float()
        else:
            if residual is not None:
                x += residual.float()
            v = x
        y = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight
        return y.to(out_dtype)

    def silu_mul(self, gu, out_dtype=None, activation="silu"):
        g, u = gu.float().chunk(2, dim=-1)
        if activation == "gelu_tanh":
            act = 0.5 * g * (1 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
        else:
            act = g / (1 + torch.exp(-g))
        return (act * u).to(out_dtype or gu.dtype)

    def linear(self, a, w, bias=None, out_dtype=None, accumulate_into=None):
        y = a.float() @ w.float().T
        if bias is not None:
            y = y + bias.float()
        if accumulate_into is not None and self.accumulate:
            accumulate_into += y
            return None
        return y.to(out_dtype or a.dtype)

    def gated_silu(self, h, w, bias=None, out_dtype=None, activation="silu"):
        return self.silu_mul(self.linear(h, w, bias, out_dtype=torch.float32), out_dtype=out_dtype or h.dtype,
                             activation=activation)

    # ------------------------------------------------------------------ attention
    def project_rope_kv_write(self, h, w, bias, *, out_dtype=None, **kw):
        qkv = self.linear(h, w, bias, out_dtype=torch.float32)
        return self.rope_kv_write(qkv, out_dtype=out_dtype or h.dtype, **kw)

    def project_attend(self, h, w, bias, *, num_heads, num_kv_heads, head_dim, scale, window, positions,
                       token_seq, cos, sin, k_pages, v_pages, writes, block_tables, page_tokens, step,
                       plan, out_dtype=None):
        q = self.project_rope_kv_write(
            h, w, bias, out_dtype=out_dtype, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
            positions=positions, token_seq=token_seq, cos=cos, sin=sin, k_pages=k_pages if writes else None,
            v_pages=v_pages if writes else None, block_tables=block_tables, page_tokens=page_tokens)
        return self.paged_attention(
            q, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, scale=scale, window=window,
            k_pages=k_pages, v_pages=v_pages, block_tables=block_tables, page_tokens=page_tokens, step=step,
            plan=plan)

    def rope_kv_write(self, qkv, *, num_heads, num_kv_heads, head_dim, positions, token_seq,
                      cos, sin, k_pages, v_pages, block_tables, page_tokens, out_dtype=None):
        T, D = qkv.shape[0], head_dim
        out_dtype = out_dtype or qkv.dtype
        heads = qkv.view(T, num_heads + 2 * num_kv_heads, D)
        pos = positions.long()
        rot = heads[:, : num_heads + num_kv_heads].float()
        if cos is not None:
            c, s = cos[pos][:, None, :], sin[pos][:, None, :]
            x1, x2 = rot[..., : D // 2], rot[..., D // 2 :]
            rot = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
        if k_pages is not None:
            page = block_tables[token_seq.long(), pos // page_tokens].long()
            off = pos % page_tokens
            k_pages[page, :, off] = rot[:, num_heads:].to(out_dtype)
            v_pages[page, :, off] = heads[:, num_heads + num_kv_heads :].to(out_dtype)
        if out_dtype == qkv.dtype:
            heads[:, :num_heads] = rot[:, :num_heads].to(qkv.dtype)
            return qkv[:, : num_heads * D]
        return rot[:, :num_heads].to(out_dtype).reshape(T, num_heads * D)

    def attention_q_tile(self, dtype, head_dim):
        return self.q_tile

    def attention_plan(self, host_step, dtype, head_dim):
        tiles, decode = [], []
        for s, n in enumerate(host_step.q_lens.tolist()):
            if n == 1:
                decode.append(s)
            else:
                tiles.extend((s, q0) for q0 in range(0, n, self.q_tile))
        return {
            "tiles": np.asarray(tiles, dtype=np.int32).reshape(-1, 2),
            "decode_seqs": np.asarray(decode, dtype=np.int32),
        }

    def paged_attention(self, q, *, num_heads, num_kv_heads, head_dim, scale, window, k_pages,
                        v_pages, block_tables, page_tokens, step, plan=None, head_scale=None,
                        slopes=None, chunk=0, sinks=None, keep_first=0, out_dtype=None):
        T, D = q.shape[0], head_dim
        qkv = q
        q = q[:, : num_heads * D].float().reshape(T, num_heads, D)
        out = torch.zeros(T, num_heads, D)
        cu = step.cu_q.tolist()
        ctx = step.ctx_lens.tolist()
        group = num_heads // num_kv_heads
        for s in range(len(ctx)):
            a, b = cu[s], cu[s + 1]
            n = b - a
            j = torch.arange(ctx[s])
            pages = block_tables[s, j // page_tokens].long()
            k = k_pages[pages, :, j % page_tokens].float().repeat_interleave(group, dim=1)
            v = v_pages[pages, :, j % page_tokens].float().repeat_interleave(group, dim=1)
            qpos = torch.arange(ctx[s] - n, ctx[s])[:, None]
            visible = j[None, :] <= qpos
            if window > 0:
                visible &= ((qpos - j[None, :]) < window) | (j[None, :] < keep_first)
            if chunk > 0:
                visible &= (qpos // chunk) == (j[None, :] // chunk)
            sc = torch.einsum("thd,shd->hts", q[a:b], k) * scale
            if head_scale is not None:
                sc = sc * head_scale.float()[:, None, None]
            if slopes is not None:
                sc = sc - slopes.float()[:, None, None] * (qpos - j[None, :]).float()[None]
            sc = sc.masked_fill(~visible, float("-inf"))
            if sinks is not None:  # a column without a value
                sc = torch.cat([sc, sinks.float()[:, None, None].expand(-1, n, 1)], -1)
                v = torch.cat([v, torch.zeros_like(v[:1])], 0)
            out[a:b] = torch.einsum("hts,shd->thd", sc.softmax(-1), v)
        return out.view(T, num_heads * D).to(out_dtype or qkv.dtype)

    def norm_rope_kv_write(self, qkv, *, num_heads, num_kv_heads, head_dim, values_are_keys, q_weight,
                           k_weight, eps, positions, token_seq, cos, sin, k_pages, v_pages,
                           block_tables, page_tokens, out_dtype, norm_dim=None):
        T, D = qkv.shape[0], head_dim
        nd = norm_dim or head_dim
        nv = 0 if values_are_keys else num_kv_heads
        heads = qkv[:, : (num_heads + num_kv_heads + nv) * D].float().reshape(T, num_heads + num_kv_heads + nv, D)
        q, k = heads[:, :num_heads], heads[:, num_heads : num_heads + num_kv_heads]
        v = k if values_are_keys else heads[:, num_heads + num_kv_heads :]
        if q_weight is not None:
            q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) / nd + eps) * q_weight
            k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) / nd + eps) * k_weight
        pos = positions.long()
        if cos is not None:
            c, s_ = cos[pos][:, None, :], sin[pos][:, None, :]
            rot = lambda x: torch.cat([x[..., : D // 2] * c - x[..., D // 2 :] * s_,
                                       x[..., D // 2 :] * c + x[..., : D // 2] * s_], -1)
            q, k = rot(q), rot(k)
        if k_pages is not None:
            page = block_tables[token_seq.long(), pos // page_tokens].long()
            off = pos % page_tokens
            k_pages[page, :, off] = k.to(k_pages.dtype)
            v_pages[page, :, off] = v.to(v_pages.dtype)
        return q.to(out_dtype).reshape(T, num_heads * D).contiguous()

    # ------------------------------------------------------------------ embedding terms, latent attention
    def hashed_pair_add(self, x, table, state, step, *, buckets, mul_previous, mul_token):
        ids, pos = step.token_ids.tolist(), step.positions.tolist()
        cu, slots = step.cu_q.tolist(), step.state_slots.tolist()
        for s_ in range(len(slots)):
            prev = int(state[slots[s_], 0])
            for t in range(cu[s_], cu[s_ + 1]):
                row = buckets if pos[t] == 0 else (prev * mul_previous + ids[t] * mul_token) % buckets
                x[t] += table[row].float()
                prev = ids[t]
            state[slots[s_], 0] = prev

    def sinusoid_add(self, x, positions, freq):
        ang = positions.float()[:, None] * freq[None, :]
        w = x.shape[1]
        x[:, 0::2] += torch.sin(ang)[:, : (w + 1) // 2]
        x[:, 1::2] += torch.cos(ang)[:, : w // 2]

    def latent_write(self, proj, col0, rank, weight, eps, pages, positions, token_seq, block_tables):
        d = proj[:, col0 : col0 + rank].float()
        c = d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * weight
        pos = positions.long()
        page_tokens = pages.shape[2]
        page = block_tables[token_seq.long(), pos // page_tokens].long()
        pages[page, 0, pos % page_tokens] = 0
        pages[page, 0, pos % page_tokens, :rank] = c.to(pages.dtype)

    def head_linear(self, a, col0, w, out_dtype, a_head_cols=0, out_head_cols=0):
        H, N, K = w.shape
        ah, oh = a_head_cols or K, out_head_cols or N
        x = a[:, col0 : col0 + H * ah].float().reshape(-1, H, ah)[:, :, :K]
        out = torch.zeros(a.shape[0], H, oh)
        out[:, :, :N] = torch.einsum("thk,hnk->thn", x, w.float())
        return out.reshape(-1, H * oh).to(out_dtype)

    @staticmethod
    def _turn_neighbours(x, rot, cos, sin, pos):
        """x [T, ..., d]: the pairs (2i, 2i+1) of the first ``rot`` dims turned by the position's angles."""
        if not rot:
            return x
        shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (rot // 2,)
        c, s_ = cos[pos].reshape(shape), sin[pos].reshape(shape)
        out = x.clone()
        u, v = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2] = u * c - v * s_
        out[..., 1:rot:2] = v * c + u * s_
        return out

    def latent_rope_write(self, proj, *, q_col0=0, q_weight=None, kv_col0=0, kv_weight=None, rot_dim=0,
                          rot=0, eps, cos=None, sin=None, pages=None, positions, token_seq, block_tables,
                          out_dtype):
        pos = positions.long()
        cq = None
        if q_weight is not None:
            d = proj[:, q_col0 : q_col0 + q_weight.numel()].float()
            cq = (d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * q_weight).to(out_dtype)
        if kv_weight is not None:
            R = kv_weight.numel()
            d = proj[:, kv_col0 : kv_col0 + R].float()
            c = d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * kv_weight
            kr = self._turn_neighbours(proj[:, kv_col0 + R : kv_col0 + R + rot_dim].float(), rot, cos, sin, pos)
            page_tokens = pages.shape[2]
            page = block_tables[token_seq.long(), pos // page_tokens].long()
            pages[page, 0, pos % page_tokens] = 0
            pages[page, 0, pos % page_tokens, : R + rot_dim] = torch.cat([c, kr], -1).to(pages.dtype)
        return cq

    def latent_query_rope(self, q, out, *, num_heads, head_dim, rot_dim, rot, cos, sin, positions, rank):
        T = q.shape[0]
        qr = q.float().reshape(T, num_heads, head_dim + rot_dim)[:, :, head_dim:]
        qr = self._turn_neighbours(qr, rot, cos, sin, positions.long())
        slots = out.view(T, num_heads, -1)
        slots[:, :, rank:] = 0
        slots[:, :, rank : rank + rot_dim] = qr.to(out.dtype)
        return out

    def sigmoid_gate_mul(self, o, g, col0, group):
        cols = col0 + torch.arange(o.shape[1]) // group
        o.copy_((o.float() * torch.sigmoid(g.float()[:, cols])).to(o.dtype))
        return o

    def activation(self, z, activation, out_dtype):
        z = z.float()
        if activation == "relu2":
            y = torch.relu(z) ** 2
        elif activation == "relu":
            y = torch.relu(z)
        elif activation == "gelu_tanh":
            y = torch.nn.functional.gelu(z, approximate="tanh")
        else:
            y = torch.nn.functional.silu(z)
        return y.to(out_dtype)

    def activated_linear(self, h, w, activation, out_dtype):
        return self.activation(self.linear(h, w, None, out_dtype=torch.float32), activation, out_dtype)

    # ------------------------------------------------------------------ routed experts
    def moe_route(self, h, router, num_experts, top, has_gate, bias=None, weights="sigmoid"):
        z = h.float() @ router.float().T
        gate = torch.sigmoid(z[:, num_experts]) if has_gate else None
        z = z[:, :num_experts] + (bias.float() if bias is not None else 0.0)
        val, idx = torch.topk(z, top, dim=-1)
        val = torch.sigmoid(val) if weights == "sigmoid" else torch.softmax(val, dim=-1)
        return idx.to(torch.int32), val, gate

    def moe_sort(self, idx, num_experts, dtype, width=0, kind=None):
        return idx  # the plain products below walk the choices as they are

    def expert_linear(self, a, w, plan, top=0, wts=None):
        idx = plan.reshape(-1).long()
        rows = a.float() if top == 0 else a.float().repeat_interleave(top, 0)
        if wts is not None:
            rows = rows * wts.reshape(-1, 1)
        return torch.einsum("rk,rnk->rn", rows, w.float()[idx])

    def moe_combine(self, y, plan, top, shared, gate, residual, wts=None):
        rows = y.view(-1, top, y.shape[1])
        out = (rows * wts[:, :, None]).sum(1) if wts is not None else rows.sum(1)
        if shared is not None:
            out = out + (gate[:, None] * shared.float() if gate is not None else shared.float())
        if residual is not None and self.accumulate:
            residual += out
            return None
        return out

    # ------------------------------------------------------------------ branch-norm blocks, state mixers
    def cast(self, x, dtype):
        return x if x.dtype == dtype else x.to(dtype)

    def token_shift(self, x, mix, state, step, out_dtype):
        cu, ctx, slots = step.cu_q.tolist(), step.ctx_lens.tolist(), step.state_slots.tolist()
        out = torch.empty_like(x)
        for s_ in range(len(ctx)):
            a, b = cu[s_], cu[s_ + 1]
            first = state[slots[s_]].clone() if ctx[s_] - (b - a) > 0 else torch.zeros_like(x[0])
            prev = torch.cat([first[None], x[a : b - 1]], 0)
            out[a:b] = x[a:b] + (prev - x[a:b]) * mix
            state[slots[s_]] = x[b - 1]
        return out.to(out_dtype)

    def mix_normed(self, branches, weights, coefficients, eps):
        y = 0
        for a, w, c in zip(branches, weights, coefficients):
            a = a.float()
            y = y + c * (a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + eps) * w)
        return y

    def rmsnorm_add(self, x, branch, weight, eps, out_dtype=None, then_weight=None, then_eps=0.0):
        y = branch.resolve() if hasattr(branch, "resolve") else branch.float()
        x += y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * weight
        if out_dtype is None:
            return None
        if then_weight is not None:
            return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + then_eps) * then_weight).to(out_dtype)
        return x.to(out_dtype)

    def decay_linear_attention(self, proj, *, num_heads, key_dim, value_dim, decay, state, step,
                               activation, key_scale, cos, sin, decay_logits=None, decay_root=1.0,
                               query_scale=1.0):
        T, H, dk, dv = proj.shape[0], num_heads, key_dim, value_dim
        p = proj.float()
        q = p[:, : H * dk].view(T, H, dk) * query_scale
        k = p[:, H * dk : 2 * H * dk].view(T, H, dk)
        v = p[:, 2 * H * dk : 2 * H * dk + H * dv].view(T, H, dv)
        if activation == "silu":
            q, k, v = (t / (1 + torch.exp(-t)) for t in (q, k, v))
        if cos is not None:
            half = cos.shape[1]
            c, s_ = cos[step.positions.long()][:, None, :], sin[step.positions.long()][:, None, :]
            rot = lambda x: torch.cat([x[..., :half] * c - x[..., half : 2 * half] * s_,
                                       x[..., half : 2 * half] * c + x[..., :half] * s_, x[..., 2 * half :]], -1)
            q, k = rot(q), rot(k)
        k = k * key_scale
        out = torch.empty(T, H, dv)
        cu, ctx, slots = step.cu_q.tolist(), step.ctx_lens.tolist(), step.state_slots.tolist()
        for s_ in range(len(ctx)):
            a, b = cu[s_], cu[s_ + 1]
            S = state[slots[s_]].clone() if ctx[s_] - (b - a) > 0 else torch.zeros_like(state[0])  # [H, dv, dk]
            for t in range(a, b):
                if decay_logits is not None:  # a decay per key channel and token: sigmoid(z)^(1/root)
                    z = decay_logits[t].float().view(H, dk)
                    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / decay_root)
                    S = alpha[:, None, :] * S + v[t][:, :, None] * k[t][:, None, :]
                    out[t] = torch.einsum("hvk,hk->hv", S, q[t])
                    continue
                S = decay[:, None, None] * S + v[t][:, :, None] * k[t][:, None, :]
                out[t] = torch.einsum("hvk,hk->hv", S, q[t])
            state[slots[s_]] = S
        return out.reshape(T, H * dv)

    def gated_group_norm(self, o, proj, *, gate_offset, group, weight, eps, gate_activation, out_dtype):
        T, N = o.shape
        g = proj[:, gate_offset : gate_offset + N].float()
        y = o.view(T, N // group, group)
        y = (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)).reshape(T, N)
        if weight is not None:
            y = y * weight
        gate = g / (1 + torch.exp(-g)) if gate_activation == "silu" else 1 / (1 + torch.exp(-g))
        return (y * gate).to(out_dtype)

    # ------------------------------------------------------------------ residual streams
    def streams_spread(self, x, streams, scale=1.0):
        return (x.float() * scale).repeat(1, streams)

    def streams_read_norm(self, x, read, weight, eps, streams, out_dtype, rows=None):
        T, W = x.shape[0], x.shape[1] // streams
        xs = x.view(T, streams, W)
        if rows is not None:
            xs = xs[rows.long()]
        u = torch.einsum("s,tsw->tw", read.float(), xs)
        return (u * torch.rsqrt(u.pow(2).mean(-1, keepdim=True) + eps) * weight).to(out_dtype)

    def streams_write(self, x, y, scale, mix, out, streams, then_read=None, then_weight=None, then_eps=0.0,
                      out_dtype=None):
        T, W = x.shape[0], x.shape[1] // streams
        y = y.resolve() if hasattr(y, "resolve") else y
        y = y.float() * scale if scale is not None else y.float()
        xs = x.view(T, streams, W)
        xs.copy_(torch.einsum("sr,tsw->trw", mix.float(), xs) + out.float()[None, :, None] * y[:, None, :])
        if then_read is None:
            return None
        return self.streams_read_norm(x, then_read, then_weight, then_eps, streams, out_dtype)

    # ------------------------------------------------------------------ rows of q, k, v prepared a token at a time
    def qkv_norm_rope_write(self, qkv, *, num_heads, num_kv_heads, num_value_heads, head_dim, value_dim, out_dim,
                            q_weight, k_weight, eps, positions, token_seq, cos, sin, k_pages,
                            v_pages, block_tables, page_tokens, out_dtype, temp_coef=0.0, temp_every=0):
        T, D, Dv, Dp = qkv.shape[0], head_dim, value_dim, out_dim
        nq, nk, nv = num_heads, num_kv_heads, num_value_heads
        p = qkv.float()
        q, k = p[:, : nq * D], p[:, nq * D : (nq + nk) * D]
        v = k.reshape(T, nk, D) if nv == 0 else p[:, (nq + nk) * D : (nq + nk) * D + nv * Dv].reshape(T, nv, Dv)
        if q_weight is not None:
            q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight
            k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_weight
        pos = positions.long()
        if temp_every:
            q = q * (1.0 + temp_coef * torch.log(torch.floor((pos.float() + 1.0) / temp_every) + 1.0))[:, None]
        q, k = q.reshape(T, nq, D), k.reshape(T, nk, D)
        if cos is not None:
            half = cos.shape[1]
            c, s_ = cos[pos][:, None, :], sin[pos][:, None, :]
            rot = lambda x: torch.cat([x[..., :half] * c - x[..., half : 2 * half] * s_,
                                       x[..., half : 2 * half] * c + x[..., :half] * s_, x[..., 2 * half :]], -1)
            q, k = rot(q), rot(k)
        if nv:
            v = v.repeat_interleave(nk // nv, dim=1)
        fill = lambda x: torch.nn.functional.pad(x, (0, Dp - x.shape[-1]))
        if k_pages is not None:
            page = block_tables[token_seq.long(), pos // page_tokens].long()
            off = pos % page_tokens
            k_pages[page, :, off] = fill(k).to(k_pages.dtype)
            v_pages[page, :, off] = fill(v).to(v_pages.dtype)
        return fill(q).to(out_dtype).reshape(T, nq * Dp).contiguous()

    def differential_combine(self, a, proj, *, gate_col0, num_heads, group, head_dim, value_dim, lam, eps,
                             out_scale, out_dtype):
        T, H, n = a.shape[0], num_heads, group
        maps = a.float().view(T, H // n, 2, n, head_dim)[..., :value_dim]  # (key group, map, head in group)
        o = (maps[:, :, 0] - lam * maps[:, :, 1]).reshape(T, H, value_dim)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * out_scale
        g = torch.sigmoid(proj[:, gate_col0 : gate_col0 + H].float())
        return (o * g[:, :, None]).reshape(T, H * value_dim).to(out_dtype)

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature, top_k, top_p, min_p, seed, draw, kinds=3):
        R, V = logits.shape
        out = torch.empty(R, dtype=torch.int32)
        for r in range(R):
            t = float(temperature[r])
            row = logits[r].float()
            if t < 1e-5:
                out[r] = int(row.argmax())
                continue
            z = row * np.float32(1.0 / np.float32(t))
            zmax = z.max()
            p = torch.exp(z - zmax)
            keep = torch.ones(V, dtype=torch.bool)
            k, tp, mp = int(top_k[r]), float(top_p[r]), float(min_p[r])
            if (0 < k < V) or tp < 1.0:
                gt = z[None, :] > z[:, None]  # gt[i, j]: z_j above z_i
                count = gt.sum(1)
                mass = (gt * p[None, :]).sum(1)
                if 0 < k < V:
                    keep &= count < k
                keep &= mass < np.float32(tp) * p.sum()
            if mp > 0:
                keep &= z >= zmax + np.log(np.float32(mp))
            sd = int(seed[r]) & 0xFFFFFFFFFFFFFFFF
            quads = np.arange((V + 3) // 4, dtype=np.uint32)
            c = philox4x32_10(
                [quads, np.full_like(quads, int(draw[r])), np.zeros_like(quads), np.zeros_like(quads)],
                sd & 0xFFFFFFFF, sd >> 32,
            )
            bits = np.stack(c, axis=1).reshape(-1)[:V].astype(np.uint32)
            u = ((bits >> 8).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
            score = z - torch.from_numpy(np.log(-np.log(u))).float()
            score[~keep] = float("-inf")
            out[r] = int(score.argmax())
        return out

    def sample_sorted(self, logits, temperature, top_k, top_p, min_p, seed, draw):
        """The same rule as :meth:`sample` with a sort instead of the all-pairs comparison, for
        vocabularies too large for a V x V matrix. An element's strictly-above count and mass are
        those of the first element of its group of equal values in descending order; masses are
        summed in float64."""
        R, V = logits.shape
        out = torch.empty(R, dtype=torch.int32)
        for r in range(R):
            t = float(temperature[r])
            row = logits[r].float()
            if t < 1e-5:
                out[r] = int(row.argmax())
                continue
            z = row * np.float32(1.0 / np.float32(t))
            zmax = z.max()
            p = torch.exp(z - zmax).double()
            keep = torch.ones(V, dtype=torch.bool)
            k, tp, mp = int(top_k[r]), float(top_p[r]), float(min_p[r])
            if (0 < k < V) or tp < 1.0:
                zs, order = torch.sort(z, descending=True, stable=True)
                ps = p[order]
                excl = torch.cumsum(ps, 0) - ps  # mass before each sorted position
                first = torch.ones(V, dtype=torch.bool)
                first[1:] = zs[1:] != zs[:-1]
                start = torch.cummax(torch.where(first, torch.arange(V), torch.zeros(V, dtype=torch.long)), 0).values
                count, mass = start, excl[start]
                ks = torch.ones(V, dtype=torch.bool)
                if 0 < k < V:
                    ks &= count < k
                ks &= mass < float(np.float32(tp)) * float(p.sum())
                keep[order] = ks
            if mp > 0:
                keep &= z >= zmax + np.log(np.float32(mp))
            sd = int(seed[r]) & 0xFFFFFFFFFFFFFFFF
            quads = np.arange((V + 3) // 4, dtype=np.uint32)
            c = philox4x32_10(
                [quads, np.full_like(quads, int(draw[r])), np.zeros_like(quads), np.zeros_like(quads)],
                sd & 0xFFFFFFFF, sd >> 32,
            )
            bits = np.stack(c, axis=1).reshape(-1)[:V].astype(np.uint32)
            u = ((bits >> 8).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
            score = z - torch.from_numpy(np.log(-np.log(u))).float()
            score[~keep] = float("-inf")
            out[r] = int(score.argmax())
        return out

    def logsumexp(self, logits):
        return torch.logsumexp(logits.float(), dim=-1)

    def apply_penalties(self, logits, row, token, count, presence, frequency, repetition):
        for i in range(row.shape[0]):
            r, t = int(row[i]), int(token[i])
            v = float(logits[r, t])
            if int(count[i]) > 0:
                v -= float(frequency[i]) * int(count[i]) + float(presence[i])
            rp = float(repetition[i])
            if rp != 1.0:
                v = v / rp if v > 0 else v * rp
            logits[r, t] = v

    PROMPT_BIT = 1 << 30

    def token_state_add(self, state, slot, token, in_prompt):
        for s_, t, f in zip(slot.tolist(), token.tolist(), in_prompt.tolist()):
            if f:
                state[s_, t] |= self.PROMPT_BIT
            else:
                state[s_, t] += 1

    def apply_penalties_dense(self, logits, row, slot, presence, frequency, repetition, state):
        for j in range(row.shape[0]):
            r, st = int(row[j]), state[int(slot[j])]
            for t in torch.nonzero(st).flatten().tolist():
                v = float(logits[r, t])
                c = int(st[t]) & (self.PROMPT_BIT - 1)
                if c > 0:
                    v -= float(frequency[j]) * c + float(presence[j])
                rp = float(repetition[j])
                if rp != 1.0:
                    v = v / rp if v > 0 else v * rp
                logits[r, t] = v

    def ban_tokens(self, logits, row, token):
        logits[row.long(), token.long()] = float("-inf")
