"""The Rirovik architecture written out plainly in float64, one function per mechanism.

A slow oracle for the tests: whole sequences only, no cache, no batching, no kernels; it shares no
code with the engine. Weights come as a dict of tensors under the checkpoint's names and the
configuration as the plain dict of ``config.json``.

Notation: ``x`` is the residual stream ``[n, width]`` of one sequence whose tokens sit at
positions 0 .. n-1; ``h`` is a sublayer's normed input.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """The layers' norm: the stored weight lies around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    """The latents' norm: an ordinary weight."""
    return unit_rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(v, dims, base):
    """v [n, ..., d]: of the first ``dims`` entries, neighbours (2i, 2i+1) turn by the angle
    ``p * base^(-2i/dims)`` at position p; the rest pass."""
    n = v.shape[0]
    i = torch.arange(dims // 2, dtype=F64)
    ang = torch.arange(n, dtype=F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    shape = (n,) + (1,) * (v.dim() - 2) + (dims // 2,)
    cos, sin = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def visible(n, size=0, keep_first=0):
    """[n, n] bool: query i sees key j if j <= i and (no window, or i - j < size, or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if size > 0:
        seen = seen & ((i - j < size) | (j < keep_first))
    return seen


def masked_softmax(scores, seen):
    return torch.softmax(scores.masked_fill(~seen, -math.inf), dim=-1)


def latent_rows(h, w, prefix, m, eps):
    """What a latent layer with a down-projection of its own caches per token: the normed latent
    ``c [n, kv_rank]`` and the rotated key part ``[n, rot_dim]`` that all heads share."""
    d = h @ w[prefix + "dkv"].to(F64).T
    R = m["kv_rank"]
    c = plain_norm(d[:, :R], w[prefix + "dkv.norm"].to(F64), eps)
    kr = rotate_pairs(d[:, R:], m["rot"]["dims"], m["rot"]["base"])
    return c, kr


def latent_attention(h, c, kr, w, prefix, m, eps, gated):
    """h [n, width]; c, kr: the cached rows this layer reads (its own or another layer's)."""
    n = h.shape[0]
    H, D, Dr, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    mask = m.get("mask") or {}
    cq = plain_norm(h @ w[prefix + "dq"].to(F64).T, w[prefix + "dq.norm"].to(F64), eps)
    q = (cq @ w[prefix + "uq"].to(F64).T).view(n, H, D + Dr)
    qn = q[..., :D]
    qr = rotate_pairs(q[..., D:], m["rot"]["dims"], m["rot"]["base"])
    k = (c @ w[prefix + "uk"].to(F64).T).view(n, H, D)
    v = (c @ w[prefix + "uv"].to(F64).T).view(n, H, V)
    seen = visible(n, int(mask.get("size", 0) or 0), 0)
    out = torch.zeros(n, H, V, dtype=F64)
    for hd in range(H):
        s = (qn[:, hd] @ k[:, hd].T + qr[:, hd] @ kr.T) * m["scale"]
        out[:, hd] = masked_softmax(s, seen) @ v[:, hd]
    if gated:
        out = out * torch.sigmoid(h @ w[prefix + "g"].to(F64).T)[:, :, None]
    return out.reshape(n, H * V) @ w[prefix + "o"].to(F64).T


def grouped_attention(h, w, prefix, m, eps):
    """Query heads in groups on fewer key/value heads; biases; q and k divided by their root mean
    square; no positions; a window that also keeps the sequence's first tokens; an output gate
    per element."""
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    mask = m.get("mask") or {}

    def lin(name):
        return h @ w[prefix + name].to(F64).T + w[prefix + name + ".b"].to(F64)

    q = unit_rms(lin("q").view(n, H, D), eps)
    k = unit_rms(lin("k").view(n, G, D), eps)
    v = lin("v").view(n, G, V)
    seen = visible(n, int(mask.get("size", 0) or 0), int(mask.get("keep_first", 0) or 0))
    out = torch.zeros(n, H, V, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        out[:, hd] = masked_softmax(s, seen) @ v[:, g]
    out = out.reshape(n, H * V) * torch.sigmoid(h @ w[prefix + "g"].to(F64).T)
    return out @ w[prefix + "o"].to(F64).T


def expert(h, w, prefix):
    z = torch.relu(h @ w[prefix + "up"].to(F64).T)
    return (z * z) @ w[prefix + "down"].to(F64).T


def route(h, w, prefix, top):
    """Indices [n, top] of the largest router logits and the softmax over those logits alone."""
    z = h @ w[prefix + "router"].to(F64).T + w[prefix + "router.b"].to(F64)
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe(h, w, prefix, mlp):
    idx, wt = route(h, w, prefix, mlp["router"]["top"])
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(idx[t].tolist(), wt[t]):
            y[t] += p * expert(h[t : t + 1], w, f"{prefix}e{e}.")[0]
    if mlp.get("shared"):
        y = y + expert(h, w, prefix + "shared.")
    return y


def embed(tokens, w, cfg):
    return w["embed"].to(F64)[list(tokens)] * cfg["embedding"]["scale"]


def forward(tokens, w, cfg, return_layers=False):
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w, cfg)
    cached = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        h = offset_norm(x, w[p + "norm1"].to(F64), eps)
        if kind == "attention":
            a = grouped_attention(h, w, p + "mix.", m, eps)
        elif kind in ("latent_attention", "latent_attention_2"):
            src = m.get("kv_from")
            if src is None:
                cached[i] = latent_rows(h, w, p + "mix.", m, eps)
                src = i
            c, kr = cached[src]
            a = latent_attention(h, c, kr, w, p + "mix.", m, eps, gated=kind == "latent_attention")
        else:
            raise ValueError(kind)
        x = x + offset_norm(a, w[p + "norm1b"].to(F64), eps)
        if layer.get("mlp"):
            h = offset_norm(x, w[p + "norm2"].to(F64), eps)
            x = x + offset_norm(moe(h, w, p + "mlp.", layer["mlp"]), w[p + "norm2b"].to(F64), eps)
        after.append(x.clone())
    logits = offset_norm(x, w["final.norm"].to(F64), eps) @ w["head"].to(F64).T
    return (logits, after) if return_layers else logits


_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}


def read_safetensors(path):
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = bytearray(raw[8 + n + lo : 8 + n + hi])
        out[name] = torch.frombuffer(buf, dtype=_DTYPES[info["dtype"]]).reshape(info["shape"]).clone()
    return out


def load(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


def model_logits(folder, tokens):
    cfg, w = load(folder)
    return forward(tokens, w, cfg)


def greedy(folder, prompt, n):
    cfg, w = load(folder)
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(seq, w, cfg)[-1].argmax()))
    return seq[len(prompt):]
