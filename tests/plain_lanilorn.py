"""The Lanilorn architecture written out plainly in float64, one function per mechanism.

A slow oracle for the tests: whole sequences only, no cache, no batching, no kernels; it shares no
code with the engine. Weights come as a dict of tensors under the checkpoint's names and the
configuration as the plain dict of ``config.json``.

Notation: ``X`` is the residual state ``[n, streams, width]`` of one sequence whose tokens sit at
positions 0 .. n-1; ``h`` is a sublayer's normed input ``[n, width]``.
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


def weighted_norm(x, w, eps):
    return unit_rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------------------- streams
def streams_read(X, w_in):
    """What a sublayer reads of the streams: ``u = sum_s w_in[s] X[:, s]``."""
    return torch.einsum("s,nsw->nw", w_in, X)


def streams_write(X, y, w_mix, w_out):
    """All streams at once from the old ones: ``X'[:, t] = sum_s w_mix[s, t] X[:, s] + w_out[t] y``."""
    return torch.einsum("st,nsw->ntw", w_mix, X) + w_out[None, :, None] * y[:, None, :]


# ------------------------------------------------------------------------------- rotation
def yarn_frequencies(dims, base, scaling):
    """float64 ``[dims/2]`` frequencies and the factor on cos and sin."""
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    if scaling is None:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half_part(v, positions, dims, base, scaling):
    """v ``[n, heads, d]``: of each head's first ``dims`` entries, entry i is paired with entry
    i + dims/2 and the pair turns by ``p * f_i``; both cos and sin carry the factor."""
    f, mag = yarn_frequencies(dims, base, scaling)
    ang = positions.to(F64)[:, None] * f[None, :]
    cos, sin = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    half = dims // 2
    a, b = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


# ------------------------------------------------------------------------------- softmax attention
def attend(q, k, v, scale, seen, sink=None):
    """q ``[n, H, d]``, k ``[n, G, d]``, v ``[n, G, dv]``; ``seen [n, n]`` bool; ``sink [H]`` joins
    each head's denominator as ``exp(sink_h)`` without a key or a value. Returns ``[n, H, dv]``."""
    n, H, _ = q.shape
    G = k.shape[1]
    kk = k.repeat_interleave(H // G, dim=1)
    vv = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    s = s.masked_fill(~seen[None], float("-inf"))
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None, None])
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - top)
    return torch.einsum("hij,jhd->ihd", e / den, vv)


def causal(n, window=0):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if window:
        seen &= (i - j) < window
    return seen


def windowed_attention(h, w, p, m, eps):
    """Queries and keys normed over the whole projection, part of each head rotated, the values
    are the keys as projected, a window, a sink per head, a sigmoid gate per head."""
    n = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = h @ w[p + "q"].to(F64).T
    k = h @ w[p + "k"].to(F64).T
    v = k.view(n, G, d)
    q = weighted_norm(q, w[p + "q.norm"].to(F64), eps).view(n, H, d)
    k = weighted_norm(k, w[p + "k.norm"].to(F64), eps).view(n, G, d)
    rot = m.get("rot")
    if rot:
        pos = torch.arange(n)
        q = rotate_half_part(q, pos, rot["dims"], rot["base"], rot.get("scaling"))
        k = rotate_half_part(k, pos, rot["dims"], rot["base"], rot.get("scaling"))
    window = (m.get("mask") or {}).get("size", 0)
    o = attend(q, k, v, m["scale"], causal(n, window), w[p + "sink"].to(F64))
    g = torch.sigmoid(h @ w[p + "g"].to(F64).T)
    return (o * g[:, :, None]).reshape(n, -1) @ w[p + "o"].to(F64).T


def query_temperature(n, coef, every):
    pos = torch.arange(n, dtype=F64)
    return 1.0 + coef * torch.log(torch.floor((pos + 1.0) / every) + 1.0)


def differential_lambda(w, p, diff):
    a = torch.exp((w[p + "lq1"].to(F64) * w[p + "lk1"].to(F64)).sum())
    b = torch.exp((w[p + "lq2"].to(F64) * w[p + "lk2"].to(F64)).sum())
    return a - b + diff


def differential_attention(h, w, p, m, eps):
    """Two softmax maps per head over the same values; the second is subtracted with a weight,
    the difference divided by its root mean square and gated."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].to(F64).T).view(n, H, 2, d)
    k = (h @ w[p + "k"].to(F64).T).view(n, G, 2, d)
    v = (h @ w[p + "v"].to(F64).T).view(n, G, dv)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(n, qt["coef"], qt["every"])[:, None, None, None]
    seen = causal(n)
    a1 = attend(q[:, :, 0], k[:, :, 0], v, m["scale"], seen)
    a2 = attend(q[:, :, 1], k[:, :, 1], v, m["scale"], seen)
    o = a1 - differential_lambda(w, p, m["diff"]) * a2
    o = unit_rms(o, eps) * (1.0 - m["diff"])
    g = torch.sigmoid(h @ w[p + "g"].to(F64).T)
    return (o * g[:, :, None]).reshape(n, -1) @ w[p + "o"].to(F64).T


# ------------------------------------------------------------------------------- gated linear attention
def channel_decay(h, w, p, tau):
    z = (h @ w[p + "a1"].to(F64).T) @ w[p + "a2"].to(F64).T + w[p + "a2.b"].to(F64)
    return torch.sigmoid(z) ** (1.0 / tau)


def gated_linear_attention(h, w, p, m, eps, return_state=False):
    """Per head a matrix state ``S [d, dv]``: ``S <- diag(alpha_t) S + k_t v_t^T``, ``o_t = S^T q_t``."""
    n = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].to(F64).T).view(n, H, d) * d ** -0.5
    k = (h @ w[p + "k"].to(F64).T).view(n, H, d)
    v = (h @ w[p + "v"].to(F64).T).view(n, H, dv)
    alpha = channel_decay(h, w, p, m["tau"]).view(n, H, d)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(n, H, dv, dtype=F64)
    for t in range(n):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = weighted_norm(o, w[p + "norm"].to(F64), eps).reshape(n, H * dv)
    z = h @ w[p + "g"].to(F64).T
    y = (o * z * torch.sigmoid(z)) @ w[p + "o"].to(F64).T
    return (y, S) if return_state else y


# ------------------------------------------------------------------------------- feed-forward
def squared_relu_mlp(h, w, p):
    return torch.relu(h @ w[p + "up"].to(F64).T) ** 2 @ w[p + "down"].to(F64).T


MIXERS = {"attention": windowed_attention, "attention_2": differential_attention, "gla": gated_linear_attention}


# ------------------------------------------------------------------------------- the model
def forward(tokens, w, cfg, return_layers=False):
    eps = cfg["norm"]["eps"]
    S = cfg["streams"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"].to(F64)[tokens] * cfg["embedding"]["scale"]
    X = x[:, None, :].repeat(1, S, 1)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        subs = [("1", lambda h: MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps))]
        if layer.get("mlp"):
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            subs.append(("2", lambda h: squared_relu_mlp(h, w, p + "mlp.")))
        for q, fn in subs:
            hc = p + "hc" + q
            u = streams_read(X, w[hc + ".in"].to(F64))
            y = fn(weighted_norm(u, w[p + "norm" + q].to(F64), eps)) * w[p + "ls" + q].to(F64)
            X = streams_write(X, y, w[hc + ".mix"].to(F64), w[hc + ".out"].to(F64))
        after.append(X.sum(1))
    logits = weighted_norm(X.sum(1), w["final.norm"].to(F64), eps) @ w["embed"].to(F64).T * cfg["logit_scale"]
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
