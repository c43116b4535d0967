"""Oracle: the Nununex decoder in plain float64 torch on the CPU, one function per mechanism.

TEST INFRASTRUCTURE ONLY: nothing under compactor-vllm_b200/ imports this module and it imports nothing from
there.  Every function works on one whole sequence (no cache, no state slots, no batching): attention with a dense
score matrix, the recurrences token by token.

The model is given as it is stored: `cfg`, the dict of a config.json, and `tensors`, name -> tensor with the
checkpoint's names (`embed`, `bigram`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.canon1|2`, `l<i>.rg1|2(.b)`,
`final.norm`, `head`).  Linear weights are [out, in].

    x = embed[token] + bigram[hash(previous token, token)]
    per layer, for the mixer and then (if the layer has one) the feed-forward:
        h = rms_norm(x) * w;   x += sigmoid(W_rg h + b_rg) * sublayer(h + causal_conv(h))
    logits = cap * tanh(head(rms_norm(x) * w) / cap)
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
DECAY_RATE = math.exp(-0.5)      # general delta rule: w = exp(-DECAY_RATE * sigmoid(.))


def _d(x):
    return x.to(F64)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def log_sigmoid(z):
    return -softplus(-z)


def rms_unit(x, eps):
    x = _d(x)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def linear(x, w, b=None):
    y = _d(x) @ _d(w).T
    return y if b is None else y + _d(b)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((int(prev) * mul_prev + int(cur) * mul_cur) % buckets)
    return rows


def embedding(cfg, tensors, tokens):
    bg = cfg["embedding"]["bigram"]
    tok = torch.tensor(list(tokens), dtype=torch.long)
    rows = torch.tensor(bigram_rows(list(tokens), bg["buckets"], bg["mul_prev"], bg["mul_cur"]))
    return _d(tensors["embed"])[tok] + _d(tensors["bigram"])[rows]


def causal_conv(x, w, b=None):
    """x [T, C], w [C, taps]: out_t = b + sum_j w[:, j] x_(t - taps + 1 + j), zeros before the sequence."""
    x, w = _d(x), _d(w)
    T, taps = x.shape[0], w.shape[1]
    out = torch.zeros_like(x)
    for j in range(taps):
        shift = taps - 1 - j
        if shift < T:
            out[shift:] += x[:T - shift] * w[:, j]
    return out if b is None else out + _d(b)


# ---- mixers ------------------------------------------------------------------------------------------------------
def general_delta(h, m, t, p, eps):
    """Per head: S <- diag(w) S - (a u)(u^T S) + k v^T with both terms on the old S;  o = S^T r."""
    H, D = m["heads"], m["dim"]
    T = h.shape[0]
    r = linear(h, t[p + "r"]).view(T, H, D)
    k = linear(h, t[p + "k"]).view(T, H, D)
    v = linear(h, t[p + "v"]).view(T, H, D)
    w = torch.exp(-DECAY_RATE * sigmoid(linear(torch.tanh(linear(h, t[p + "w1"])), t[p + "w2"]) + _d(t[p + "w0"])))
    w = w.view(T, H, D)
    a = sigmoid(linear(h, t[p + "a"], t[p + "a.b"])).view(T, H, D)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, D, D, dtype=F64)
    o = torch.zeros(T, H, D, dtype=F64)
    for i in range(T):
        uS = torch.einsum("hk,hkv->hv", u[i], S)
        S = w[i].unsqueeze(-1) * S - (a[i] * u[i]).unsqueeze(-1) * uS.unsqueeze(1) + k[i].unsqueeze(-1) * v[i].unsqueeze(1)
        o[i] = torch.einsum("hkv,hk->hv", S, r[i])
    o = rms_unit(o, eps).reshape(T, H * D) * _d(t[p + "norm"]) * sigmoid(linear(h, t[p + "g"]))
    return linear(o, t[p + "o"])


def distance_bucket(n, rows, far):
    """Row of the distance-bias table for distance n >= 0: exact below rows // 2, logarithmic up to `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def window_attention(h, m, t, p):
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = linear(h, t[p + "q"]).view(T, H, D)
    k = linear(h, t[p + "k"]).view(T, G, D)
    v = linear(h, t[p + "v"]).view(T, G, Dv)
    rel = _d(t[p + "rel"])
    window = int((m.get("mask") or {}).get("size", 0) or 0)
    out = torch.zeros(T, H, Dv, dtype=F64)
    pos = torch.arange(T)
    dist = pos[:, None] - pos[None, :]
    seen = (dist >= 0) & ((dist < window) if window else (dist >= 0))
    rows = torch.tensor([distance_bucket(n, rel.shape[0], m["bias_max"]) for n in range(T)])[dist.clamp(min=0)]
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"] + rel[:, hh][rows]
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        sink = _d(t[p + "sink"])[hh]
        mx = torch.maximum(s.max(dim=1, keepdim=True).values, sink)
        e = torch.exp(s - mx)
        out[:, hh] = (e / (e.sum(dim=1, keepdim=True) + torch.exp(sink - mx))) @ v[:, g]
    return linear(out.reshape(T, H * Dv), t[p + "o"])


def matrix_memory(h, m, t, p, eps):
    """mLSTM with a running maximum of the log gates that starts at 0."""
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    T = h.shape[0]
    q = linear(h, t[p + "q"]).view(T, H, D) * D ** -0.5
    k = linear(h, t[p + "k"]).view(T, H, D)
    v = linear(h, t[p + "v"]).view(T, H, Dv)
    ig = cap * torch.tanh(linear(h, t[p + "i"], t[p + "i.b"]) / cap)
    fg = log_sigmoid(cap * torch.tanh(linear(h, t[p + "f"], t[p + "f.b"]) / cap))
    S = torch.zeros(H, D, Dv, dtype=F64)
    n = torch.zeros(H, D, dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    o = torch.zeros(T, H, Dv, dtype=F64)
    for i in range(T):
        m_new = torch.maximum(fg[i] + mx, ig[i])
        keep, take = torch.exp(fg[i] + mx - m_new), torch.exp(ig[i] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[i].unsqueeze(-1) * v[i].unsqueeze(1)
        n = keep[:, None] * n + take[:, None] * k[i]
        mx = m_new
        den = torch.maximum((n * q[i]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[i] = torch.einsum("hkv,hk->hv", S, q[i]) / den[:, None]
    o = rms_unit(o, eps).reshape(T, H * Dv) * _d(t[p + "norm"]) * sigmoid(linear(h, t[p + "g"]))
    return linear(o, t[p + "o"])


def parallel(h, m, t, p, eps):
    left = window_attention(h, m["left"], t, p + "left.")
    right = matrix_memory(h, m["right"], t, p + "right.", eps)
    return 0.5 * (rms_unit(left, eps) * _d(t[p + "left.out"]) + rms_unit(right, eps) * _d(t[p + "right.out"]))


def mamba1(h, m, t, p):
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    T = h.shape[0]
    xz = linear(h, t[p + "in"])
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, t[p + "conv"], t[p + "conv.b"]))
    dbc = linear(x, t[p + "x"])
    dt = softplus(linear(dbc[:, :R], t[p + "dt"], t[p + "dt.b"]))
    Bm, Cm = dbc[:, R:R + N], dbc[:, R + N:R + 2 * N]
    A = -torch.exp(_d(t[p + "A_log"]))
    S = torch.zeros(inner, N, dtype=F64)
    y = torch.zeros(T, inner, dtype=F64)
    for i in range(T):
        S = torch.exp(dt[i].unsqueeze(-1) * A) * S + (dt[i] * x[i]).unsqueeze(-1) * Bm[i].unsqueeze(0)
        y[i] = S @ Cm[i] + _d(t[p + "D"]) * x[i]
    return linear(y * silu(z), t[p + "o"])


# ---- feed-forwards -----------------------------------------------------------------------------------------------
def dense_ff(h, t, p):
    a = torch.relu(linear(h, t[p + "up"], t[p + "up.b"])) ** 2
    return linear(a, t[p + "down"], t[p + "down.b"])


def gated_expert(h, t, p):
    return linear(silu(linear(h, t[p + "gate"])) * linear(h, t[p + "up"]), t[p + "down"])


def moe_ff(h, f, t, p):
    E, top = f["router"]["experts"], f["router"]["top"]
    s = sigmoid(linear(h, t[p + "router"]))
    out = torch.zeros(h.shape[0], _d(t[p + "e0.down"]).shape[0], dtype=F64)
    for i in range(h.shape[0]):
        for e in torch.topk(s[i], top).indices.tolist():
            out[i] += gated_expert(s[i, e] * _d(h[i:i + 1]), t, p + f"e{e}.")[0]
    if f.get("shared"):
        out = out + gated_expert(h, t, p + "shared.") * sigmoid(linear(h, t[p + "shared.sg"]))
    assert E == s.shape[1]
    return out


def feed_forward(h, f, t, p):
    return dense_ff(h, t, p) if f.get("kind", "dense") == "dense" else moe_ff(h, f, t, p)


def mixer(h, layer, t, p, eps):
    kind = layer["type"]
    if kind == "general_delta":
        return general_delta(h, layer["mixer"], t, p, eps)
    if kind == "parallel":
        return parallel(h, layer["mixer"], t, p, eps)
    if kind == "mamba1":
        return mamba1(h, layer["mixer"], t, p)
    raise ValueError(kind)


def forward(cfg, tensors, tokens, collect=None):
    """Logits [T, vocab] of one whole sequence; `collect` (a list) receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = embedding(cfg, tensors, tokens)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        subs = [("1", lambda hc, layer=layer, p=p: mixer(hc, layer, tensors, p + "mix.", eps))]
        if layer.get("mlp") is not None:
            subs.append(("2", lambda hc, layer=layer, p=p: feed_forward(hc, layer["mlp"], tensors, p + "mlp.")))
        for tag, fn in subs:
            h = rms_unit(x, eps) * _d(tensors[p + "norm" + tag])
            gate = sigmoid(linear(h, tensors[p + "rg" + tag], tensors[p + "rg" + tag + ".b"]))
            x = x + gate * fn(h + causal_conv(h, tensors[p + "canon" + tag]))
        if collect is not None:
            collect.append(x.clone())
    h = rms_unit(x, eps) * _d(tensors["final.norm"])
    cap = float(cfg["logit_softcap"])
    return cap * torch.tanh(linear(h, tensors["head"]) / cap)
