"""Oracle: the Fafelix decoder in plain float64 torch on the CPU, one function per mechanism.

TEST INFRASTRUCTURE ONLY: nothing under compactor-vllm_b200/ imports this module and it imports nothing from
there.  Every function works on one whole sequence (no cache, no state slots, no batching): attention with a dense
score matrix, the recurrences token by token.

A model is a dict
  {"embed": [V, W], "bigram": [buckets + 1, W], "buckets", "mul_prev", "mul_cur", "eps", "final_norm", "final_norm_b",
   "head": [V, W], "layers": [layer, ...], "loop": None | (start, stop, times)}
a layer is
  {"norm1": [W], "norm1_b": [W], "mixer": mixer, "mlp": None | {"gate", "up", "down"}}
and a mixer is one of
  {"type": "attention", "heads", "kv_heads", "dim", "vdim", "scale", "rot_dims", "rot_base",
   "rot_scaling": None | (factor, low, high, original), "q", "q_b", "k", "k_b", "v", "v_b", "sink", "o"}
  {"type": "delta", "heads", "kv_heads", "dim", "vdim", "conv", "q", "q_conv", "k", "k_conv", "v", "v_conv", "b",
   "a", "A_log", "dt_bias", "g", "norm", "o"}
  {"type": "wkv", "heads", "dim", "mu" {"r","k","v","g","w"}, "r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o"}
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def _d(x):
    return x.to(F64)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms_unit(x, eps):
    x = _d(x)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    x = _d(x)
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * _d(w) + _d(b)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the hashed pair table for every token of a sequence; the first token takes the extra last row."""
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((int(prev) * mul_prev + int(cur) * mul_cur) % buckets)
    return rows


def embedding(model, tokens):
    tok = torch.tensor(list(tokens), dtype=torch.long)
    rows = torch.tensor(bigram_rows(list(tokens), model["buckets"], model["mul_prev"], model["mul_cur"]))
    return _d(model["embed"])[tok] + _d(model["bigram"])[rows]


def scaled_frequencies(dims, base, scaling):
    """Rotation frequencies of the dims / 2 pairs; long wavelengths are slowed by `factor`, short ones kept, the band
    between blended linearly in original / wavelength."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = scaling
            wl = 2.0 * math.pi / f
            if wl < original / high:
                pass
            elif wl > original / low:
                f = f / factor
            else:
                s = (original / wl - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_pairs(x, pos, freqs):
    """x [T, heads, D]: neighbours (2i, 2i + 1) of the first 2 * len(freqs) numbers turn by pos * freqs[i]."""
    n = freqs.numel()
    x = _d(x).clone()
    ang = _d(pos)[:, None] * freqs[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:2 * n:2].clone(), x[..., 1:2 * n:2].clone()
    x[..., 0:2 * n:2] = u * c - v * s
    x[..., 1:2 * n:2] = v * c + u * s
    return x


def attention(h, m, eps):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = _d(h)
    q = (h @ _d(m["q"]).T + _d(m["q_b"])).view(T, H, D)
    k = (h @ _d(m["k"]).T + _d(m["k_b"])).view(T, G, D)
    v = (h @ _d(m["v"]).T + _d(m["v_b"])).view(T, G, Dv)
    pos = torch.arange(T)
    fr = scaled_frequencies(m["rot_dims"], m["rot_base"], m["rot_scaling"])
    q = rms_unit(rotate_pairs(q, pos, fr), eps)
    k = rms_unit(rotate_pairs(k, pos, fr), eps)
    out = torch.zeros(T, H, Dv, dtype=F64)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~causal, -math.inf)
        sink = _d(m["sink"])[hh]
        mx = torch.maximum(s.max(dim=-1, keepdim=True).values, sink)
        e = torch.exp(s - mx)
        p = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - mx))
        out[:, hh] = p @ v[:, g]
    return out.reshape(T, H * Dv) @ _d(m["o"]).T


def short_conv(x, w):
    """x [T, C], w [C, taps] (last column = the current token): causal, zeros before the start, then silu."""
    T, C = x.shape
    taps = w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=F64), _d(x)], dim=0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y = y + xp[j:j + T] * _d(w)[:, j][None, :]
    return silu(y)


def delta(h, m, eps):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = _d(h)
    q = short_conv(h @ _d(m["q"]).T, m["q_conv"]).view(T, G, D)
    k = short_conv(h @ _d(m["k"]).T, m["k_conv"]).view(T, G, D)
    v = short_conv(h @ _d(m["v"]).T, m["v_conv"]).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = sigmoid(h @ _d(m["b"]).T)
    decay = torch.exp(-torch.exp(_d(m["A_log"])) * softplus(h @ _d(m["a"]).T + _d(m["dt_bias"])))
    gate = silu(h @ _d(m["g"]).T).view(T, H, Dv)
    o = torch.zeros(T, H, Dv, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(D, Dv, dtype=F64)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hh] = S.T @ q[t, g]
    o = rms_unit(o, eps) * _d(m["norm"])[None, None, :] * gate
    return o.reshape(T, H * Dv) @ _d(m["o"]).T


def wkv(h, m, eps):
    T, W = h.shape
    H, D = m["heads"], m["dim"]
    h = _d(h)
    prev = torch.cat([torch.zeros(1, W, dtype=F64), h[:-1]], dim=0)

    def mix(name):
        return h + (prev - h) * _d(m["mu"][name])[None, :]

    r = (mix("r") @ _d(m["r"]).T).view(T, H, D)
    k = (mix("k") @ _d(m["k"]).T).view(T, H, D)
    v = (mix("v") @ _d(m["v"]).T).view(T, H, D)
    gate = silu(mix("g") @ _d(m["g"]).T)
    w = torch.exp(-torch.exp(torch.tanh(mix("w") @ _d(m["w1"]).T) @ _d(m["w2"]).T + _d(m["w0"]))).view(T, H, D)
    u = _d(m["u"])
    o = torch.zeros(T, H, D, dtype=F64)
    for hh in range(H):
        S = torch.zeros(D, D, dtype=F64)
        for t in range(T):
            kv = torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = (S + u[hh][:, None] * kv).T @ r[t, hh]
            S = w[t, hh][:, None] * S + kv
    o = rms_unit(o, eps).reshape(T, H * D) * _d(m["norm"])[None, :] * gate
    return o @ _d(m["o"]).T


def feed_forward(h, f):
    h = _d(h)
    return (silu(h @ _d(f["gate"]).T) * (h @ _d(f["up"]).T)) @ _d(f["down"]).T


MIXERS = {"attention": attention, "delta": delta, "wkv": wkv}


def layer_runs(n_layers, loop):
    """[(layer, starts a later pass of the loop)] in execution order."""
    if loop is None:
        return [(i, False) for i in range(n_layers)]
    start, stop, times = loop
    runs = [(i, False) for i in range(start)]
    for p in range(times):
        runs += [(i, p > 0 and i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n_layers)]


def forward(model, tokens, collect=None):
    """tokens of ONE sequence from its start -> logits [T, V] (float64).  `collect`: a list that receives the
    residual stream after every layer run."""
    eps = model["eps"]
    x0 = embedding(model, tokens)
    x = x0.clone()
    for li, again in layer_runs(len(model["layers"]), model.get("loop")):
        L = model["layers"][li]
        if again:
            x = x + x0
        h = layer_norm(x, L["norm1"], L["norm1_b"], eps)
        y = MIXERS[L["mixer"]["type"]](h, L["mixer"], eps)
        if L["mlp"] is not None:
            y = y + feed_forward(h, L["mlp"])
        x = x + y
        if collect is not None:
            collect.append(x.clone())
    return layer_norm(x, model["final_norm"], model["final_norm_b"], eps) @ _d(model["head"]).T


def from_checkpoint(cfg: dict, tensors: dict) -> dict:
    """The oracle's model dict from a config.json dict and the checkpoint's tensors by name."""
    f = lambda name: tensors[name].float()
    bg = cfg["embedding"]["bigram"]
    lp = cfg.get("loop")
    model = {"embed": f("embed"), "bigram": f("bigram"), "buckets": bg["buckets"], "mul_prev": bg["mul_prev"],
             "mul_cur": bg["mul_cur"], "eps": cfg["norm"]["eps"], "final_norm": f("final.norm"),
             "final_norm_b": f("final.norm.b"), "head": f("head"), "layers": [],
             "loop": (lp["start"], lp["stop"], lp["times"]) if lp else None}
    for i, entry in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = dict(entry["mixer"])
        m["type"] = entry["type"]
        g = lambda name: f(p + "mix." + name)
        if entry["type"] == "attention":
            rot = m.pop("rot", None) or {}
            sc = rot.get("scaling")
            m.update(rot_dims=rot.get("dims", 0), rot_base=rot.get("base", 10000.0),
                     rot_scaling=(sc["factor"], sc["low"], sc["high"], sc["original"]) if sc else None)
            m.setdefault("kv_heads", m["heads"])
            m.setdefault("vdim", m["dim"])
            for n in "qkv":
                m[n], m[n + "_b"] = g(n), g(n + ".b")
            m["sink"], m["o"] = g("sink"), g("o")
        elif entry["type"] == "delta":
            m.setdefault("kv_heads", m["heads"])
            m.setdefault("vdim", m["dim"])
            for n in "qkv":
                m[n], m[n + "_conv"] = g(n), g(n + ".conv")
            for n in ("b", "a", "A_log", "dt_bias", "g", "norm", "o"):
                m[n] = g(n)
        else:
            m["mu"] = {n: g("mu." + n) for n in "rkvgw"}
            for n in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o"):
                m[n] = g(n)
        mlp = None
        if entry.get("mlp") is not None:
            mlp = {n: f(p + "mlp." + n) for n in ("gate", "up", "down")}
        model["layers"].append({"norm1": f(p + "norm1"), "norm1_b": f(p + "norm1.b"), "mixer": m, "mlp": mlp})
    return model
