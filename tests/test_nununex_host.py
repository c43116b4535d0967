"""Host-side tests of the Nununex design (no GPU): the configuration reader and its refusals, the distance buckets, and
the oracle against second formulations of its own mechanisms."""
import json
import math

import pytest
import torch

from nununex_common import clean, config_a, dense, gdelta, model_cfg, moe, par, random_checkpoint, scan, tokens


def test_config_reader():
    from compactor_vllm.config.model_config import NununexConfig

    c = NununexConfig.from_json(clean(config_a()))
    assert [l.mixer_type for l in c.layers] == ["mamba1", "general_delta", "parallel", "general_delta", "parallel", "mamba1"]
    assert c.num_hidden_layers == 6 and c.layers[2].mlp is None and c.layers[0].mlp.ff == 40
    assert (c.canon_taps, c.logit_softcap, c.buckets, c.mul_prev, c.mul_cur) == (3, 12.0, 61, 29, 7)
    a = c.layers[2].mixer.left
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.bias_max) == (4, 2, 12, 10, 7, 24)
    r = c.layers[4].mixer.right
    assert (r.heads, r.dim, r.vdim, r.gate_cap) == (2, 12, 6, 9.0)
    s = c.layers[5].mixer
    assert (s.inner, s.state, s.dt_rank, s.conv) == (20, 9, 2, 4)
    m = c.layers[1].mlp
    assert (m.kind, m.experts, m.top, m.ff, m.shared_ff) == ("moe", 5, 2, 12, 20) and c.layers[4].mlp.shared_ff == 0
    assert (c.num_key_value_heads, c.num_attention_heads, c.head_dim) == (3, 4, 12)
    plain = NununexConfig.from_json(clean(model_cfg([(scan(), None)])))
    assert plain.num_key_value_heads == 1
    nowin = clean(model_cfg([(par(), None)]))
    del nowin["layers"][0]["mixer"]["left"]["mask"]
    assert NununexConfig.from_json(nowin).layers[0].mixer.left.window == 0


def test_config_refusals():
    from compactor_vllm.config.model_config import NununexConfig

    with pytest.raises(ValueError):
        NununexConfig.from_json(model_cfg([({"type": "conv", "mixer": {}}, None)]))
    with pytest.raises(ValueError):
        NununexConfig.from_json(clean(model_cfg([(par(4, 3), None)])))              # heads do not split into kv heads
    with pytest.raises(ValueError):
        NununexConfig.from_json(clean(model_cfg([(par(cap=0.0), None)])))
    with pytest.raises(ValueError):
        NununexConfig.from_json(clean(model_cfg([(gdelta(), moe(3, 4))])))          # more choices than experts
    with pytest.raises(ValueError):
        NununexConfig.from_json(clean(model_cfg([(gdelta(), {"kind": "glu", "ff": 8})])))
    with pytest.raises(ValueError):
        NununexConfig.from_json(clean(model_cfg([(scan(conv=0), None)])))
    bad = clean(model_cfg([(gdelta(), None)]))
    del bad["embedding"]
    with pytest.raises(ValueError):
        NununexConfig.from_json(bad)


def test_config_is_found_by_its_architecture_name(tmp_path):
    from compactor_vllm.config.model_config import NununexConfig, load_model_config
    from compactor_vllm.models import MODEL_REGISTRY, registry_key

    (tmp_path / "config.json").write_text(json.dumps(clean(config_a())))
    c = load_model_config(str(tmp_path))
    assert isinstance(c, NununexConfig) and registry_key(c) == "nununex" and "nununex" in MODEL_REGISTRY


def test_distance_buckets():
    from compactor_vllm.layers.attention import distance_buckets
    from oracle import nununex as O

    for rows, far in ((16, 120), (8, 24), (6, 12), (32, 1000), (2, 5), (16, 128)):
        got = distance_buckets(rows, far, far + 40)
        assert got == [O.distance_bucket(n, rows, far) for n in range(far + 40)]
        half = rows // 2
        assert got[:half] == list(range(half)) and got[half] == half        # exact below half, the first shared bucket
        assert all(b2 >= b1 for b1, b2 in zip(got, got[1:])) and max(got) == rows - 1
        assert got[far] == rows - 1 and got[-1] == rows - 1
    # a far end inside the exact rows leaves no room for logarithmic buckets: the last row takes everything beyond
    assert distance_buckets(8, 3, 10) == [0, 1, 2, 3, 7, 7, 7, 7, 7, 7]


# ---- the oracle against second formulations ----------------------------------------------------------------------
def _h(T, W, seed):
    return torch.randn(T, W, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)


def test_general_delta_as_a_product_of_transition_matrices():
    """S_t = (diag(w) - (a u) u^T) S_(t-1) + k v^T: the rule is one matrix acting on the old state."""
    from oracle import nununex as O

    cfg = clean(model_cfg([(gdelta(2, 6), None)], width=16))
    t = random_checkpoint(model_cfg([(gdelta(2, 6), None)], width=16), 1)
    h, p, m = _h(9, 16, 2), "l0.mix.", cfg["layers"][0]["mixer"]
    want = O.general_delta(h, m, t, p, 1e-5)
    H, D = 2, 6
    r, k, v = (O.linear(h, t[p + n]).view(9, H, D) for n in "rkv")
    w = torch.exp(-math.exp(-0.5) * O.sigmoid(O.linear(torch.tanh(O.linear(h, t[p + "w1"])), t[p + "w2"]) + t[p + "w0"].double())).view(9, H, D)
    a = O.sigmoid(O.linear(h, t[p + "a"], t[p + "a.b"])).view(9, H, D)
    out = torch.zeros(9, H, D, dtype=torch.float64)
    for hh in range(H):
        S = torch.zeros(D, D, dtype=torch.float64)
        for i in range(9):
            u = k[i, hh] / torch.sqrt((k[i, hh] ** 2).sum() + 1e-6)
            S = (torch.diag(w[i, hh]) - torch.outer(a[i, hh] * u, u)) @ S + torch.outer(k[i, hh], v[i, hh])
            out[i, hh] = S.T @ r[i, hh]
    out = O.rms_unit(out, 1e-5).reshape(9, H * D) * t[p + "norm"].double() * O.sigmoid(O.linear(h, t[p + "g"]))
    assert torch.allclose(O.linear(out, t[p + "o"]), want, rtol=1e-10, atol=1e-12)


def test_matrix_memory_without_the_running_maximum():
    """With small gates the exponentials need no stabilizer: S = sum_j exp(i_j + sum_(l>j) f_l) k_j v_j^T directly, and
    the denominator's floor exp(-m) with m the maximum of those exponents and 0."""
    from oracle import nununex as O

    layer = par(1, 1, 4, 4, window=2, bias_max=5, rows=4, mheads=2, mdim=5, mvdim=7, cap=3.0)
    cfg = clean(model_cfg([(layer, None)], width=16))
    t = random_checkpoint(model_cfg([(layer, None)], width=16), 2)
    h, p, m = _h(12, 16, 3), "l0.mix.right.", cfg["layers"][0]["mixer"]["right"]
    want = O.matrix_memory(h, m, t, p, 1e-5)
    H, D, Dv, cap = 2, 5, 7, 3.0
    q = O.linear(h, t[p + "q"]).view(12, H, D) * D ** -0.5
    k, v = O.linear(h, t[p + "k"]).view(12, H, D), O.linear(h, t[p + "v"]).view(12, H, Dv)
    ig = cap * torch.tanh(O.linear(h, t[p + "i"], t[p + "i.b"]) / cap)
    fg = torch.log(O.sigmoid(cap * torch.tanh(O.linear(h, t[p + "f"], t[p + "f.b"]) / cap)))
    out = torch.zeros(12, H, Dv, dtype=torch.float64)
    for hh in range(H):
        for i in range(12):
            expo = torch.stack([ig[j, hh] + fg[j + 1:i + 1, hh].sum() for j in range(i + 1)])
            mx = torch.maximum(expo.max(), fg[:i + 1, hh].sum())      # the maximum's own start, 0, decays with the gates too
            wts = torch.exp(expo - mx)
            S = sum(wts[j] * torch.outer(k[j, hh], v[j, hh]) for j in range(i + 1))
            n = sum(wts[j] * k[j, hh] for j in range(i + 1))
            out[i, hh] = S.T @ q[i, hh] / (torch.maximum((n @ q[i, hh]).abs(), torch.exp(-mx)) + 1e-6)
    out = O.rms_unit(out, 1e-5).reshape(12, H * Dv) * t[p + "norm"].double() * O.sigmoid(O.linear(h, t[p + "g"]))
    assert torch.allclose(O.linear(out, t[p + "o"]), want, rtol=1e-9, atol=1e-11)


def test_window_attention_as_a_softmax_with_one_more_column():
    from oracle import nununex as O

    layer = par(4, 2, 6, 5, window=4, bias_max=12, rows=6)
    cfg = clean(model_cfg([(layer, None)], width=16))
    t = random_checkpoint(model_cfg([(layer, None)], width=16), 3)
    h, p, m = _h(15, 16, 4), "l0.mix.left.", cfg["layers"][0]["mixer"]["left"]
    want = O.window_attention(h, m, t, p)
    q = O.linear(h, t[p + "q"]).view(15, 4, 6)
    k, v = O.linear(h, t[p + "k"]).view(15, 2, 6), O.linear(h, t[p + "v"]).view(15, 2, 5)
    out = torch.zeros(15, 4, 5, dtype=torch.float64)
    for hh in range(4):
        for i in range(15):
            js = list(range(max(0, i - 3), i + 1))
            s = torch.stack([q[i, hh] @ k[j, hh // 2] * m["scale"] + t[p + "rel"].double()[O.distance_bucket(i - j, 6, 12), hh]
                             for j in js] + [t[p + "sink"].double()[hh]])
            pr = torch.softmax(s, 0)[:-1]
            out[i, hh] = sum(pr[n] * v[j, hh // 2] for n, j in enumerate(js))
    assert torch.allclose(O.linear(out.reshape(15, 20), t[p + "o"]), want, rtol=1e-10, atol=1e-12)


def test_selective_scan_as_a_sum_over_earlier_tokens():
    from oracle import nununex as O

    layer = scan(6, 3, 2, 3)
    cfg = clean(model_cfg([(layer, None)], width=16))
    t = random_checkpoint(model_cfg([(layer, None)], width=16), 4)
    h, p, m = _h(10, 16, 5), "l0.mix.", cfg["layers"][0]["mixer"]
    want = O.mamba1(h, m, t, p)
    xz = O.linear(h, t[p + "in"])
    x, z = xz[:, :6], xz[:, 6:]
    xc = torch.zeros_like(x)
    for i in range(10):
        for j in range(3):
            if i - 2 + j >= 0:
                xc[i] += t[p + "conv"].double()[:, j] * x[i - 2 + j]
    xc = O.silu(xc + t[p + "conv.b"].double())
    dbc = O.linear(xc, t[p + "x"])
    dt = torch.log1p(torch.exp(O.linear(dbc[:, :2], t[p + "dt"], t[p + "dt.b"])))
    A = -torch.exp(t[p + "A_log"].double())
    y = torch.zeros(10, 6, dtype=torch.float64)
    for i in range(10):
        for j in range(i + 1):
            decay = torch.exp(A * dt[j + 1:i + 1].sum(0).unsqueeze(-1))            # [channels, state]
            y[i] += (decay * (dt[j] * xc[j]).unsqueeze(-1) * dbc[j, 2:5]) @ dbc[i, 5:8]
        y[i] += t[p + "D"].double() * xc[i]
    assert torch.allclose(O.linear(y * O.silu(z), t[p + "o"]), want, rtol=1e-10, atol=1e-12)


def test_expert_weights_on_inputs_and_the_shared_gate():
    from oracle import nununex as O

    f = moe(4, 2, 6, 5)
    t = random_checkpoint(model_cfg([(gdelta(1, 4), f)], width=16), 5)
    h, p = _h(7, 16, 6), "l0.mlp."
    want = O.moe_ff(h, f, t, p)
    s = O.sigmoid(O.linear(h, t[p + "router"]))
    for i in range(7):
        best = sorted(range(4), key=lambda e: -float(s[i, e]))[:2]
        row = sum(O.linear(O.silu(O.linear(s[i, e] * h[i:i + 1], t[p + f"e{e}.gate"])) * O.linear(s[i, e] * h[i:i + 1], t[p + f"e{e}.up"]),
                           t[p + f"e{e}.down"]) for e in best)
        row = row + O.gated_expert(h[i:i + 1], t, p + "shared.") * O.sigmoid(h[i:i + 1] @ t[p + "shared.sg"].double().T)
        assert torch.allclose(row[0], want[i], rtol=1e-10, atol=1e-12)


def test_layer_arrangement_and_the_logit_cap():
    """A model of one layer, rebuilt from the mechanisms: norm, convolution on the way in, gate on the way out."""
    from oracle import nununex as O

    cfg0 = model_cfg([(scan(8, 3, 2, 2), dense(10))], width=16, taps=3, cap=2.0)
    cfg, t = clean(cfg0), random_checkpoint(cfg0, 6)
    toks = tokens(9, 83, 7)
    want = O.forward(cfg, t, toks)
    x = O.embedding(cfg, t, toks)
    assert torch.equal(x[0], t["embed"].double()[toks[0]] + t["bigram"].double()[61])
    for tag, fn in (("1", lambda hc: O.mamba1(hc, cfg["layers"][0]["mixer"], t, "l0.mix.")),
                    ("2", lambda hc: O.dense_ff(hc, t, "l0.mlp."))):
        h = O.rms_unit(x, 1e-5) * t["l0.norm" + tag].double()
        hc = h.clone()
        for i in range(9):
            for j in range(3):
                if i - 2 + j >= 0:
                    hc[i] += t["l0.canon" + tag].double()[:, j] * h[i - 2 + j]
        x = x + O.sigmoid(O.linear(h, t["l0.rg" + tag], t["l0.rg" + tag + ".b"])) * fn(hc)
    logits = O.linear(O.rms_unit(x, 1e-5) * t["final.norm"].double(), t["head"])
    assert torch.allclose(2.0 * torch.tanh(logits / 2.0), want, rtol=1e-10, atol=1e-12)
    assert want.abs().max() <= 2.0 and (logits.abs() > 2.0).any()
