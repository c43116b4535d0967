"""Host-side tests of the Fafelix design (no GPU): the configuration reader and its refusals, the order of layer runs,
and the oracle against second formulations of its own mechanisms."""
import math

import pytest
import torch

from fafelix_common import attn, config_a, delta, dense, model_cfg, random_checkpoint, wkv


def test_config_reader_and_layer_runs():
    from compactor_vllm.config.model_config import FafelixConfig, load_model_config

    c = FafelixConfig.from_json(config_a())
    assert [l.mixer_type for l in c.layers] == ["attention", "wkv", "delta", "attention", "delta"]
    assert c.layer_runs == [(0, False), (1, False), (0, True), (1, False), (2, False), (3, False),
                            (4, False)]
    assert c.num_hidden_layers == 7 and c.layers[2].mlp is None and c.layers[0].mlp.ff == 40
    a = c.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.rot_dims) == (4, 2, 12, 10, 6) and a.rot_scaling == (4.0, 1.0, 4.0, 64.0)
    assert c.layers[3].mixer.rot_scaling is None and (c.buckets, c.mul_prev, c.mul_cur) == (61, 29, 7)
    plain = FafelixConfig.from_json(model_cfg([(wkv(), None)]))
    assert plain.loop is None and plain.layer_runs == [(0, False)] and plain.num_key_value_heads == 1
    late = FafelixConfig.from_json(model_cfg([(wkv(), None), (delta(), None), (attn(), None)], loop=(1, 3, 2)))
    assert late.layer_runs == [(0, False), (1, False), (2, False), (1, True), (2, False)]
    once = FafelixConfig.from_json(model_cfg([(wkv(), None), (delta(), None)], loop=(0, 2, 1)))
    assert once.layer_runs == [(0, False), (1, False)]


def test_config_refusals():
    from compactor_vllm.config.model_config import FafelixConfig

    with pytest.raises(ValueError):
        FafelixConfig.from_json(model_cfg([({"type": "conv", "mixer": {}}, None)]))
    with pytest.raises(ValueError):
        FafelixConfig.from_json(model_cfg([(attn(4, 3), None)]))                  # heads do not split into kv heads
    with pytest.raises(ValueError):
        FafelixConfig.from_json(model_cfg([(attn(rot=7), None)]))                  # odd rotation size
    with pytest.raises(ValueError):
        FafelixConfig.from_json(model_cfg([(attn(dim=8, rot=10), None)]))          # rotation wider than the head
    with pytest.raises(ValueError):
        FafelixConfig.from_json(model_cfg([(wkv(), None)], loop=(1, 0, 2)))
    with pytest.raises(ValueError):
        FafelixConfig.from_json(model_cfg([(wkv(), {"kind": "moe", "ff": 8})]))
    bad = model_cfg([(wkv(), None)])
    del bad["embedding"]
    with pytest.raises(ValueError):
        FafelixConfig.from_json(bad)


def test_config_is_found_by_its_architecture_name(tmp_path):
    import json

    from compactor_vllm.config.model_config import FafelixConfig, load_model_config
    from compactor_vllm.models import MODEL_REGISTRY, registry_key

    (tmp_path / "config.json").write_text(json.dumps(config_a()))
    c = load_model_config(str(tmp_path))
    assert isinstance(c, FafelixConfig) and registry_key(c) == "fafelix" and "fafelix" in MODEL_REGISTRY


def test_frequency_scaling_matches_the_product_table():
    from compactor_vllm.layers.attention import pair_rotation_frequencies
    from oracle import fafelix as O

    for dims, base, sc in ((24, 300000.0, (6.0, 1.0, 4.0, 2048)), (64, 10000.0, (4.0, 2.0, 8.0, 512)), (8, 100.0, None)):
        assert torch.allclose(pair_rotation_frequencies(dims, base, sc), O.scaled_frequencies(dims, base, sc), rtol=1e-12)
    # a wavelength exactly on a band's edge belongs to the blend, which meets both neighbours there
    f = 2 * math.pi / 16.0
    base = f ** (-8.0 / 2.0)          # dims 8: pair 1 has exactly this frequency
    got = pair_rotation_frequencies(8, base, (4.0, 1.0, 4.0, 64.0))
    assert math.isclose(float(got[1]), f, rel_tol=1e-9)


def _oracle_model(layers, **kw):
    from oracle import fafelix as O

    cfg = model_cfg(layers, **kw)
    return O, O.from_checkpoint(cfg, random_checkpoint(cfg, seed=1))


def test_oracle_delta_rule_against_the_unrolled_update():
    """S_t = g_t (I - beta_t k_t k_t^T) S_(t-1) + beta_t k_t v_t^T, written as one matrix product per token."""
    O, om = _oracle_model([(delta(2, 1, 6, 5, 3), None)])
    m, eps = om["layers"][0]["mixer"], om["eps"]
    T = 9
    h = torch.randn(T, 48, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    want = O.delta(h, m, eps)
    D, Dv, H = 6, 5, 2
    q = O.short_conv(h @ m["q"].double().T, m["q_conv"]).view(T, 1, D)
    k = O.short_conv(h @ m["k"].double().T, m["k_conv"]).view(T, 1, D)
    v = O.short_conv(h @ m["v"].double().T, m["v_conv"]).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(D)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = O.sigmoid(h @ m["b"].double().T)
    g = torch.exp(-torch.exp(m["A_log"].double()) * O.softplus(h @ m["a"].double().T + m["dt_bias"].double()))
    o = torch.zeros(T, H, Dv, dtype=torch.float64)
    for hh in range(H):
        S = torch.zeros(D, Dv, dtype=torch.float64)
        for t in range(T):
            kt = k[t, 0]
            S = g[t, hh] * (torch.eye(D, dtype=torch.float64) - beta[t, hh] * torch.outer(kt, kt)) @ S \
                + beta[t, hh] * torch.outer(kt, v[t, hh])
            o[t, hh] = S.T @ q[t, 0]
    o = O.rms_unit(o, eps) * m["norm"].double() * O.silu(h @ m["g"].double().T).view(T, H, Dv)
    assert torch.allclose(o.reshape(T, -1) @ m["o"].double().T, want, rtol=1e-9, atol=1e-9)


def test_oracle_wkv_against_the_sum_over_earlier_tokens():
    """o_t = sum_(s<t) (prod_(s<j<t) w_j) k_s (r_t . ) v_s + bonus term, written without a state."""
    O, om = _oracle_model([(wkv(2, 5), None)])
    m, eps = om["layers"][0]["mixer"], om["eps"]
    T, H, D = 8, 2, 5
    h = torch.randn(T, 48, dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    want = O.wkv(h, m, eps)
    prev = torch.cat([torch.zeros(1, 48, dtype=torch.float64), h[:-1]])
    mix = lambda n: h + (prev - h) * m["mu"][n].double()
    r, k, v = ((mix(n) @ m[n].double().T).view(T, H, D) for n in "rkv")
    w = torch.exp(-torch.exp(torch.tanh(mix("w") @ m["w1"].double().T) @ m["w2"].double().T + m["w0"].double())).view(T, H, D)
    o = torch.zeros(T, H, D, dtype=torch.float64)
    for hh in range(H):
        for t in range(T):
            acc = (r[t, hh] * m["u"].double()[hh] * k[t, hh]).sum() * v[t, hh]
            for s in range(t):
                decay = torch.ones(D, dtype=torch.float64)
                for j in range(s + 1, t):
                    decay = decay * w[j, hh]
                acc = acc + (r[t, hh] * decay * k[s, hh]).sum() * v[s, hh]
            o[t, hh] = acc
    o = O.rms_unit(o, eps).reshape(T, -1) * m["norm"].double() * O.silu(mix("g") @ m["g"].double().T)
    assert torch.allclose(o @ m["o"].double().T, want, rtol=1e-9, atol=1e-9)


def test_oracle_attention_sink_and_rotation():
    """Softmax with the sink as one more column of score sink_h and value zero; rotation by complex multiplication."""
    O, om = _oracle_model([(attn(2, 1, 8, 6, 4, base=30.0, scaling=None, scale=0.7), None)])
    m, eps = om["layers"][0]["mixer"], om["eps"]
    T = 7
    h = torch.randn(T, 48, dtype=torch.float64, generator=torch.Generator().manual_seed(4))
    want = O.attention(h, m, eps)
    q = (h @ m["q"].double().T + m["q_b"].double()).view(T, 2, 8)
    k = (h @ m["k"].double().T + m["k_b"].double()).view(T, 1, 8)
    v = (h @ m["v"].double().T + m["v_b"].double()).view(T, 1, 6)

    def rot(x):
        z = torch.view_as_complex(x[..., :4].reshape(*x.shape[:-1], 2, 2).contiguous())
        ang = torch.arange(T, dtype=torch.float64)[:, None] * torch.tensor([1.0, 30.0 ** -0.5], dtype=torch.float64)
        z = z * torch.polar(torch.ones_like(ang), ang)[:, None, :]
        return torch.cat([torch.view_as_real(z).reshape(*x.shape[:-1], 4), x[..., 4:]], dim=-1)

    q, k = O.rms_unit(rot(q), eps), O.rms_unit(rot(k), eps)
    out = torch.zeros(T, 2, 6, dtype=torch.float64)
    for hh in range(2):
        for t in range(T):
            s = torch.cat([(k[:t + 1, 0] @ q[t, hh]) * 0.7, m["sink"].double()[hh:hh + 1]])
            p = torch.softmax(s, dim=0)
            out[t, hh] = p[:-1] @ v[:t + 1, 0]
    assert torch.allclose(out.reshape(T, -1) @ m["o"].double().T, want, rtol=1e-9, atol=1e-9)


def test_oracle_loop_readds_the_embedding_once_per_later_pass():
    O, om = _oracle_model([(wkv(2, 5), dense(12)), (delta(2, 1, 6, 5, 3), None)], loop=(0, 2, 2))
    toks = [3, 9, 9, 4, 60, 1]
    col = []
    O.forward(om, toks, col)
    assert len(col) == 4
    x0 = O.embedding(om, toks)
    L0 = om["layers"][0]
    # the stream after the first layer of the second pass = (stream after pass one + embedding) + that layer's update
    x = col[1] + x0
    hn = O.layer_norm(x, L0["norm1"], L0["norm1_b"], om["eps"])
    assert torch.allclose(col[2], x + O.wkv(hn, L0["mixer"], om["eps"]) + O.feed_forward(hn, L0["mlp"]), rtol=1e-10, atol=1e-10)
    assert O.bigram_rows(toks, 61, 29, 7) == [61, (3 * 29 + 9 * 7) % 61, (9 * 29 + 9 * 7) % 61, (9 * 29 + 4 * 7) % 61,
                                              (4 * 29 + 60 * 7) % 61, (60 * 29 + 7) % 61]
