"""Helpers of the Fafelix tests: small configurations, checkpoints with random tensors, the engine's parameters as the
oracle's dict."""
import json
import struct
from pathlib import Path

import torch


def attn(heads=4, kv_heads=2, dim=16, vdim=12, rot=8, base=300.0, scaling=(4.0, 1.0, 4.0, 64), scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 1.2 * dim ** -0.5,
         "rot": {"base": base, "dims": rot}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "attention", "mixer": m}


def delta(heads=4, kv_heads=2, dim=12, vdim=10, conv=3):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def wkv(heads=3, dim=12):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def model_cfg(layers, vocab=83, width=48, eps=1e-5, loop=None, buckets=61, mul_prev=29, mul_cur=7):
    c = {"architecture": "Fafelix", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
         "layers": [dict(mixer_layer, mlp=mlp) for mixer_layer, mlp in layers]}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


def config_a():
    """All three mixers, a loop over an attention and a wkv layer, a layer without feed-forward, odd sizes (the
    kernels' scalar paths)."""
    return model_cfg([
        (attn(4, 2, 12, 10, 6), dense(40)),
        (wkv(3, 12), dense(28)),
        (delta(4, 2, 12, 10, 3), None),
        (attn(3, 3, 10, 14, 10, scaling=None), dense(36)),
        (delta(2, 2, 20, 6, 4), dense(30)),
    ], loop=(0, 2, 2))


def config_b():
    """Sizes in multiples of 16: the vector and tensor-core paths of the attention kernels; a loop over a delta layer."""
    return model_cfg([
        (wkv(4, 16), dense(64)),
        (attn(4, 2, 32, 32, 16, base=10000.0, scaling=(8.0, 1.0, 4.0, 32)), dense(64)),
        (delta(4, 2, 16, 32, 4), dense(48)),
        (attn(2, 1, 64, 64, 64, base=500.0, scaling=None), None),
    ], vocab=96, width=64, eps=1e-6, loop=(2, 3, 2), buckets=127, mul_prev=1000003, mul_cur=31)


def make_runner(cfg_json, dtype="float32", pages=24, page_size=16, max_seqs=4, seed=0, max_batched_tokens=None,
                device_allocator=False, eager=True):
    from compactor_vllm.config.engine_config import LLMConfig
    from compactor_vllm.config.model_config import FafelixConfig
    from compactor_vllm.core.model_runner import ModelRunner

    hf = FafelixConfig.from_json(cfg_json)
    cfg = LLMConfig(model="synthetic", hf_config=hf, dtype=dtype, max_num_seqs=max_seqs, kvcache_page_size=page_size,
                    max_model_len=pages * page_size, enforce_eager=eager)
    return ModelRunner(cfg, num_pages=pages, seed=seed, device_allocator=device_allocator,
                       max_batched_tokens=max_batched_tokens)


def oracle_model(model):
    """The engine model's parameters as the oracle's dict (fp32 copies on the CPU)."""
    cfg = model.config
    f = lambda p: p.detach().float().cpu()
    layers = []
    for i, layer in enumerate(model.layers):
        a, mx = cfg.layers[i].mixer, layer.mixer
        w = f(layer.in_proj.weight) if layer.in_proj is not None else None
        parts, at = {}, 0
        for name, n in mx.in_parts:
            parts[name] = w[at:at + n]
            at += n
        if layer.kind == "attention":
            b = f(layer.in_proj.bias)
            nq, nk = a.heads * a.dim, a.kv_heads * a.dim
            m = {"type": "attention", "heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim,
                 "scale": a.scale, "rot_dims": a.rot_dims, "rot_base": a.rot_base, "rot_scaling": a.rot_scaling,
                 "q": parts["q"], "k": parts["k"], "v": parts["v"], "q_b": b[:nq], "k_b": b[nq:nq + nk],
                 "v_b": b[nq + nk:mx.in_cols], "sink": f(mx.attn.sink_logits), "o": f(mx.o_proj.weight)}
        elif layer.kind == "delta":
            cw = f(mx.conv_weight)
            nq = a.kv_heads * a.dim
            m = {"type": "delta", "heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "conv": a.conv,
                 "q": parts["q"], "k": parts["k"], "v": parts["v"], "g": parts["g"], "b": parts["b"], "a": parts["a"],
                 "q_conv": cw[:nq], "k_conv": cw[nq:2 * nq], "v_conv": cw[2 * nq:], "A_log": f(mx.A_log),
                 "dt_bias": f(mx.dt_bias), "norm": f(mx.norm_weight), "o": f(mx.o_proj.weight)}
        else:
            r4 = f(mx.rkvg)
            m = {"type": "wkv", "heads": a.heads, "dim": a.dim, "mu": {n: f(mx.mu)[k] for k, n in enumerate("rkvgw")},
                 "r": r4[0], "k": r4[1], "v": r4[2], "g": r4[3], "w1": f(mx.w1.weight), "w2": f(mx.w2.weight),
                 "w0": f(mx.w0), "u": f(mx.bonus).view(a.heads, a.dim), "norm": f(mx.norm_weight),
                 "o": f(mx.o_proj.weight)}
        mlp = None
        if layer.ff:
            gu = w[mx.in_cols:]
            mlp = {"gate": gu[:layer.ff], "up": gu[layer.ff:], "down": f(layer.down_proj.weight)}
        layers.append({"norm1": f(layer.norm1.weight), "norm1_b": f(layer.norm1.bias), "mixer": m, "mlp": mlp})
    return {"embed": f(model.embed.tokens.weight), "bigram": f(model.embed.pairs.weight), "buckets": cfg.buckets,
            "mul_prev": cfg.mul_prev, "mul_cur": cfg.mul_cur, "eps": cfg.rms_norm_eps, "final_norm": f(model.norm.weight),
            "final_norm_b": f(model.norm.bias), "head": f(model.lm_head.weight), "layers": layers, "loop": cfg.loop}


def random_checkpoint(cfg: dict, seed: int = 0, decay_rank: int = 5) -> dict:
    """Every tensor name of the design with random bfloat16 values, for the given config.json dict."""
    W, V = cfg["width"], cfg["vocab"]
    g = torch.Generator().manual_seed(seed)
    t = {}

    def mat(name, *shape, scale=None):
        t[name] = (torch.randn(*shape, generator=g) * (scale if scale is not None else shape[-1] ** -0.5)).to(torch.bfloat16)

    def vec(name, *shape, mean=0.0, spread=0.1):
        t[name] = (mean + spread * torch.randn(*shape, generator=g)).to(torch.bfloat16)

    mat("embed", V, W, scale=1.0)
    mat("bigram", cfg["embedding"]["bigram"]["buckets"] + 1, W, scale=0.5)
    mat("head", V, W)
    vec("final.norm", W, mean=1.0)
    vec("final.norm.b", W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        vec(p + "norm1", W, mean=1.0)
        vec(p + "norm1.b", W)
        H, D = m["heads"], m["dim"]
        G, Dv = m.get("kv_heads", H), m.get("vdim", D)
        if layer["type"] == "attention":
            mat(p + "mix.q", H * D, W); mat(p + "mix.k", G * D, W); mat(p + "mix.v", G * Dv, W)
            vec(p + "mix.q.b", H * D); vec(p + "mix.k.b", G * D); vec(p + "mix.v.b", G * Dv)
            vec(p + "mix.sink", H, spread=1.0); mat(p + "mix.o", W, H * Dv)
        elif layer["type"] == "delta":
            taps = m["conv"]
            mat(p + "mix.q", G * D, W); mat(p + "mix.k", G * D, W); mat(p + "mix.v", H * Dv, W)
            mat(p + "mix.q.conv", G * D, taps, scale=0.5); mat(p + "mix.k.conv", G * D, taps, scale=0.5)
            mat(p + "mix.v.conv", H * Dv, taps, scale=0.5)
            mat(p + "mix.b", H, W); mat(p + "mix.a", H, W); mat(p + "mix.g", H * Dv, W)
            vec(p + "mix.A_log", H, spread=0.5); vec(p + "mix.dt_bias", H, mean=-0.5, spread=0.5)
            vec(p + "mix.norm", Dv, mean=1.0); mat(p + "mix.o", W, H * Dv)
        else:
            for n in "rkvgw":
                t[p + "mix.mu." + n] = torch.rand(W, generator=g).to(torch.bfloat16)
            for n in "rkvg":
                mat(p + "mix." + n, H * D, W)
            mat(p + "mix.w1", decay_rank, W); mat(p + "mix.w2", H * D, decay_rank)
            vec(p + "mix.w0", H * D, mean=-1.0, spread=0.7); vec(p + "mix.u", H, D, spread=0.5)
            vec(p + "mix.norm", H * D, mean=1.0); mat(p + "mix.o", W, H * D)
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            mat(p + "mlp.gate", ff, W); mat(p + "mlp.up", ff, W); mat(p + "mlp.down", W, ff)
    return t


def write_checkpoint(folder: Path, cfg: dict, tensors: dict) -> None:
    header, blob = {}, b""
    for name, x in tensors.items():
        raw = x.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(x.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    h = json.dumps(header).encode()
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + blob)


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def row_errs(got, want):
    """Per row: rms of the centred difference over the rms of the centred expectation."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()


def rel_err(got, want):
    return row_errs(got, want).max().item()


TOL = {"float32": 3e-5, "bfloat16": 6e-2}


def new_seq():
    from compactor_vllm.utils.sequence import Sequence

    return Sequence(prompt_token_ids=[])


def feed(runner, seq, toks, all_rows=True):
    seq.prompt_token_ids.extend(toks)
    return runner.run_step([(seq, toks)], rows=list(range(len(toks))) if all_rows else None)


def run_in_portions(runner, toks, sizes):
    """The request alone, cut into portions of the given sizes (cycled); logits of every position."""
    seq, out, at, k = new_seq(), [], 0, 0
    while at < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - at)
        out.append(feed(runner, seq, toks[at:at + n]))
        at, k = at + n, k + 1
    runner.release([seq])
    return torch.cat(out)
