"""Fafelix: a decoder whose layers run their mixer and their feed-forward side by side on ONE layer-normed input,

    x = embed[token] + pair[hash(previous token, token)];   per layer:  h = layer_norm(x),  x += mixer(h) + ff(h);
    logits = head(layer_norm(x))

on a 32-bit residual stream.  A span of layers may run several times in a row with the same weights; every pass owns
its cache layer or state, and the embedding output is added to the stream again in front of every pass but the first.

Built from the engine's blocks:
  * embedding = `HashedPairEmbedding` (layers/pair_embedding.py), the previous token in the state pool;
  * mixer "attention" = `BiasedChunkAttention` (layers/attention.py) with biased projections, a rotation of
    neighbouring pairs on part of every head (stretched long wavelengths), an RMS norm without weight on q and k and a
    learned sink per head; no distance bias, no chunks;
  * mixer "delta" = `DeltaRuleMixer`, mixer "wkv" = `WkvMixer` (layers/recurrent.py), their states in the state pool;
  * feed-forward = down(silu(gate h) * up h); its gate and up rows ride in the same GEMM as the mixer's projections of
    h (`in_proj`), the gated activation is the engine's kernel;
  * every norm is one `residual_norm` launch (layers/layernorm.py): the residual sum of the layer before (mixer + ff,
    plus the embedding at the start of a pass) and the layer norm in front of this one, also into the final norm.
Weights: `load_weights` takes the checkpoint's tensors (`embed`, `bigram`, `final.norm|norm.b`, `head`, `l<i>.norm1|norm1.b`,
attention `l<i>.mix.q|k|v` (+ `.b`) `|sink|o`, delta `l<i>.mix.q|k|v` (+ `.conv`) `|b|a|A_log|dt_bias|g|norm|o`, wkv
`l<i>.mix.mu.r|k|v|g|w`, `l<i>.mix.r|k|v|g|w1|w2|w0|u|norm|o`, `l<i>.mlp.gate|up|down`); `init_synthetic_weights` draws
random ones.
"""
from __future__ import annotations

import sys
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from compactor_vllm.config.model_config import FafelixConfig
from compactor_vllm.layers.attention import BiasedChunkAttention, pair_rotation_frequencies
from compactor_vllm.layers.layernorm import NORM_LAYER, LayerNormWeight, residual_norm
from compactor_vllm.layers.moe import ACT_SILU, gated_act
from compactor_vllm.layers.pair_embedding import HashedPairEmbedding
from compactor_vllm.layers.recurrent import DeltaRuleMixer, MixerState, WkvMixer
from compactor_vllm.utils.context import get_context


def make_attention(a, eps: float) -> BiasedChunkAttention:
    rot = pair_rotation_frequencies(a.rot_dims, a.rot_base, a.rot_scaling) if a.rot_dims > 0 else None
    return BiasedChunkAttention(a.heads, a.kv_heads, a.dim, a.vdim, a.scale, sink=True, learned_sink=True, rotation=rot,
                                qk_norm=False, norm=True, eps=eps)


class RotaryAttentionMixer(nn.Module):
    """q | k | v columns (biased) of the layer's input projection -> rotation, norm, paged attention, W_o."""

    def __init__(self, width: int, a, eps: float):
        super().__init__()
        self.attn = make_attention(a, eps)
        G, D, H, Dv = a.kv_heads, a.dim, a.heads, a.vdim
        self.in_parts = [("q", H * D), ("k", G * D), ("v", G * Dv)]
        self.in_cols, self.in_bias = self.attn.qkv_width, True
        self.o_proj = nn.Linear(H * Dv, width, bias=False)

    def forward(self, h: torch.Tensor, cols: torch.Tensor, attn: BiasedChunkAttention) -> torch.Tensor:
        return self.o_proj(attn(cols))


class FafelixLayer(nn.Module):
    def __init__(self, cfg: FafelixConfig, index: int, dtype):
        super().__init__()
        lc = cfg.layers[index]
        W, eps = cfg.hidden_size, cfg.rms_norm_eps
        a = lc.mixer
        self.kind = lc.mixer_type
        if self.kind == "attention":
            self.mixer = RotaryAttentionMixer(W, a, eps)
        elif self.kind == "delta":
            self.mixer = DeltaRuleMixer(W, a.heads, a.kv_heads, a.dim, a.vdim, a.conv, eps)
        else:
            self.mixer = WkvMixer(W, a.heads, a.dim, a.decay_rank, eps, dtype=dtype)
        self.ff = 0 if lc.mlp is None else int(lc.mlp.ff)
        self.norm1 = LayerNormWeight(W)
        # one GEMM for everything that reads h: the mixer's columns, then the feed-forward's gate | up
        cols = self.mixer.in_cols + 2 * self.ff
        self.in_proj = nn.Linear(W, cols, bias=self.mixer.in_bias) if cols > 0 else None
        self.down_proj = nn.Linear(self.ff, W, bias=False) if self.ff else None

    def forward(self, h: torch.Tensor, run_state) -> List[Optional[torch.Tensor]]:
        """h = the normed input -> [mixer(h), ff(h) | None], to be summed into the residual stream."""
        proj = self.in_proj(h) if self.in_proj is not None else None
        n = self.mixer.in_cols
        y_mix = self.mixer(h, None if n == 0 else proj[:, :n], run_state)
        y_ff = None
        if self.ff:
            y_ff = self.down_proj(gated_act(proj[:, n:], ACT_SILU))
        return [y_mix, y_ff]


class FafelixForCausalLM(nn.Module):
    mixed_steps = True        # the runner may hand it portions of prompts beside single tokens in one step

    def __init__(self, cfg: FafelixConfig):
        super().__init__()
        self.config = cfg
        dtype = torch.get_default_dtype()
        W = cfg.hidden_size
        self.embed = HashedPairEmbedding(cfg.vocab_size, W, cfg.buckets, cfg.mul_prev, cfg.mul_cur)
        self.layers = nn.ModuleList([FafelixLayer(cfg, i, dtype) for i in range(len(cfg.layers))])
        self.norm = LayerNormWeight(W)
        self.lm_head = nn.Linear(W, cfg.vocab_size, bias=False)
        self.layer_runs = cfg.layer_runs
        # what every layer RUN owns: an attention object with its own cache views (same parameters and constants as
        # the layer's), or a holder of state tensors
        self.run_state = nn.ModuleList()
        seen = set()
        for li, _ in self.layer_runs:
            layer = self.layers[li]
            if layer.kind != "attention":
                self.run_state.append(layer.mixer.make_state())
            elif li not in seen:
                self.run_state.append(layer.mixer.attn)
            else:
                twin = make_attention(cfg.layers[li].mixer, cfg.rms_norm_eps)
                twin.sink_logits = layer.mixer.attn.sink_logits      # shared parameter
                self.run_state.append(twin)
            seen.add(li)
        self.debug_residuals: Optional[list] = None   # a list collects the residual stream after every layer run

    # ---- what the cache manager asks ----------------------------------------------------------------------
    def cache_specs(self):
        """One entry per cache layer (= run of an attention layer): (attention module, kv heads, key size, value size)."""
        return [(a, a.num_kv_heads, a.head_dim, a.v_head_dim) for a in self.run_state
                if isinstance(a, BiasedChunkAttention)]

    def state_layers(self):
        """Everything that carries state between steps in slots of the state pool: the embedding's previous token and
        one holder per run of a recurrent layer."""
        return [self.embed] + [s for s in self.run_state if isinstance(s, MixerState)]

    # ---- forward ----------------------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        eps = cfg.rms_norm_eps
        dtype = self.lm_head.weight.dtype
        x0 = self.embed(input_ids)                                   # fp32, kept for the later passes of the loop
        again = any(flag for _, flag in self.layer_runs)
        x = x0.clone() if again else x0
        pending: List[Optional[torch.Tensor]] = []
        for run, (li, readd) in enumerate(self.layer_runs):
            layer = self.layers[li]
            h = residual_norm(x, add=tuple(pending), add_f32=x0 if readd else None, weight=layer.norm1.weight,
                              bias=layer.norm1.bias, eps=eps, kind=NORM_LAYER, out_dtype=dtype)
            pending = layer(h, self.run_state[run])
            if self.debug_residuals is not None:
                residual_norm(x, add=tuple(pending))
                pending = []
                self.debug_residuals.append(x.clone())
        return residual_norm(x, add=tuple(pending), weight=self.norm.weight, bias=self.norm.bias, eps=eps,
                             kind=NORM_LAYER, out_dtype=dtype)

    def compute_logits(self, hidden_states: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Logits of the given rows of the step (None: the last token of every sequence of the step)."""
        if rows is None:
            rows = get_context().cu_seqlens_q[1:].long() - 1
        return self.lm_head(hidden_states.index_select(0, rows))

    # ---- weights ----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        used = set()

        def get(name):
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            return tensors[name]

        def put(param, *names, shape=None):
            src = torch.cat([get(n) for n in names], dim=0) if len(names) > 1 else get(names[0])
            if shape is not None:
                if src.numel() != param.numel():
                    raise ValueError(f"{names}: {tuple(src.shape)} does not fit {tuple(param.shape)}")
                src = src.reshape(shape)
            if tuple(src.shape) != tuple(param.shape):
                raise ValueError(f"{names}: shape {tuple(src.shape)} does not fit {tuple(param.shape)}")
            param.copy_(src.to(param.dtype))

        put(self.embed.tokens.weight, "embed")
        put(self.embed.pairs.weight, "bigram")
        put(self.norm.weight, "final.norm")
        put(self.norm.bias, "final.norm.b")
        put(self.lm_head.weight, "head")
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            put(layer.norm1.weight, p + "norm1")
            put(layer.norm1.bias, p + "norm1.b")
            mx = layer.mixer
            rows = [p + "mix." + name for name, _ in mx.in_parts]
            if layer.ff:
                rows += [p + "mlp.gate", p + "mlp.up"]
                put(layer.down_proj.weight, p + "mlp.down")
            if rows:
                put(layer.in_proj.weight, *rows)
            if layer.kind == "attention":
                layer.in_proj.bias.zero_()
                layer.in_proj.bias[:mx.in_cols].copy_(torch.cat([get(p + f"mix.{n}.b") for n in "qkv"]).to(layer.in_proj.bias.dtype))
                put(mx.attn.sink_logits, p + "mix.sink")
            elif layer.kind == "delta":
                put(mx.conv_weight, p + "mix.q.conv", p + "mix.k.conv", p + "mix.v.conv")
                for param, name in ((mx.A_log, "A_log"), (mx.dt_bias, "dt_bias"), (mx.norm_weight, "norm")):
                    put(param, p + "mix." + name)
            else:
                put(mx.mu, *[p + "mix.mu." + n for n in mx.BLENDS], shape=mx.mu.shape)
                put(mx.rkvg, *[p + "mix." + n for n in "rkvg"], shape=mx.rkvg.shape)
                w1 = get(p + "mix.w1")
                if tuple(w1.shape) != tuple(mx.w1.weight.shape):     # the decay's inner size comes with the checkpoint
                    dev, dt = mx.w1.weight.device, mx.w1.weight.dtype
                    mx.w1 = nn.Linear(w1.shape[1], w1.shape[0], bias=False, device=dev, dtype=dt)
                    mx.w2 = nn.Linear(w1.shape[0], mx.w2.weight.shape[0], bias=False, device=dev, dtype=dt)
                put(mx.w1.weight, p + "mix.w1")
                put(mx.w2.weight, p + "mix.w2")
                put(mx.w0, p + "mix.w0")
                put(mx.bonus, p + "mix.u", shape=mx.bonus.shape)
                put(mx.norm_weight, p + "mix.norm")
            put(mx.o_proj.weight, p + "mix.o")
        extra = sorted(set(tensors) - used)
        if extra:
            print(f"fafelix: {len(extra)} checkpoint tensors are not used: {extra[:8]}", file=sys.stderr)

    @torch.no_grad()
    def init_synthetic_weights(self, seed: int = 0) -> None:
        """Random weights drawn on the parameters' device: matrices N(0, 1/fan_in), norm gains near 1, small biases,
        decays in the range where the recurrences neither die nor saturate."""
        for i, (name, p) in enumerate(self.named_parameters()):
            gen = torch.Generator(device=p.device).manual_seed(seed * 100003 + i)
            val = torch.randn(p.shape, generator=gen, device=p.device, dtype=torch.float32)
            leaf = name.rsplit(".", 1)[-1]
            if name.startswith("embed."):
                val = val * (0.5 if "pairs" in name else 1.0)
            elif leaf == "norm_weight" or (leaf == "weight" and p.dim() == 1):
                val = 1.0 + 0.1 * val
            elif leaf == "mu":
                val = torch.sigmoid(val)
            elif leaf == "A_log":
                val = 0.5 * val
            elif leaf == "dt_bias":
                val = -1.0 + 0.5 * val
            elif leaf == "w0":
                val = -1.5 + 0.7 * val
            elif leaf in ("bonus", "sink_logits"):
                val = 0.5 * val
            elif leaf == "conv_weight":
                val = val * 0.5
            elif leaf == "bias":
                val = 0.1 * val
            else:
                val = val * (p.shape[-1] ** -0.5)
            p.copy_(val.to(p.dtype))
        for layer in self.layers:      # the feed-forward's columns of the shared input projection have no bias
            if layer.in_proj is not None and layer.in_proj.bias is not None:
                layer.in_proj.bias[layer.mixer.in_cols:].zero_()
