"""Nununex: a decoder on a 32-bit residual stream whose every sublayer reads an RMS-normed input through a short causal
convolution and returns through a learned gate,

    x = embed[token] + pair[hash(previous token, token)]
    per layer, for the mixer and then (if the layer has one) the feed-forward:
        h = rms_norm(x) * w;   x += sigmoid(W_rg h + b_rg) * sublayer(h + causal_conv(h))
    logits = cap * tanh(head(rms_norm(x) * w) / cap)

with three kinds of mixer in any order and a dense or routed feed-forward.

Built from the engine's blocks:
  * embedding = `HashedPairEmbedding` (layers/pair_embedding.py), the previous token in the state pool;
  * the convolution in front of every sublayer = `ResidualShortConv` (layers/ssm.py), its last inputs in the state pool;
  * mixer "general_delta" = `GeneralDeltaMixer` (layers/recurrent.py);
  * mixer "parallel" = `BiasedChunkAttention` (layers/attention.py) with a sliding window, a learned bias per distance
    bucket and a learned sink, no rotation and no q/k norm, beside `MatrixMemoryMixer` (layers/recurrent.py); the two
    outputs are RMS-normed with weights of their own and averaged by `dual_norm_blend`;
  * mixer "mamba1" = `SelectiveScanMixer` (layers/ssm.py);
  * feed-forward = `PlainMLP` (relu squared, biases) or `RoutedExperts` (layers/moe.py) with ROUTE_SIGMOID routing, the
    routing weight on the experts' inputs, and a shared expert gated by one logit per token;
  * every norm is one `gated_residual_norm` launch (layers/layernorm.py): the gated residual sum of the sublayer
    before and the RMS norm in front of this one, also into the final norm; the logit cap is `cvllm_softcap`.
Everything that reads a sublayer's convolved input rides in ONE GEMM (`in_proj`); the gate reads the unconvolved norm
output (`rg`).  Weights: `load_weights` takes the checkpoint's tensors (`embed`, `bigram`, `final.norm`, `head`,
`l<i>.norm1|norm2|canon1|canon2|rg1|rg1.b|rg2|rg2.b`, general_delta `l<i>.mix.r|k|v|g|a|a.b|w1|w2|w0|norm|o`, parallel
`l<i>.mix.left.q|k|v|rel|sink|o|out` and `l<i>.mix.right.q|k|v|g|i|i.b|f|f.b|norm|o|out`, mamba1
`l<i>.mix.in|conv|conv.b|x|dt|dt.b|A_log|D|o`, dense `l<i>.mlp.up|up.b|down|down.b`, routed `l<i>.mlp.router`,
`l<i>.mlp.e<j>.gate|up|down`, `l<i>.mlp.shared.gate|up|down|sg`); `init_synthetic_weights` draws random ones.
"""
from __future__ import annotations

import math
import sys
from typing import Dict, List, Optional, Tuple

import torch
from torch import nn

from compactor_vllm import _native as N
from compactor_vllm.config.model_config import NununexConfig, ScaledMoEConfig
from compactor_vllm.layers.attention import BiasedChunkAttention
from compactor_vllm.layers.layernorm import NormWeight, dual_norm_blend, gated_residual_norm
from compactor_vllm.layers.moe import ACT_SILU, ROUTE_SIGMOID, PlainMLP, RoutedExperts
from compactor_vllm.layers.pair_embedding import HashedPairEmbedding
from compactor_vllm.layers.recurrent import GeneralDeltaMixer, MatrixMemoryMixer, MixerState
from compactor_vllm.layers.ssm import ResidualShortConv, SelectiveScanMixer
from compactor_vllm.utils.context import get_context

DELTA_DECAY_RATE = math.exp(-0.5)     # the general delta rule's decay is exp(-rate * sigmoid(.))


def make_feed_forward(width: int, m: Optional[ScaledMoEConfig], dtype) -> Optional[nn.Module]:
    if m is None:
        return None
    if m.kind == "dense":
        return PlainMLP(width, m.ff)
    return RoutedExperts(width, m.ff, m.experts, 0, m.top, 1, 1, m.shared_ff, ACT_SILU, dtype,
                         route_mode=ROUTE_SIGMOID, shared_gate=bool(m.shared_ff), scale_inputs=True)


class ParallelMixer(nn.Module):
    """Windowed attention and a matrix memory on the same input; 0.5 * (norm(left) * w_left + norm(right) * w_right)."""

    def __init__(self, width: int, m, eps: float):
        super().__init__()
        a, r = m.left, m.right
        self.eps = eps
        self.attn = BiasedChunkAttention(a.heads, a.kv_heads, a.dim, a.vdim, a.scale, sink=True, learned_sink=True,
                                         qk_norm=False, norm=False, eps=eps, window=a.window,
                                         bucket_bias=(a.bias_rows, a.bias_max))
        self.left_o = nn.Linear(a.heads * a.vdim, width, bias=False)
        self.memory = MatrixMemoryMixer(width, r.heads, r.dim, r.vdim, r.gate_cap, eps)
        self.left_out, self.right_out = NormWeight(width), NormWeight(width)
        self.left_cols = self.attn.qkv_width
        self.in_cols, self.in_bias = self.left_cols + self.memory.in_cols, True     # bias on the two gate logits only

    def make_state(self) -> MixerState:
        return self.memory.make_state()

    def forward(self, cols: torch.Tensor, state: MixerState) -> torch.Tensor:
        left = self.left_o(self.attn(cols[:, :self.left_cols]))
        right = self.memory(cols[:, self.left_cols:], state)
        return dual_norm_blend(left, self.left_out.weight, right, self.right_out.weight, self.eps, 0.5)


class NununexLayer(nn.Module):
    def __init__(self, cfg: NununexConfig, index: int, dtype):
        super().__init__()
        lc = cfg.layers[index]
        W, eps, taps = cfg.hidden_size, cfg.rms_norm_eps, cfg.canon_taps
        self.kind = lc.mixer_type
        m = lc.mixer
        if self.kind == "general_delta":
            self.mixer = GeneralDeltaMixer(W, m.heads, m.dim, m.decay_rank, DELTA_DECAY_RATE, eps)
        elif self.kind == "parallel":
            self.mixer = ParallelMixer(W, m, eps)
        else:
            self.mixer = SelectiveScanMixer(W, m.inner, m.state, m.dt_rank, m.conv)
        # what the mixer carries between steps, when that is not the mixer module's own attribute
        self.state = self.mixer.make_state() if hasattr(self.mixer, "make_state") else None
        self.norm1, self.canon1 = NormWeight(W), ResidualShortConv(W, taps)
        self.rg1 = nn.Linear(W, W, bias=True)
        self.in_proj = nn.Linear(W, self.mixer.in_cols, bias=self.mixer.in_bias)
        self.mlp = make_feed_forward(W, lc.mlp, dtype)
        if self.mlp is not None:
            self.norm2, self.canon2 = NormWeight(W), ResidualShortConv(W, taps)
            self.rg2 = nn.Linear(W, W, bias=True)

    def run_mixer(self, hc: torch.Tensor) -> torch.Tensor:
        cols = self.in_proj(hc)
        if self.kind == "general_delta":
            return self.mixer(hc, cols, self.state)
        if self.kind == "parallel":
            return self.mixer(cols, self.state)
        return self.mixer(cols)


class NununexForCausalLM(nn.Module):
    mixed_steps = True        # the runner may hand it portions of prompts beside single tokens in one step

    def __init__(self, cfg: NununexConfig):
        super().__init__()
        self.config = cfg
        dtype = torch.get_default_dtype()
        W = cfg.hidden_size
        self.embed = HashedPairEmbedding(cfg.vocab_size, W, cfg.buckets, cfg.mul_prev, cfg.mul_cur)
        self.layers = nn.ModuleList([NununexLayer(cfg, i, dtype) for i in range(len(cfg.layers))])
        self.norm = NormWeight(W)
        self.lm_head = nn.Linear(W, cfg.vocab_size, bias=False)
        self.debug_residuals: Optional[list] = None   # a list collects the residual stream after every layer

    # ---- what the cache manager asks ----------------------------------------------------------------------
    def cache_specs(self):
        """One entry per cache layer (= layer with attention): (attention module, kv heads, key size, value size)."""
        return [(l.mixer.attn, l.mixer.attn.num_kv_heads, l.mixer.attn.head_dim, l.mixer.attn.v_head_dim)
                for l in self.layers if l.kind == "parallel"]

    def state_layers(self):
        """Everything that carries state between steps in slots of the state pool: the embedding's previous token,
        the last inputs of every sublayer's convolution, and the mixers' recurrent states."""
        out: list = [self.embed]
        for l in self.layers:
            out.append(l.canon1)
            out.append(l.state if l.state is not None else l.mixer)
            if l.mlp is not None:
                out.append(l.canon2)
        return out

    # ---- forward ----------------------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        eps = self.config.rms_norm_eps
        dtype = self.lm_head.weight.dtype
        x = self.embed(input_ids)                                    # fp32 residual stream
        pending: Tuple[Optional[torch.Tensor], Optional[torch.Tensor]] = (None, None)    # (sublayer output, gate logits)
        for layer in self.layers:
            h = gated_residual_norm(x, branch=pending[0], gate=pending[1], weight=layer.norm1.weight, eps=eps,
                                    out_dtype=dtype)
            pending = (layer.run_mixer(layer.canon1(h)), layer.rg1(h))
            if layer.mlp is not None:
                h = gated_residual_norm(x, branch=pending[0], gate=pending[1], weight=layer.norm2.weight, eps=eps,
                                        out_dtype=dtype)
                pending = (layer.mlp(layer.canon2(h)), layer.rg2(h))
            if self.debug_residuals is not None:
                gated_residual_norm(x, branch=pending[0], gate=pending[1])
                pending = (None, None)
                self.debug_residuals.append(x.clone())
        return gated_residual_norm(x, branch=pending[0], gate=pending[1], weight=self.norm.weight, eps=eps,
                                   out_dtype=dtype)

    def compute_logits(self, hidden_states: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp32 logits of the given rows of the step (None: the last token of every sequence of the step)."""
        if rows is None:
            rows = get_context().cu_seqlens_q[1:].long() - 1
        return self.compute_all_logits(hidden_states.index_select(0, rows))

    def compute_all_logits(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """fp32 logits of every given row: the head, then the tanh cap."""
        logits = self.lm_head(hidden_states)
        cap = float(self.config.logit_softcap)
        if cap <= 0.0:
            return logits.float()
        out = torch.empty(logits.shape, dtype=torch.float32, device=logits.device)
        N.check(N.lib().cvllm_softcap(N.ptr(logits), logits.stride(0), N.ptr(out), out.stride(0), logits.shape[0],
                                      logits.shape[1], cap, N.block_dtype_code(logits.dtype), N.stream(logits.device)),
                "cvllm_softcap")
        return out

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

        def put_bias(linear, at: int, *names):
            linear.bias.zero_()
            src = torch.cat([get(n) for n in names], dim=0)
            linear.bias[at:at + src.numel()].copy_(src.to(linear.bias.dtype))

        put(self.embed.tokens.weight, "embed")
        put(self.embed.pairs.weight, "bigram")
        put(self.norm.weight, "final.norm")
        put(self.lm_head.weight, "head")
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            for tag in ("1", "2") if layer.mlp is not None else ("1",):
                put(getattr(layer, "norm" + tag).weight, p + "norm" + tag)
                put(getattr(layer, "canon" + tag).weight, p + "canon" + tag)
                put(getattr(layer, "rg" + tag).weight, p + "rg" + tag)
                put(getattr(layer, "rg" + tag).bias, p + "rg" + tag + ".b")
            mx, q = layer.mixer, p + "mix."
            if layer.kind == "general_delta":
                rank = get(q + "w1").shape[0]
                if rank != dict(mx.in_parts)["w1"]:      # the decay's inner size comes with the checkpoint
                    mx.set_decay_rank(rank)
                    lin = layer.in_proj
                    layer.in_proj = nn.Linear(lin.in_features, mx.in_cols, bias=True, device=lin.weight.device,
                                              dtype=lin.weight.dtype)
                put(layer.in_proj.weight, *[q + n for n, _ in mx.in_parts])
                put_bias(layer.in_proj, 4 * mx.heads * mx.dim, q + "a.b")
                put(mx.w2.weight, q + "w2")
                put(mx.w0, q + "w0")
                put(mx.norm_weight, q + "norm")
                put(mx.o_proj.weight, q + "o")
            elif layer.kind == "parallel":
                mem = mx.memory
                put(layer.in_proj.weight, q + "left.q", q + "left.k", q + "left.v",
                    *[q + "right." + n for n, _ in mem.in_parts])
                put_bias(layer.in_proj, mx.in_cols - 2 * mem.heads, q + "right.i.b", q + "right.f.b")
                rel = get(q + "left.rel")
                if rel.dim() != 2 or rel.shape[1] != mx.attn.num_heads:
                    raise ValueError(f"{q}left.rel: shape {tuple(rel.shape)} for {mx.attn.num_heads} heads")
                mx.attn.refresh_distance_bias(rel)
                put(mx.attn.sink_logits, q + "left.sink")
                put(mx.left_o.weight, q + "left.o")
                put(mx.left_out.weight, q + "left.out")
                put(mem.norm_weight, q + "right.norm")
                put(mem.o_proj.weight, q + "right.o")
                put(mx.right_out.weight, q + "right.out")
            else:
                put(layer.in_proj.weight, q + "in")
                put(mx.conv_weight, q + "conv")
                put(mx.conv_bias, q + "conv.b")
                put(mx.x_proj.weight, q + "x")
                put(mx.dt_proj.weight, q + "dt")
                put(mx.dt_bias, q + "dt.b")
                put(mx.A_log, q + "A_log")
                put(mx.D, q + "D")
                put(mx.o_proj.weight, q + "o")
            mlp, f = layer.mlp, p + "mlp."
            if mlp is None:
                continue
            if isinstance(mlp, PlainMLP):
                put(mlp.up_proj.weight, f + "up")
                put(mlp.up_proj.bias, f + "up.b")
                put(mlp.down_proj.weight, f + "down")
                put(mlp.down_proj.bias, f + "down.b")
                continue
            E = mlp.n_real
            mlp.router[:E].copy_(get(f + "router").float())
            for e in range(E):
                put(mlp.gate_up[e], f + f"e{e}.gate", f + f"e{e}.up")
                put(mlp.down[e], f + f"e{e}.down")
            if mlp.shared is not None:
                put(mlp.shared.gate_up_proj.weight, f + "shared.gate", f + "shared.up")
                put(mlp.shared.down_proj.weight, f + "shared.down")
                mlp.router[E:].copy_(get(f + "shared.sg").float().reshape(1, -1))
        extra = sorted(set(tensors) - used)
        if extra:
            print(f"nununex: {len(extra)} checkpoint tensors are not used: {extra[:8]}", file=sys.stderr)

    @torch.no_grad()
    def init_synthetic_weights(self, seed: int = 0) -> None:
        """Random weights drawn on the parameters' device: matrices N(0, 1/fan_in), norm gains near 1, small biases,
        decays and step sizes in the range where the recurrences neither die nor saturate."""
        for i, (name, p) in enumerate(self.named_parameters()):
            gen = torch.Generator(device=p.device).manual_seed(seed * 100003 + i)
            val = torch.randn(p.shape, generator=gen, device=p.device, dtype=torch.float32)
            leaf = name.rsplit(".", 1)[-1]
            if name.startswith("embed."):
                val = val * (0.5 if "pairs" in name else 1.0)
            elif leaf in ("norm_weight", "D") or (leaf == "weight" and p.dim() == 1):
                val = 1.0 + 0.1 * val
            elif leaf == "A_log":
                val = 0.5 * val
            elif leaf == "dt_bias":
                val = -1.0 + 0.5 * val
            elif leaf == "w0":
                val = 0.5 * val
            elif leaf in ("sink_logits", "rel"):
                val = 0.5 * val
            elif leaf == "conv_weight" or ("canon" in name and leaf == "weight"):
                val = val * 0.3
            elif leaf in ("bias", "conv_bias"):
                val = 0.1 * val
            else:
                val = val * (p.shape[-1] ** -0.5)
            p.copy_(val.to(p.dtype))
        for layer in self.layers:
            if layer.kind == "general_delta":      # only the removal-rate columns of the input projection are biased
                hd = layer.mixer.heads * layer.mixer.dim
                layer.in_proj.bias[:4 * hd].zero_()
                layer.in_proj.bias[5 * hd:].zero_()
            elif layer.kind == "parallel":         # only the two gate logits
                layer.in_proj.bias[:layer.mixer.in_cols - 2 * layer.mixer.memory.heads].zero_()
                layer.mixer.attn.refresh_distance_bias()
