"""Model configurations the engine reads itself (a folder's config.json), beside the HF ones `AutoConfig` resolves.

`load_model_config(path)` looks at config.json: a top-level "architecture" naming one of the designs below is
parsed here; anything else goes to transformers.  The result carries the attribute names the cache manager and the
runner read from an HF config (`model_type`, `torch_dtype`, `vocab_size`, `max_position_embeddings`, ...).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, List, Optional, Tuple

import torch


@dataclass
class AttentionMixerConfig:
    """Grouped-query attention without rotation: per-head RMS norm of q and k, a linear distance bias
    (slope of head h = 2 ** (-8 (h + 1) / heads)), a chunk mask and a softmax sink."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int = 0            # keys are visible inside the query's chunk of this many positions; 0 = no chunking

    @classmethod
    def from_json(cls, m: dict) -> "AttentionMixerConfig":
        mask = m.get("mask") or {}
        dim = int(m["dim"])
        return cls(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=dim,
                   vdim=int(m.get("vdim", dim)), scale=float(m.get("scale", dim ** -0.5)),
                   chunk=int(mask.get("size", 0) or 0))


@dataclass
class FeedForwardConfig:
    """kind "dense": down(gelu_tanh(gate h) * up h).  kind "moe": `experts` silu-gated experts of size `ff` plus
    `identity` experts that return their input; every token takes `top` of them (see layers/moe.py)."""
    kind: str
    ff: int
    experts: int = 0
    identity: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0        # 0 = no shared expert

    @classmethod
    def from_json(cls, m: Optional[dict]) -> Optional["FeedForwardConfig"]:
        if m is None:
            return None
        kind = m.get("kind", "dense")
        if kind == "dense":
            return cls(kind="dense", ff=int(m["ff"]))
        if kind != "moe":
            raise ValueError(f"unknown feed-forward kind {kind!r}")
        r = m["router"]
        g = r.get("groups") or {}
        shared = m.get("shared") or {}
        return cls(kind="moe", ff=int(m["expert"]["ff"]), experts=int(r["experts"]), identity=int(r.get("identity", 0)),
                   top=int(r["top"]), groups=int(g.get("count", 1)), keep=int(g.get("keep", g.get("count", 1))),
                   shared_ff=int(shared.get("ff", 0) or 0))


@dataclass
class MovolornLayerConfig:
    mixer_type: str
    mixer: AttentionMixerConfig
    mlp: Optional[FeedForwardConfig]


@dataclass
class MovolornConfig:
    """config.json of a Movolorn model: `vocab`, `width`, `embedding.scale`, `norm.eps`, `layers` (each with `type`,
    `mixer`, `mlp`), `loop` (`start`, `stop`, `times`: layers start..stop-1 run `times` times in a row with the same
    weights and a cache of their own per pass)."""
    vocab_size: int
    hidden_size: int
    embedding_scale: float
    rms_norm_eps: float
    layers: List[MovolornLayerConfig]
    loop: Optional[Tuple[int, int, int]] = None
    torch_dtype: Any = torch.bfloat16
    max_position_embeddings: int = 1 << 30      # positions enter through distances only: no table to outgrow
    model_type: str = "movolorn"
    tie_word_embeddings: bool = False
    raw: dict = field(default_factory=dict, repr=False)

    @classmethod
    def from_json(cls, c: dict) -> "MovolornConfig":
        layers = []
        for entry in c["layers"]:
            kind = entry.get("type", "attention")
            if kind != "attention":
                raise ValueError(f"unknown mixer type {kind!r}")
            layers.append(MovolornLayerConfig(kind, AttentionMixerConfig.from_json(entry["mixer"]),
                                              FeedForwardConfig.from_json(entry.get("mlp"))))
        lp = c.get("loop")
        loop = (int(lp["start"]), int(lp["stop"]), int(lp.get("times", 1))) if lp else None
        if loop is not None and not (0 <= loop[0] <= loop[1] <= len(layers) and loop[2] >= 1):
            raise ValueError(f"bad loop {loop} for {len(layers)} layers")
        return cls(vocab_size=int(c["vocab"]), hidden_size=int(c["width"]),
                   embedding_scale=float((c.get("embedding") or {}).get("scale", 1.0)),
                   rms_norm_eps=float((c.get("norm") or {}).get("eps", 1e-6)), layers=layers, loop=loop, raw=c)

    # ---- layer runs: the order in which layers execute, one cache layer per run ----------------------
    @property
    def layer_runs(self) -> List[int]:
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    # ---- the names the cache manager reads from an HF config ----------------------------------------
    @property
    def num_hidden_layers(self) -> int:
        return len(self.layer_runs)

    @property
    def num_key_value_heads(self) -> int:
        return max(l.mixer.kv_heads for l in self.layers)

    @property
    def num_attention_heads(self) -> int:
        return max(l.mixer.heads for l in self.layers)

    @property
    def head_dim(self) -> int:
        return max(l.mixer.dim for l in self.layers)


@dataclass
class LatentAttentionConfig:
    """Attention whose queries and keys/values pass through low-rank latents (layers/latent_attention.py): `heads`
    heads with `dim` unrotated + `rot_dim` rotated query/key numbers and `vdim` values each; the kv latent has
    `kv_rank` numbers, the query latent `q_rank`; `kv_from` names the layer whose cached latent this layer reads
    instead of making its own."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    kv_from: Optional[int] = None

    @classmethod
    def from_json(cls, m: dict) -> "LatentAttentionConfig":
        rot = m.get("rot") or {}
        rot_dim = int(m.get("rot_dim", rot.get("dims", 0)))
        if int(rot.get("dims", rot_dim)) != rot_dim:
            raise ValueError("latent attention rotates its whole rotated part: rot.dims must equal rot_dim")
        if rot_dim % 2:
            raise ValueError(f"rot_dim {rot_dim} is odd")
        dim = int(m["dim"])
        kv_from = m.get("kv_from")
        return cls(heads=int(m["heads"]), dim=dim, rot_dim=rot_dim, vdim=int(m.get("vdim", dim)),
                   kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]),
                   scale=float(m.get("scale", (dim + rot_dim) ** -0.5)), rot_base=float(rot.get("base", 10000.0)),
                   kv_from=None if kv_from is None else int(kv_from))


@dataclass
class StateSpaceConfig:
    """Scalar-decay state-space mixer (layers/ssm.py): `heads` heads of `vdim` channels with `state` state channels,
    B and C shared by the heads of each of `groups` groups, a causal convolution of `conv` taps in front and an RMS
    norm in `norm_groups` equal parts behind."""
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_json(cls, m: dict) -> "StateSpaceConfig":
        c = cls(heads=int(m["heads"]), vdim=int(m["vdim"]), state=int(m["state"]), groups=int(m.get("groups", 1)),
                conv=int(m.get("conv", 4)), norm_groups=int(m.get("norm_groups", 1)))
        if c.heads % c.groups or (c.heads * c.vdim) % c.norm_groups:
            raise ValueError(f"state-space mixer: {c.heads} heads do not split into {c.groups} groups / "
                             f"{c.norm_groups} norm parts")
        return c

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state


@dataclass
class ClampedMoEConfig:
    """Mixture of clamped gated experts (layers/moe.py, ACT_CLAMPED_GLU + ROUTE_TOP_LOGITS): `experts` experts of
    size `ff`, `top` per token chosen by the largest router logits (with a bias), weights = softmax over the chosen;
    a shared expert of size `shared_ff` (0 = none) scaled by the sigmoid of one logit per token."""
    ff: int
    limit: float
    experts: int
    top: int
    shared_ff: int = 0
    shared_limit: float = 0.0

    @classmethod
    def from_json(cls, m: Optional[dict]) -> Optional["ClampedMoEConfig"]:
        if m is None:
            return None
        if m.get("kind", "moe") != "moe":
            raise ValueError(f"unknown feed-forward kind {m.get('kind')!r}")
        shared = m.get("shared") or {}
        return cls(ff=int(m["expert"]["ff"]), limit=float(m["expert"]["limit"]), experts=int(m["router"]["experts"]),
                   top=int(m["router"]["top"]), shared_ff=int(shared.get("ff", 0) or 0),
                   shared_limit=float(shared.get("limit", 0.0) or 0.0))


@dataclass
class BatasunLayerConfig:
    mixer_type: str                     # "latent_attention" | "mamba2"
    mixer: Any                          # LatentAttentionConfig | StateSpaceConfig
    mlp: Optional[ClampedMoEConfig]


@dataclass
class BatasunConfig:
    """config.json of a Batasun model: `vocab`, `width`, `norm.eps`, `layers` (each with `type`, `mixer`, `mlp`).
    Layers are latent-attention or state-space mixers in any order, each followed by a mixture of experts or by
    nothing; norms sit on the sublayers' outputs only and have gains stored around zero."""
    vocab_size: int
    hidden_size: int
    rms_norm_eps: float
    layers: List[BatasunLayerConfig]
    torch_dtype: Any = torch.bfloat16
    max_position_embeddings: int = 1 << 30      # rotation angles are computed from the position: no table to outgrow
    model_type: str = "batasun"
    tie_word_embeddings: bool = False
    raw: dict = field(default_factory=dict, repr=False)

    @classmethod
    def from_json(cls, c: dict) -> "BatasunConfig":
        layers = []
        for i, entry in enumerate(c["layers"]):
            kind = entry["type"]
            if kind == "latent_attention":
                mixer = LatentAttentionConfig.from_json(entry["mixer"])
            elif kind == "mamba2":
                mixer = StateSpaceConfig.from_json(entry["mixer"])
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            layers.append(BatasunLayerConfig(kind, mixer, ClampedMoEConfig.from_json(entry.get("mlp"))))
        for i, lc in enumerate(layers):
            j = lc.mixer.kv_from if lc.mixer_type == "latent_attention" else None
            if j is None:
                continue
            if not (0 <= j < i) or layers[j].mixer_type != "latent_attention" or layers[j].mixer.kv_from is not None:
                raise ValueError(f"layer {i}: kv_from {j} is not an earlier latent-attention layer with a latent of its own")
            a, o = lc.mixer, layers[j].mixer
            if (a.kv_rank, a.rot_dim, a.rot_base) != (o.kv_rank, o.rot_dim, o.rot_base):
                raise ValueError(f"layer {i}: latent sizes differ from layer {j}'s")
        return cls(vocab_size=int(c["vocab"]), hidden_size=int(c["width"]),
                   rms_norm_eps=float((c.get("norm") or {}).get("eps", 1e-6)), layers=layers, raw=c)

    # ---- the names the cache manager and the runner read from an HF config --------------------------
    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def num_key_value_heads(self) -> int:
        return 1                    # the cached latent is shared by all heads

    @property
    def num_attention_heads(self) -> int:
        return max([l.mixer.heads for l in self.layers if l.mixer_type == "latent_attention"] or [1])

    @property
    def head_dim(self) -> int:
        return max([l.mixer.kv_rank + l.mixer.rot_dim for l in self.layers if l.mixer_type == "latent_attention"] or [1])


@dataclass
class RotaryAttentionConfig:
    """Grouped-query attention with biased projections, a rotation of neighbouring pairs on the first `rot_dims`
    numbers of every head (frequencies base ** (-2 i / rot_dims), optionally stretched: `rot_scaling` =
    (factor, low, high, original)), an RMS norm without weight on q and k after the rotation, and a learned softmax
    sink per head."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[Tuple[float, float, float, float]] = None

    @classmethod
    def from_json(cls, m: dict) -> "RotaryAttentionConfig":
        dim = int(m["dim"])
        rot = m.get("rot") or {}
        sc = rot.get("scaling")
        c = cls(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=dim,
                vdim=int(m.get("vdim", dim)), scale=float(m.get("scale", dim ** -0.5)),
                rot_dims=int(rot.get("dims", 0) or 0), rot_base=float(rot.get("base", 10000.0)),
                rot_scaling=None if not sc else (float(sc["factor"]), float(sc["low"]), float(sc["high"]),
                                                 float(sc["original"])))
        if c.heads % c.kv_heads or c.rot_dims % 2 or c.rot_dims > c.dim:
            raise ValueError(f"attention: {c.heads} heads / {c.kv_heads} kv heads, rotation of {c.rot_dims} of {c.dim}")
        return c


@dataclass
class DeltaRuleConfig:
    """Gated delta rule (layers/recurrent.py): `heads` value heads of `vdim`, `kv_heads` query/key heads of `dim`,
    a causal convolution of `conv` taps on q, k and v."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_json(cls, m: dict) -> "DeltaRuleConfig":
        dim = int(m["dim"])
        c = cls(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=dim,
                vdim=int(m.get("vdim", dim)), conv=int(m.get("conv", 4)))
        if c.heads % c.kv_heads or c.conv < 1:
            raise ValueError(f"delta rule: {c.heads} heads / {c.kv_heads} kv heads, {c.conv} taps")
        return c


@dataclass
class WkvConfig:
    """Time mixing with a per-channel decay (layers/recurrent.py): `heads` heads of `dim` key and value channels.
    `decay_rank` (the inner size of the decay's two-step projection) is not part of config.json: a checkpoint's
    tensors give it; the default serves synthetic weights."""
    heads: int
    dim: int
    decay_rank: int = 32

    @classmethod
    def from_json(cls, m: dict) -> "WkvConfig":
        return cls(heads=int(m["heads"]), dim=int(m["dim"]), decay_rank=int(m.get("decay_rank", 32)))


@dataclass
class FafelixLayerConfig:
    mixer_type: str                     # "attention" | "delta" | "wkv"
    mixer: Any                          # RotaryAttentionConfig | DeltaRuleConfig | WkvConfig
    mlp: Optional[FeedForwardConfig]    # dense, or None


@dataclass
class FafelixConfig:
    """config.json of a Fafelix model: `vocab`, `width`, `norm.eps`, `embedding.bigram` (`buckets`, `mul_prev`,
    `mul_cur`), `layers` (each with `type`, `mixer`, `mlp`), `loop` (`start`, `stop`, `times`).  Every layer is
    x += mixer(h) + ff(h) with h = layer_norm(x); the looped span re-adds the embedding before each later pass."""
    vocab_size: int
    hidden_size: int
    rms_norm_eps: float
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: List[FafelixLayerConfig]
    loop: Optional[Tuple[int, int, int]] = None
    torch_dtype: Any = torch.bfloat16
    max_position_embeddings: int = 1 << 30      # rotation angles are computed from the position: no table to outgrow
    model_type: str = "fafelix"
    tie_word_embeddings: bool = False
    raw: dict = field(default_factory=dict, repr=False)

    MIXERS = {"attention": RotaryAttentionConfig, "delta": DeltaRuleConfig, "wkv": WkvConfig}

    @classmethod
    def from_json(cls, c: dict) -> "FafelixConfig":
        layers = []
        for i, entry in enumerate(c["layers"]):
            kind = entry["type"]
            if kind not in cls.MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            ff = entry.get("mlp")
            if ff is not None and ff.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: feed-forward kind {ff.get('kind')!r} is not part of this design")
            mlp = FeedForwardConfig.from_json(ff)
            layers.append(FafelixLayerConfig(kind, cls.MIXERS[kind].from_json(entry["mixer"]), mlp))
        lp = c.get("loop")
        loop = (int(lp["start"]), int(lp["stop"]), int(lp.get("times", 1))) if lp else None
        if loop is not None and not (0 <= loop[0] <= loop[1] <= len(layers) and loop[2] >= 1):
            raise ValueError(f"bad loop {loop} for {len(layers)} layers")
        bg = (c.get("embedding") or {}).get("bigram")
        if not bg:
            raise ValueError("embedding.bigram is missing")
        return cls(vocab_size=int(c["vocab"]), hidden_size=int(c["width"]),
                   rms_norm_eps=float((c.get("norm") or {}).get("eps", 1e-6)), buckets=int(bg["buckets"]),
                   mul_prev=int(bg["mul_prev"]), mul_cur=int(bg["mul_cur"]), layers=layers, loop=loop, raw=c)

    @property
    def layer_runs(self) -> List[Tuple[int, bool]]:
        """(layer, re-add the embedding in front of it) in execution order; the flag marks the first layer of every
        pass of the loop but the first."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, False) for i in range(start)]
        for p in range(times):
            runs += [(i, p > 0 and i == start) for i in range(start, stop)]
        return runs + [(i, False) for i in range(stop, n)]

    # ---- the names the cache manager and the runner read from an HF config --------------------------
    def _attn(self):
        return [l.mixer for l in self.layers if l.mixer_type == "attention"]

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layer_runs)

    @property
    def num_key_value_heads(self) -> int:
        return max([a.kv_heads for a in self._attn()] or [1])

    @property
    def num_attention_heads(self) -> int:
        return max([a.heads for a in self._attn()] or [1])

    @property
    def head_dim(self) -> int:
        return max([a.dim for a in self._attn()] or [1])


@dataclass
class GeneralDeltaConfig:
    """General delta rule (layers/recurrent.py): `heads` heads of `dim` key and value channels, a decay and a removal
    rate per key channel.  `decay_rank` (the inner size of the decay's two-step projection) is not part of
    config.json: a checkpoint's tensors give it; the default serves synthetic weights."""
    heads: int
    dim: int
    decay_rank: int = 16

    @classmethod
    def from_json(cls, m: dict) -> "GeneralDeltaConfig":
        return cls(heads=int(m["heads"]), dim=int(m["dim"]), decay_rank=int(m.get("decay_rank", 16)))


@dataclass
class WindowAttentionConfig:
    """Grouped-query attention without rotation: a sliding window of `window` positions (0 = none), a learned bias per
    distance bucket (a table of `bias_rows` rows per head - a checkpoint's tensor gives the count -, exact distances
    below half of it, logarithmic buckets up to `bias_max`) and a learned softmax sink per head."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    bias_max: int
    bias_rows: int = 16

    @classmethod
    def from_json(cls, m: dict) -> "WindowAttentionConfig":
        dim = int(m["dim"])
        c = cls(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=dim,
                vdim=int(m.get("vdim", dim)), scale=float(m.get("scale", dim ** -0.5)),
                window=int((m.get("mask") or {}).get("size", 0) or 0), bias_max=int(m["bias_max"]),
                bias_rows=int(m.get("bias_rows", 16)))
        if c.heads % c.kv_heads or c.window < 0 or c.bias_max < 2:
            raise ValueError(f"attention: {c.heads} heads / {c.kv_heads} kv heads, window {c.window}, bias_max {c.bias_max}")
        return c


@dataclass
class MatrixMemoryConfig:
    """Matrix memory with exponential gates (layers/recurrent.py): `heads` heads of `dim` key and `vdim` value
    channels; the log gates are capped at +-`gate_cap` by a tanh."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_json(cls, m: dict) -> "MatrixMemoryConfig":
        dim = int(m["dim"])
        c = cls(heads=int(m["heads"]), dim=dim, vdim=int(m.get("vdim", dim)), gate_cap=float(m["gate_cap"]))
        if c.gate_cap <= 0:
            raise ValueError(f"matrix memory: gate_cap {c.gate_cap}")
        return c


@dataclass
class ParallelMixerConfig:
    """Two mixers side by side on one input: windowed attention (`left`) and a matrix memory (`right`)."""
    left: WindowAttentionConfig
    right: MatrixMemoryConfig

    @classmethod
    def from_json(cls, m: dict) -> "ParallelMixerConfig":
        return cls(WindowAttentionConfig.from_json(m["left"]), MatrixMemoryConfig.from_json(m["right"]))


@dataclass
class SelectiveScanConfig:
    """State-space mixer with a decay per (channel, state channel) (layers/ssm.py): `inner` channels with `state` state
    channels each, step sizes through a projection of rank `dt_rank`, a causal convolution of `conv` taps in front."""
    inner: int
    state: int
    dt_rank: int
    conv: int

    @classmethod
    def from_json(cls, m: dict) -> "SelectiveScanConfig":
        c = cls(inner=int(m["inner"]), state=int(m["state"]), dt_rank=int(m["dt_rank"]), conv=int(m.get("conv", 4)))
        if min(c.inner, c.state, c.dt_rank, c.conv) < 1:
            raise ValueError(f"selective scan: {c}")
        return c


@dataclass
class ScaledMoEConfig:
    """kind "dense": down(relu(up h + b)^2) + b.  kind "moe": `experts` silu-gated experts of size `ff`, `top` per token
    by the largest sigmoid(router logit); the weight (that sigmoid, not renormalized) multiplies the expert's INPUT; a
    shared expert of size `shared_ff` (0 = none) is added, scaled by the sigmoid of one logit per token."""
    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    shared_ff: int = 0

    @classmethod
    def from_json(cls, m: Optional[dict]) -> Optional["ScaledMoEConfig"]:
        if m is None:
            return None
        kind = m.get("kind", "dense")
        if kind == "dense":
            return cls(kind="dense", ff=int(m["ff"]))
        if kind != "moe":
            raise ValueError(f"unknown feed-forward kind {kind!r}")
        shared = m.get("shared") or {}
        c = cls(kind="moe", ff=int(m["expert"]["ff"]), experts=int(m["router"]["experts"]), top=int(m["router"]["top"]),
                shared_ff=int(shared.get("ff", 0) or 0))
        if not 1 <= c.top <= c.experts:
            raise ValueError(f"mixture of experts: top {c.top} of {c.experts}")
        return c


@dataclass
class NununexLayerConfig:
    mixer_type: str                     # "general_delta" | "parallel" | "mamba1"
    mixer: Any                          # GeneralDeltaConfig | ParallelMixerConfig | SelectiveScanConfig
    mlp: Optional[ScaledMoEConfig]


@dataclass
class NununexConfig:
    """config.json of a Nununex model: `vocab`, `width`, `norm.eps`, `canon.taps`, `logit_softcap`,
    `embedding.bigram` (`buckets`, `mul_prev`, `mul_cur`), `layers` (each with `type`, `mixer`, `mlp`).  Every sublayer
    is x += sigmoid(W_rg h + b) * sublayer(h + causal_conv(h)) with h = rms_norm(x); the logits pass a tanh cap."""
    vocab_size: int
    hidden_size: int
    rms_norm_eps: float
    canon_taps: int
    logit_softcap: float                # 0 = none
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: List[NununexLayerConfig]
    torch_dtype: Any = torch.bfloat16
    max_position_embeddings: int = 1 << 30      # positions enter through distances only: no table to outgrow
    model_type: str = "nununex"
    tie_word_embeddings: bool = False
    raw: dict = field(default_factory=dict, repr=False)

    MIXERS = {"general_delta": GeneralDeltaConfig, "parallel": ParallelMixerConfig, "mamba1": SelectiveScanConfig}

    @classmethod
    def from_json(cls, c: dict) -> "NununexConfig":
        layers = []
        for i, entry in enumerate(c["layers"]):
            kind = entry["type"]
            if kind not in cls.MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            layers.append(NununexLayerConfig(kind, cls.MIXERS[kind].from_json(entry["mixer"]),
                                             ScaledMoEConfig.from_json(entry.get("mlp"))))
        bg = (c.get("embedding") or {}).get("bigram")
        if not bg:
            raise ValueError("embedding.bigram is missing")
        taps = int((c.get("canon") or {}).get("taps", 1))
        if taps < 1:
            raise ValueError(f"canon.taps {taps}")
        return cls(vocab_size=int(c["vocab"]), hidden_size=int(c["width"]),
                   rms_norm_eps=float((c.get("norm") or {}).get("eps", 1e-6)), canon_taps=taps,
                   logit_softcap=float(c.get("logit_softcap", 0.0) or 0.0), buckets=int(bg["buckets"]),
                   mul_prev=int(bg["mul_prev"]), mul_cur=int(bg["mul_cur"]), layers=layers, raw=c)

    # ---- the names the cache manager and the runner read from an HF config --------------------------
    def _attn(self):
        return [l.mixer.left for l in self.layers if l.mixer_type == "parallel"]

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def num_key_value_heads(self) -> int:
        return max([a.kv_heads for a in self._attn()] or [1])

    @property
    def num_attention_heads(self) -> int:
        return max([a.heads for a in self._attn()] or [1])

    @property
    def head_dim(self) -> int:
        return max([a.dim for a in self._attn()] or [1])


ARCHITECTURES = {"Movolorn": MovolornConfig, "Batasun": BatasunConfig, "Fafelix": FafelixConfig,
                 "Nununex": NununexConfig}


def load_model_config(path: str):
    """config.json of `path` -> a config object; designs of ARCHITECTURES are parsed here, the rest by transformers."""
    cfg_file = os.path.join(path, "config.json")
    if os.path.isfile(cfg_file):
        with open(cfg_file) as f:
            raw = json.load(f)
        arch = raw.get("architecture")
        if isinstance(arch, str) and arch in ARCHITECTURES:
            return ARCHITECTURES[arch].from_json(raw)
    from transformers import AutoConfig

    return AutoConfig.from_pretrained(path)
