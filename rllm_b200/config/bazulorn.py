"""Typed configuration of the Bazulorn design, read from its own config.json keys.

A Bazulorn model is a list of layers whose two sublayers read one normed input, x <- x + (mixer(n) + ff(n)) with
n = norm1(x). The mixer is either `parallel`: grouped-query attention without rotation (biased projections, values
normed per head, a sliding window, a sink of score 0 in the softmax, the heads' weights mixed by a matrix) beside a
state-space recurrence with a short convolution, each output RMS-normed and the two averaged; or `channel_delta`: a
gated delta rule with a decay per key channel. The feed-forward is dense (gelu in its tanh form times a linear half),
a mixture of clamped gated experts with an optional shared expert, or absent. The embedding adds a row of a second
table addressed by a hash of the token and the one before it, and is normed. config.json gives every size and every
constant that can differ between models; nothing here assumes a value. Keys:

    architecture            "Bazulorn"
    vocab, width            sizes of the embedding table (also the output matrix)
    embedding.bigram        absent, or {buckets, mul_prev, mul_cur}
    norm.eps                eps of every RMS norm
    layers[i].type          "parallel" or "channel_delta"
    layers[i].mixer         parallel: {left {heads, kv_heads, dim, vdim, scale, mask {size} or absent},
                                       right {heads, vdim, state, groups, norm_groups, conv}}
                            channel_delta: {heads, kv_heads, dim, vdim, conv; optionally decay_rank and gate_rank,
                            which a checkpoint's tensors give otherwise}
    layers[i].mlp           null, {kind "dense", ff}, or {kind "moe", expert {ff, limit}, router {experts, top},
                            shared {ff, limit} or absent}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError, ModelConfig, require_float, require_int


def _obj(raw: dict, key: str, where: str, optional: bool = False):
    v = raw.get(key)
    if v is None:
        if optional:
            return None
        raise ConfigError(f"{where} lacks required key {key!r}")
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {key!r} must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class TalkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int                      # query/key size per head
    vdim: int                     # value size per head
    scale: float                  # factor on the scores
    window: int | None = None     # a query sees itself and the window - 1 positions before it; None: all

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "TalkAttentionConfig":
        mask = _obj(m, "mask", where, optional=True)
        c = cls(require_int(m, "heads"), require_int(m, "kv_heads"), require_int(m, "dim"), require_int(m, "vdim"),
                require_float(m, "scale"), None if mask is None else require_int(mask, "size"))
        if c.heads % c.kv_heads:
            raise ConfigError(f"{where}: {c.heads} heads do not divide over {c.kv_heads} kv_heads")
        return c

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int                     # channels per head
    state: int                    # state rows per head
    groups: int                   # heads share the input and output vectors of the state in this many groups
    norm_groups: int              # the gated output is normed in this many equal parts
    conv: int                     # taps of the short convolution

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "StateSpaceConfig":
        c = cls(require_int(m, "heads"), require_int(m, "vdim"), require_int(m, "state"), require_int(m, "groups"),
                require_int(m, "norm_groups"), require_int(m, "conv"))
        if c.heads % c.groups:
            raise ConfigError(f"{where}: {c.heads} heads do not divide over {c.groups} groups")
        if (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"{where}: {c.heads * c.vdim} channels do not form {c.norm_groups} equal parts")
        return c

    def to_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                "norm_groups": self.norm_groups, "conv": self.conv}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: TalkAttentionConfig
    right: StateSpaceConfig

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "ParallelMixerConfig":
        return cls(TalkAttentionConfig.from_dict(_obj(m, "left", where), where + ".left"),
                   StateSpaceConfig.from_dict(_obj(m, "right", where), where + ".right"))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class DeltaRuleConfig:
    heads: int                    # value heads (one state each)
    kv_heads: int                 # query/key heads, shared by groups of value heads
    dim: int                      # key channels per head
    vdim: int
    conv: int                     # taps of the short convolutions
    decay_rank: int | None = None     # rows of the decay's first projection; None: the checkpoint's tensor says
    gate_rank: int | None = None      # rows of the output gate's first projection; None: likewise

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "DeltaRuleConfig":
        c = cls(require_int(m, "heads"), require_int(m, "kv_heads"), require_int(m, "dim"), require_int(m, "vdim"),
                require_int(m, "conv"), None if m.get("decay_rank") is None else require_int(m, "decay_rank"),
                None if m.get("gate_rank") is None else require_int(m, "gate_rank"))
        if c.heads % c.kv_heads:
            raise ConfigError(f"{where}: {c.heads} heads do not divide over {c.kv_heads} kv_heads")
        return c

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.decay_rank is not None:
            d["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            d["gate_rank"] = self.gate_rank
        return d


@dataclass(frozen=True)
class BazulornMLP:
    kind: str                     # "dense" or "moe"
    ff: int                       # inner size (of one expert for "moe")
    limit: float = 0.0            # clamp of an expert's gate and linear halves
    experts: int = 0
    top: int = 0
    shared_ff: int | None = None  # inner size of the expert every token uses; None: there is none
    shared_limit: float = 0.0

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "BazulornMLP":
        kind = m.get("kind")
        if kind == "dense":
            return cls("dense", require_int(m, "ff"))
        if kind == "moe":
            expert, router = _obj(m, "expert", where), _obj(m, "router", where)
            shared = _obj(m, "shared", where, optional=True)
            c = cls("moe", require_int(expert, "ff"), require_float(expert, "limit"), require_int(router, "experts"),
                    require_int(router, "top"), None if shared is None else require_int(shared, "ff"),
                    0.0 if shared is None else require_float(shared, "limit"))
            if c.top > c.experts:
                raise ConfigError(f"{where}: top {c.top} exceeds the {c.experts} experts")
            return c
        raise ConfigError(f"{where}: feed-forward kind {kind!r} is not known (known: 'dense', 'moe')")

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                             "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return d


@dataclass(frozen=True)
class BigramConfig:
    buckets: int
    mul_prev: int
    mul_cur: int

    @classmethod
    def from_dict(cls, m: dict) -> "BigramConfig":
        return cls(require_int(m, "buckets"), require_int(m, "mul_prev", minimum=0), require_int(m, "mul_cur", minimum=0))

    def to_dict(self) -> dict:
        return {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}


MIXER_CONFIGS = {"parallel": ParallelMixerConfig, "channel_delta": DeltaRuleConfig}


@dataclass(frozen=True)
class BazulornLayer:
    type: str
    mixer: Any
    mlp: BazulornMLP | None


@dataclass(frozen=True)
class BazulornConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    bigram: BigramConfig | None = None
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "BazulornConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in MIXER_CONFIGS:
                raise ConfigError(f"{where}: 'type' must be one of {sorted(MIXER_CONFIGS)}, got "
                                  f"{L.get('type') if isinstance(L, dict) else L!r}")
            mixer = MIXER_CONFIGS[L["type"]].from_dict(_obj(L, "mixer", where), where + ".mixer")
            mlp = L.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"{where}: 'mlp' must be an object or null")
            layers.append(BazulornLayer(L["type"], mixer, None if mlp is None else BazulornMLP.from_dict(mlp, where + ".mlp")))
        emb = _obj(raw, "embedding", "config.json", optional=True)
        bigram = None if emb is None else _obj(emb, "bigram", "embedding", optional=True)
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (eos,)
        return cls(require_int(raw, "vocab"), require_int(raw, "width"),
                   require_float(_obj(raw, "norm", "config.json"), "eps"), tuple(layers),
                   None if bigram is None else BigramConfig.from_dict(bigram), tuple(int(e) for e in eos))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": "Bazulorn", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [{"type": L.type, "mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict()}
                       for L in self.layers]}
        if self.bigram is not None:
            d["embedding"] = {"bigram": self.bigram.to_dict()}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
