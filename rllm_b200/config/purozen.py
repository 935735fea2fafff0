"""Typed configuration of the Purozen design, read from its own config.json keys.

A Purozen model is a list of pre-norm layers whose sublayers are gated into the stream:
x <- x + sigmoid(W_1 n + b_1) * mixer(n) with n = norm1(x), then the same with norm2 and the feed-forward (which may be
absent). Norm weights are stored around zero (the factor is 1 + w). A layer's mixer is one of three kinds. `parallel`:
grouped-query attention without rotation and without softmax (a visible key's weight is the sigmoid of its score plus
a number per head) beside a gated recurrence whose gates read only the current token, the two added with a
coefficient each. `attention`: grouped-query attention with a rotation of part of each head (every frequency
optionally divided by a factor), queries and keys brought to root mean square 1, a sliding window that keeps the
first tokens visible, and optionally the values mixed with those of the first layer that says so. `latent_attention`:
attention over a cached latent per token, without positions. The feed-forward is W_down gelu_tanh(W_up n). config.json
gives every size and every constant that can differ between models; nothing here assumes a value. Keys:

    architecture            "Purozen"
    vocab, width            sizes of the embedding table (also the output matrix)
    norm.eps                eps of every RMS norm
    layers[i].type          "parallel", "attention" or "latent_attention"
    layers[i].mixer         parallel: {left {heads, kv_heads, dim, vdim, scale}, right {width}, left_scale, right_scale}
                            attention: {heads, kv_heads, dim, vdim, scale; optionally mask {size, keep_first},
                                        rot {base, dims, scaling {factor}}, v_mix}
                            latent_attention: {heads, dim, vdim, kv_rank, scale}
    layers[i].mlp           null, or {kind "dense", ff}
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


def _heads(m: dict, where: str):
    heads, kv = require_int(m, "heads"), require_int(m, "kv_heads")
    if heads % kv:
        raise ConfigError(f"{where}: {heads} heads do not divide over {kv} kv_heads")
    return heads, kv


@dataclass(frozen=True)
class SigmoidAttentionConfig:
    heads: int
    kv_heads: int
    dim: int                      # query/key size per head
    vdim: int                     # value size per head
    scale: float                  # factor on the scores

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "SigmoidAttentionConfig":
        heads, kv = _heads(m, where)
        return cls(heads, kv, require_int(m, "dim"), require_int(m, "vdim"), require_float(m, "scale"))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}


@dataclass(frozen=True)
class PurozenParallelConfig:
    left: SigmoidAttentionConfig
    right_width: int              # channels of the recurrence
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "PurozenParallelConfig":
        return cls(SigmoidAttentionConfig.from_dict(_obj(m, "left", where), where + ".left"),
                   require_int(_obj(m, "right", where), "width"), require_float(m, "left_scale"),
                   require_float(m, "right_scale"))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": {"width": self.right_width}, "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None = None         # a query sees itself and the window - 1 positions before it; None: all
    keep_first: int = 0               # and, whatever the window, the positions below this number
    rot_dims: int = 0                 # leading dimensions of a head that are rotated; 0: no rotation
    rot_base: float = 10000.0
    rot_factor: float | None = None   # every frequency is divided by it; None: no scaling
    v_mix: bool = False

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "WindowAttentionConfig":
        heads, kv = _heads(m, where)
        mask, rot = _obj(m, "mask", where, optional=True), _obj(m, "rot", where, optional=True)
        window = keep = None
        if mask is not None:
            window = require_int(mask, "size")
            keep = require_int(mask, "keep_first", minimum=0, default=0)
        dims, base, factor = 0, 10000.0, None
        if rot is not None:
            dims, base = require_int(rot, "dims", minimum=0), require_float(rot, "base")
            scaling = _obj(rot, "scaling", where + ".rot", optional=True)
            if scaling is not None:
                factor = require_float(scaling, "factor")
                if factor <= 0:
                    raise ConfigError(f"{where}.rot.scaling: factor must be > 0, got {factor}")
        v_mix = m.get("v_mix", False)
        if not isinstance(v_mix, bool):
            raise ConfigError(f"{where}: 'v_mix' must be true or false, got {v_mix!r}")
        c = cls(heads, kv, require_int(m, "dim"), require_int(m, "vdim"), require_float(m, "scale"), window, keep or 0,
                dims, base, factor, v_mix)
        if c.rot_dims % 2 or c.rot_dims > c.dim:
            raise ConfigError(f"{where}.rot: {c.rot_dims} rotated dimensions must be even and at most dim {c.dim}")
        return c

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_factor is not None:
                d["rot"]["scaling"] = {"factor": self.rot_factor}
        if self.v_mix:
            d["v_mix"] = True
        return d


@dataclass(frozen=True)
class PlainLatentConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "PlainLatentConfig":
        return cls(require_int(m, "heads"), require_int(m, "dim"), require_int(m, "vdim"), require_int(m, "kv_rank"),
                   require_float(m, "scale"))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "scale": self.scale}


MIXER_CONFIGS = {"parallel": PurozenParallelConfig, "attention": WindowAttentionConfig,
                 "latent_attention": PlainLatentConfig}


@dataclass(frozen=True)
class PurozenLayer:
    type: str
    mixer: Any
    ff: int | None                # inner size of the dense feed-forward; None: the layer has none


@dataclass(frozen=True)
class PurozenConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "PurozenConfig":
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
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"{where}: 'mlp' must be an object or null")
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp: feed-forward kind {mlp.get('kind')!r} is not known (known: 'dense')")
                ff = require_int(mlp, "ff")
            layers.append(PurozenLayer(L["type"], mixer, ff))
        mixed = [L.mixer for L in layers if L.type == "attention" and L.mixer.v_mix]
        if len({(m.kv_heads, m.vdim) for m in mixed}) > 1:
            raise ConfigError("layers that mix their values with the first such layer's must agree in kv_heads and vdim")
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (eos,)
        return cls(require_int(raw, "vocab"), require_int(raw, "width"),
                   require_float(_obj(raw, "norm", "config.json"), "eps"), tuple(layers), tuple(int(e) for e in eos))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": "Purozen", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [{"type": L.type, "mixer": L.mixer.to_dict(),
                        "mlp": None if L.ff is None else {"kind": "dense", "ff": L.ff}} for L in self.layers]}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
