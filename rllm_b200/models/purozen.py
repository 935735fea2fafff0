"""Purozen assembled from parts: pre-norm layers whose sublayers are gated into the stream (`GatedPreNormBlock`), norm
weights stored around zero. The mixer is sigmoid-weighted attention beside a gated recurrence (`parallel`: two cache
layers, pages and a state), windowed attention that keeps the first tokens visible (`attention`: pages, those of the
kept tokens never given back), or attention over cached latents without positions (`latent_attention`); the
feed-forward is dense with gelu in its tanh form, or absent. Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`,
`l<i>.rg1`, `l<i>.rg2` (with `.b`), `l<i>.mix.*` (`left.*`, `right.*` for a parallel mixer), `l<i>.mlp.*`,
`final.norm`; the output matrix is the embedding table. Everything numeric that can differ between models comes from
the configuration."""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.llama import RopeScaling
from ..config.purozen import PurozenConfig
from ..parts import (ActFFN, Embedding, GatedPreNormBlock, LatentAttention, MinGRUMixer, RMSNorm, RotaryEmbedding,
                     SideBySideMixer, SinkGQAttention, make_part)
from .model import LayerCall, Model

NORM_OFFSET = 1.0         # a norm's factor is 1 + the stored weight


def _mixer(cfg: PurozenConfig, layer, first_mixed: bool):
    m, W, eps = layer.mixer, cfg.width, cfg.norm_eps
    if layer.type == "parallel":
        a = m.left
        left = SinkGQAttention(W, a.heads, a.kv_heads, a.dim, a.vdim, scale=a.scale, weights="sigmoid", score_bias="pb")
        return SideBySideMixer(W, left, MinGRUMixer(W, m.right_width), scales=(m.left_scale, m.right_scale))
    if layer.type == "attention":
        position = None
        if m.rot_dims:
            scaling = None if m.rot_factor is None else RopeScaling(rope_type="linear", factor=m.rot_factor)
            position = RotaryEmbedding(m.dim, m.rot_base, scaling, rot_dim=m.rot_dims)
        mix = None if not m.v_mix else ("first" if first_mixed else "mix", "v_mix")
        return SinkGQAttention(W, m.heads, m.kv_heads, m.dim, m.vdim, position=position, scale=m.scale, window=m.window,
                               qk_norm=True, qk_norm_weight=False, eps=eps, keep_first=m.keep_first, value_mix=mix)
    if layer.type == "latent_attention":
        return LatentAttention(W, m.heads, m.dim, 0, m.vdim, m.kv_rank, m.scale, None, eps=eps, gate=False)
    raise ValueError(f"no mixer for layer type {layer.type!r}")


def build_purozen(cfg: PurozenConfig) -> Model:
    W, eps = cfg.width, cfg.norm_eps
    emb = Embedding(cfg.vocab, W, name="embed")
    emb.prefix = ""
    blocks, schedule, cache_layer, mixed_seen = [], [], 0, False
    for i, layer in enumerate(cfg.layers):
        mixes = layer.type == "attention" and layer.mixer.v_mix
        mixer = _mixer(cfg, layer, mixes and not mixed_seen)
        mixed_seen = mixed_seen or mixes
        ffn = None if layer.ff is None else ActFFN(W, layer.ff, "gelu_tanh")
        block = GatedPreNormBlock(W, RMSNorm(W, eps, "norm1", NORM_OFFSET), mixer,
                                  None if ffn is None else RMSNorm(W, eps, "norm2", NORM_OFFSET), ffn)
        block.set_prefix(f"l{i}.")
        blocks.append(block)
        if layer.type == "parallel":            # pages for the attention, a state for the recurrence
            schedule.append(LayerCall(i, (cache_layer, cache_layer + 1), True))
            cache_layer += 2
        else:
            schedule.append(LayerCall(i, cache_layer, True))
            cache_layer += 1
    final_norm = RMSNorm(W, eps, "norm", NORM_OFFSET)
    final_norm.prefix = "final."
    head = make_part("head", "linear", vocab=cfg.vocab, hidden=W, norm=final_norm, tied_to=emb)
    head.prefix = ""
    return Model(cfg, emb, blocks, schedule, head, prefix="")


register_architecture("Purozen", PurozenConfig, build_purozen, model_types=("purozen",))
