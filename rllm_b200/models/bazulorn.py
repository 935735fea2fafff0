"""Bazulorn assembled from parts: layers with one norm whose output the mixer and the feed-forward both read. The
mixer is attention with mixed heads beside a state-space recurrence (`parallel`: two cache layers, pages and a state),
or a gated delta rule (`channel_delta`: a state); the feed-forward is dense, a mixture of clamped gated experts with
an optional shared expert, or absent. The embedding adds a row addressed by a hash of each token and the one before
it and is normed; it keeps the last token of every request. Tensor names: `embed`, `bigram`, `embed.norm`,
`l<i>.norm1`, `l<i>.mix.*` (`left.*`, `right.*` for a parallel mixer), `l<i>.mlp.*`, `final.norm`; the output matrix
is the embedding table. Everything numeric that can differ between models comes from the configuration."""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.bazulorn import BazulornConfig
from ..parts import (DeltaRuleMixer, GluFFN, GluRoutedExperts, PairEmbedding, ParallelBlock, RMSNorm, SideBySideMixer,
                     StateSpaceMixer, TalkingHeadsAttention, make_part)
from .model import LayerCall, Model

SWISH_ALPHA = 1.702       # the experts' gate is g * sigmoid(1.702 g)
UNIT_EPS = 1e-6           # inside the root of the delta rule's unit vectors


def _mixer(cfg: BazulornConfig, layer):
    m, W, eps = layer.mixer, cfg.width, cfg.norm_eps
    if layer.type == "parallel":
        a, r = m.left, m.right
        left = TalkingHeadsAttention(W, a.heads, a.kv_heads, a.dim, a.vdim, scale=a.scale, window=a.window, bias=True,
                                     value_norm=True, sink=0.0, eps=eps)
        right = StateSpaceMixer(W, r.heads, r.vdim, r.state, r.groups, r.norm_groups, r.conv, eps=eps)
        return SideBySideMixer(W, left, right, coef=0.5, eps=eps)
    if layer.type == "channel_delta":
        return DeltaRuleMixer(W, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, eps=eps, unit_eps=UNIT_EPS,
                              decay_rank=m.decay_rank, gate_rank=m.gate_rank)
    raise ValueError(f"no mixer for layer type {layer.type!r}")


def _ffn(cfg: BazulornConfig, f):
    if f.kind == "dense":
        return GluFFN(cfg.width, f.ff, "gelu_tanh")
    shared = None if f.shared_ff is None else GluFFN(cfg.width, f.shared_ff, "swish_clamped", f.shared_limit, SWISH_ALPHA)
    return GluRoutedExperts(cfg.width, f.ff, f.experts, f.top, "swish_clamped", f.limit, SWISH_ALPHA,
                            score="softmax_chosen", router_bias=True, shared=shared)


def build_bazulorn(cfg: BazulornConfig) -> Model:
    W, eps = cfg.width, cfg.norm_eps
    b = cfg.bigram
    emb = PairEmbedding(cfg.vocab, W, eps=eps, name="embed", norm_name="embed.norm",
                        **({"pair_name": None} if b is None else
                           {"pair_name": "bigram", "buckets": b.buckets, "mul_prev": b.mul_prev, "mul_cur": b.mul_cur}))
    emb.prefix = ""
    blocks, schedule, cache_layer = [], [], 0
    for i, layer in enumerate(cfg.layers):
        block = ParallelBlock(RMSNorm(W, eps, "norm1"), _mixer(cfg, layer), None if layer.mlp is None else _ffn(cfg, layer.mlp))
        block.set_prefix(f"l{i}.")
        blocks.append(block)
        if layer.type == "parallel":            # pages for the attention, a state for the recurrence
            schedule.append(LayerCall(i, (cache_layer, cache_layer + 1), True))
            cache_layer += 2
        else:
            schedule.append(LayerCall(i, cache_layer, True))
            cache_layer += 1
    final_norm = RMSNorm(W, eps, "norm")
    final_norm.prefix = "final."
    head = make_part("head", "linear", vocab=cfg.vocab, hidden=W, norm=final_norm, tied_to=emb)
    head.prefix = ""
    return Model(cfg, emb, blocks, schedule, head, prefix="")


register_architecture("Bazulorn", BazulornConfig, build_bazulorn, model_types=("bazulorn",))
