"""Token embedding and output head. Embedding is a row copy (src/gpu/cuda/shaders/embed.cu:24-59),
times `scale` for designs that scale it (1 otherwise; a head tied to the table uses the table itself); the head is final norm, then a product with
`lm_head.weight`, or with the embedding table when the two are tied
(src/model/primitives.rs:124-143, 1467; src/model/loader/mod.rs:693-702). Logits are
float32 and are computed only for the rows that were asked for."""
from __future__ import annotations

from .base import Param, Part, Source, StateSpec, register_part


class Embedding(Part):
    graph_safe = True

    def __init__(self, vocab: int, hidden: int, name: str = "embed_tokens.weight", scale: float = 1.0):
        self.vocab, self.hidden, self.name, self.scale = vocab, hidden, name, float(scale)
        self.table = None

    def params(self):
        return [Param("table", (Source(self.name, (self.vocab, self.hidden)),))]

    def forward(self, ctx):
        if self.scale == 1.0:
            return ctx.backend.embed(ctx.token_ids, self.table, err=ctx.extras.get("err_flag"))
        return ctx.backend.embed(ctx.token_ids, self.table, err=ctx.extras.get("err_flag"), scale=self.scale)


class OutputHead(Part):
    """`tied_to`: the Embedding whose table doubles as the output matrix, or None."""
    graph_safe = True

    def __init__(self, vocab: int, hidden: int, norm: Part, tied_to: Embedding | None,
                 name: str = "weight"):
        self.vocab, self.hidden, self.norm, self.tied_to, self.name = vocab, hidden, norm, tied_to, name
        self.weight = None

    def children(self):
        return [self.norm]

    def params(self):
        if self.tied_to is not None:
            return []
        return [Param("weight", (Source(self.name, (self.vocab, self.hidden)),))]

    def matrix(self):
        return self.tied_to.table if self.tied_to is not None else self.weight

    def forward(self, h, rows, ctx):
        """h: float32 [T, hidden]; rows: int32 device vector of the wanted rows -> [R, vocab]."""
        if hasattr(self.norm, "deferred"):
            n = self.norm.deferred(h, ctx, rows)      # gather, norm and product may be one kernel
        else:
            n = self.norm.forward(ctx.backend.gather_rows(h, rows), ctx)
        return ctx.backend.linear_f32(n, self.matrix())


register_part("embedding", "table", Embedding)
register_part("head", "linear", OutputHead)


class PairEmbedding(Part):
    """Token embedding plus a row of a second table addressed by a hash of the token and the one before it in its
    sequence, (previous * mul_prev + token * mul_cur) mod buckets; a sequence's first token takes row `buckets` (the
    table has buckets + 1 rows). The sum is RMS-normed with a weight (`norm_name`; None: no norm) and returned as the
    float stream. The token before a portion's first one is per-request state (`StateSpec`, one int32), so a prompt
    may be cut anywhere. `pair_name` None: the plain table, normed."""
    graph_safe = True

    def __init__(self, vocab: int, hidden: int, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0, eps: float = 1e-6,
                 name: str = "embed", pair_name: str | None = "bigram", norm_name: str | None = "embed.norm"):
        self.vocab, self.hidden, self.buckets, self.mul_prev, self.mul_cur = vocab, hidden, buckets, mul_prev, mul_cur
        self.eps, self.name, self.pair_name, self.norm_name = float(eps), name, pair_name, norm_name
        if pair_name is not None and buckets <= 0:
            raise ValueError("a pair table needs a positive number of buckets")
        self.table = self.pair = self.norm_w = None

    def params(self):
        ps = [Param("table", (Source(self.name, (self.vocab, self.hidden)),))]
        if self.pair_name is not None:
            ps.append(Param("pair", (Source(self.pair_name, (self.buckets + 1, self.hidden)),)))
        if self.norm_name is not None:
            ps.append(Param("norm_w", (Source(self.norm_name, (self.hidden,), init="norm"),), role="vector"))
        return ps

    def cache_spec(self):
        import torch
        return None if self.pair_name is None else StateSpec((("prev", (), torch.int32),))

    def finalize(self, device, dtype):
        self._norm = None if self.norm_w is None else self.norm_w.float().contiguous()

    def forward(self, ctx, cache=None):
        return ctx.backend.pair_embed(ctx, self.table, self.pair, self.buckets, self.mul_prev, self.mul_cur, self._norm,
                                      self.eps, None if cache is None else cache.state["prev"])


register_part("embedding", "pair", PairEmbedding)
