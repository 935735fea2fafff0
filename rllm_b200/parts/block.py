"""How a layer's parts are arranged. Pre-norm residual block, the reference's Llama layer
order (src/model/registry/llama.rs:163-245): h += mixer(norm(h)); h += ffn(norm(h)).
`SandwichBlock` norms each sublayer's output as well: h += norm_b(mixer(norm(h))), the same for
the feed-forward, which may be absent. `LoopStep` is a block that only adds a learned vector to
every row: what a pass of a looped stretch of layers begins with. `PostNormBlock` norms after the sum,
h = norm(alpha h + sublayer(h)), the sublayers reading the stream itself. `ParallelBlock` has one norm whose
output both sublayers read: h += mixer(n) + ffn(n), n = norm(h). `GatedPreNormBlock` is the pre-norm order with a
gate on each sublayer's way into the stream: h += sigmoid(W_g n + b_g) * sublayer(n), n = norm(h), W_g a square matrix."""
from __future__ import annotations

from .base import Param, Part, Source, register_part


class PreNormBlock(Part):
    """`names` maps the four parts to their checkpoint sub-prefixes."""
    graph_safe = True

    def __init__(self, mixer_norm: Part, mixer: Part, ffn_norm: Part, ffn: Part,
                 names=("input_layernorm.", "self_attn.", "post_attention_layernorm.", "mlp.")):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.names = names

    def children(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def set_prefix(self, prefix: str):
        self.prefix = prefix
        for part, sub in zip(self.children(), self.names):
            part.prefix = prefix + sub
            for c in part.children():
                if not c.prefix:
                    c.prefix = part.prefix

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, h, ctx, cache):
        """h: float32 residual stream [T, hidden], updated in place."""
        self.mixer.forward(self._norm(self.mixer_norm, self.mixer, h, ctx), ctx, cache, h)
        self.ffn.forward(self._norm(self.ffn_norm, self.ffn, h, ctx), ctx, h)
        return h

    @staticmethod
    def _norm(norm, consumer, h, ctx):
        """A consumer that hands its input straight to the backend's products (`takes_deferred`)
        gets the norm in deferred form, so that it can run inside the first product."""
        if getattr(consumer, "takes_deferred", False) and hasattr(norm, "deferred"):
            return norm.deferred(h, ctx)
        return norm.forward(h, ctx)


class SandwichBlock(Part):
    """A norm before and after each sublayer. The post-norm, the sum over a routed feed-forward's
    parts and the residual sum are one float kernel. `names`: checkpoint sub-prefixes of mixer and
    feed-forward; the four norms' weights are tensors named `norm_names` under the block's prefix."""
    graph_safe = True

    def __init__(self, mixer_norm: Part, mixer: Part, mixer_post: Part, ffn_norm: Part | None = None,
                 ffn: Part | None = None, ffn_post: Part | None = None, names=("mix.", "mlp.")):
        self.mixer_norm, self.mixer, self.mixer_post = mixer_norm, mixer, mixer_post
        self.ffn_norm, self.ffn, self.ffn_post = ffn_norm, ffn, ffn_post
        self.names = names

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_post, self.ffn_norm, self.ffn, self.ffn_post)
                if p is not None]

    def set_prefix(self, prefix: str):
        self.prefix = prefix
        for norm in (self.mixer_norm, self.mixer_post, self.ffn_norm, self.ffn_post):
            if norm is not None:
                norm.prefix = prefix            # a norm's tensor is named by its `weight_name`
        for part, sub in ((self.mixer, self.names[0]), (self.ffn, self.names[1])):
            if part is not None:
                part.prefix = prefix + sub
                for c in part.children():
                    if not c.prefix:
                        c.prefix = part.prefix

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, h, ctx, cache):
        """h: float32 residual stream [T, hidden], updated in place."""
        be = ctx.backend
        x = PreNormBlock._norm(self.mixer_norm, self.mixer, h, ctx)
        be.rmsnorm_add(h, self._output(self.mixer, h, x, ctx, cache), self.mixer_post.weight_f32(), self.mixer_post.eps)
        if self.ffn is not None:
            x = PreNormBlock._norm(self.ffn_norm, self.ffn, h, ctx)
            be.rmsnorm_add(h, self._output(self.ffn, h, x, ctx), self.ffn_post.weight_f32(), self.ffn_post.eps)
        return h

    @staticmethod
    def _output(part, h, x, ctx, *cache):
        """The sublayer's float output: returned by parts that can (`returns_output`), else gathered
        in a zeroed buffer that stands in for the residual stream."""
        if getattr(part, "returns_output", False):
            return part.forward(x, ctx, *cache, None)
        import torch
        y = torch.zeros_like(h)
        part.forward(x, ctx, *cache, y)
        return y


class PostNormBlock(Part):
    """h <- norm1(alpha h + mixer(h)); h <- norm2(alpha h + ffn(h)) (the feed-forward may be absent). The
    sublayers read the stream itself, in the run's storage type; sum and norm are one float kernel, which
    also writes the copy that the next sublayer's products read. A feed-forward may return its output as
    `Summands` (parts to be added in order, and a second summand with a sigmoid gate per row), which that
    kernel takes as they come. `names`: checkpoint sub-prefixes of mixer and feed-forward; the norms'
    weights are tensors named by each norm's `weight_name` under the block's prefix."""
    graph_safe = True

    def __init__(self, mixer: Part, mixer_norm: Part, ffn: Part | None = None, ffn_norm: Part | None = None,
                 alpha: float = 1.0, names=("mix.", "mlp.")):
        self.mixer, self.mixer_norm, self.ffn, self.ffn_norm = mixer, mixer_norm, ffn, ffn_norm
        self.alpha, self.names = float(alpha), names

    def children(self):
        return [p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None]

    def set_prefix(self, prefix: str):
        self.prefix = prefix
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None:
                norm.prefix = prefix
        for part, sub in ((self.mixer, self.names[0]), (self.ffn, self.names[1])):
            if part is not None:
                if hasattr(part, "set_prefix"):
                    part.set_prefix(prefix + sub)          # a part with named children of its own
                    continue
                part.prefix = prefix + sub
                for c in part.children():
                    if not c.prefix:
                        c.prefix = part.prefix

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, h, ctx, cache):
        """h: float32 residual stream [T, hidden], updated in place."""
        be = ctx.backend
        kept = ctx.per_forward.get("stream_copy")
        x = kept[1] if kept is not None and kept[0] is h else be.stream_copy(h)
        y = self.mixer.forward(x, ctx, cache, None)
        x = be.postnorm(h, y, self.alpha, self.mixer_norm.weight_f32(), self.mixer_norm.eps)
        if self.ffn is not None:
            y = self.ffn.forward(x, ctx, None)
            x = be.postnorm(h, y, self.alpha, self.ffn_norm.weight_f32(), self.ffn_norm.eps)
        ctx.per_forward["stream_copy"] = (h, x)        # what the next block's mixer reads
        return h


class ParallelBlock(Part):
    """h <- h + (mixer(n) + ffn(n)) with n = norm(h): one norm, both sublayers read its output, the feed-forward may
    be absent. Sublayers return their float outputs (a tensor, `Summands`, or `NormedSum` for a mixer whose members are
    normed before they are added); the sum of all of them and the residual sum are one float kernel. A mixer made
    of several mixers gets a tuple of cache layers. `names`: checkpoint sub-prefixes of mixer and feed-forward; the
    norm's weight is a tensor named by its `weight_name` under the block's prefix."""
    graph_safe = True

    def __init__(self, norm: Part, mixer: Part, ffn: Part | None = None, names=("mix.", "mlp.")):
        self.norm, self.mixer, self.ffn, self.names = norm, mixer, ffn, names

    def children(self):
        return [p for p in (self.norm, self.mixer, self.ffn) if p is not None]

    def set_prefix(self, prefix: str):
        self.prefix = prefix
        self.norm.prefix = prefix
        for part, sub in ((self.mixer, self.names[0]), (self.ffn, self.names[1])):
            if part is None:
                continue
            if hasattr(part, "set_prefix"):
                part.set_prefix(prefix + sub)
                continue
            part.prefix = prefix + sub
            for c in part.children():
                if not c.prefix:
                    c.prefix = part.prefix

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, h, ctx, cache):
        """h: float32 residual stream [T, hidden], updated in place."""
        n = self.norm.forward(h, ctx)
        m = self.mixer.forward(n, ctx, cache, None)
        f = None if self.ffn is None else self.ffn.forward(n, ctx, None)
        return ctx.backend.combine(h, m, f)


class GatedPreNormBlock(Part):
    """n = norm1(h); h += sigmoid(W_1 n + b_1) * mixer(n); then the same with norm2, W_2, b_2 and the feed-forward, which
    may be absent. The gates are as wide as the stream. A sublayer returns its float output (a tensor, or `ScaledSum`
    for a mixer made of mixers); the gate's sigmoid, the product with the output and the residual sum are one float
    kernel. `names`: checkpoint sub-prefixes of mixer and feed-forward; `gate_names`: the gates' matrices under the
    block's prefix (their biases: the same names with `.b`); the norms' weights are tensors named by each norm's
    `weight_name` under the block's prefix."""
    graph_safe = True

    def __init__(self, hidden: int, mixer_norm: Part, mixer: Part, ffn_norm: Part | None = None, ffn: Part | None = None,
                 names=("mix.", "mlp."), gate_names=("rg1", "rg2")):
        self.hidden, self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = hidden, mixer_norm, mixer, ffn_norm, ffn
        self.names, self.gate_names = names, gate_names
        self.w_g1 = self.b_g1 = self.w_g2 = self.b_g2 = None

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def params(self):
        W = self.hidden
        g1, g2 = self.gate_names
        ps = [Param("w_g1", (Source(g1, (W, W)),)), Param("b_g1", (Source(g1 + ".b", (W,)),), role="vector")]
        if self.ffn is not None:
            ps += [Param("w_g2", (Source(g2, (W, W)),)), Param("b_g2", (Source(g2 + ".b", (W,)),), role="vector")]
        return ps

    def set_prefix(self, prefix: str):
        self.prefix = prefix
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None:
                norm.prefix = prefix
        for part, sub in ((self.mixer, self.names[0]), (self.ffn, self.names[1])):
            if part is None:
                continue
            if hasattr(part, "set_prefix"):
                part.set_prefix(prefix + sub)
                continue
            part.prefix = prefix + sub
            for c in part.children():
                if not c.prefix:
                    c.prefix = part.prefix

    def cache_spec(self):
        return self.mixer.cache_spec()

    def finalize(self, device, dtype):
        self._b1 = self.b_g1.float().contiguous()
        self._b2 = None if self.b_g2 is None else self.b_g2.float().contiguous()

    def forward(self, h, ctx, cache):
        """h: float32 residual stream [T, hidden], updated in place."""
        be = ctx.backend
        n = self.mixer_norm.deferred(h, ctx)
        gate = be.linear_f32(n, self.w_g1, tag="gate")
        be.gated_add(h, gate, self._b1, self.mixer.forward(n, ctx, cache, None))
        if self.ffn is not None:
            n = self.ffn_norm.deferred(h, ctx)
            gate = be.linear_f32(n, self.w_g2, tag="gate")
            be.gated_add(h, gate, self._b2, self.ffn.forward(n, ctx, None))
        return h


class LoopStep(Part):
    """h += table[index] on every row. The passes of one loop share the table [times, hidden]: the
    first owns the tensor (`owner` None), the others name the first."""
    graph_safe = True

    def __init__(self, hidden: int, times: int, index: int, owner: "LoopStep | None" = None, name: str = "step"):
        self.hidden, self.times, self.index, self.owner, self.name = hidden, times, index, owner, name
        self.table = None

    def params(self):
        if self.owner is not None:
            return []
        return [Param("table", (Source(self.name, (self.times, self.hidden)),), role="vector")]

    def cache_spec(self):
        return None

    def finalize(self, device, dtype):
        table = (self.owner or self).table
        self._row = table[self.index].float().contiguous()

    def forward(self, h, ctx, cache=None):
        return ctx.backend.add_row(h, self._row)


register_part("block", "prenorm", PreNormBlock)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "postnorm", PostNormBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "prenorm_gated", GatedPreNormBlock)
register_part("block", "loop_step", LoopStep)
