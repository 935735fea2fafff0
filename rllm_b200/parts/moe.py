"""A routed feed-forward (mixture of experts) as a part.

Router logits z = W_router h in float (h in the run dtype), scores s = softmax(z) over all experts.
The experts form `groups` equal groups of neighbours; a group's score is its largest; only experts of
the best `keep` groups can be chosen; of those the `top` largest scores are taken, with the scores
themselves as weights (`renorm`: divided by their sum). An expert is W_down act(W_up h) without
biases, act = relu(.)^2. The experts of all tokens run as two grouped products over a row list
sorted by expert that a small kernel writes on the device, so the launches depend on the step's
size only; the weighted outputs land in one float row per (token, chosen expert), which the
caller sums in slot order (`SandwichBlock` does it inside its norm).
"""
from __future__ import annotations

from .base import Param, Part, Source, Summands, register_part


class RoutedExperts(Part):
    graph_safe = True
    returns_output = True

    def __init__(self, hidden: int, ff: int, experts: int, top: int, groups: int = 1, keep: int = 1,
                 renorm: bool = False, act: str = "relu2"):
        self.hidden, self.ff, self.experts, self.top = hidden, ff, experts, top
        self.groups, self.keep, self.renorm, self.act = groups, keep, renorm, act
        self.w_router = self.w_up = self.w_down = None

    def params(self):
        E, W, F = self.experts, self.hidden, self.ff
        return [Param("w_router", (Source("router", (E, W)),)),
                Param("w_up", tuple(Source(f"e{e}.up", (F, W)) for e in range(E))),
                Param("w_down", tuple(Source(f"e{e}.down", (W, F)) for e in range(E)))]

    def finalize(self, device, dtype):
        self._up = self.w_up.view(self.experts, self.ff, self.hidden)
        self._down = self.w_down.view(self.experts, self.hidden, self.ff)

    def forward(self, x, ctx, residual=None):
        """-> float [T, top, hidden]: the chosen experts' weighted outputs, to be summed over dim 1."""
        if residual is not None:
            raise NotImplementedError("RoutedExperts returns its parts; the block sums them")
        be = ctx.backend
        x = x.tensor() if hasattr(x, "tensor") else x
        _, _, plan = be.route(be.linear_f32(x, self.w_router), self.top, self.groups, self.keep, self.renorm,
                              tile_rows=be.expert_tile_rows(x, self._up, self._down, x.shape[0] * self.top))
        return be.experts_down(be.experts_up(x, self._up, plan, self.act), self._down, plan, x.shape[0], self.top)


class GatedRoutedExperts(Part):
    """A mixture of gated experts: expert(h) = W_down (silu(W_gate h) * (W_up h)), no biases.

    Router logits z = W_router h in float; scores by `score` ("sigmoid": each logit by itself; "softmax": over
    all experts); the `top` largest scores are chosen and are the weights (`renorm`: divided by their sum).
    The weight multiplies the expert's *input*: the output is the sum over the chosen experts of
    expert(weight * h). Because gate and up projections are linear, the weight is applied to their float
    results before the activation. `shared`: a dense gated feed-forward every token uses (its tensors under
    `shared.`), added times sigmoid(W_sg h) (`shared.sg`, one row) when `shared_gate`. Returns `Summands`: one
    float row per (token, chosen expert), the shared expert's output and its gate logit; the block's norm
    kernel adds them."""
    graph_safe = True
    returns_output = True

    def __init__(self, hidden: int, ff: int, experts: int, top: int, score: str = "sigmoid", renorm: bool = False,
                 shared: Part | None = None, shared_gate: bool = False):
        if top > experts:
            raise ValueError(f"top {top} exceeds the {experts} experts")
        self.hidden, self.ff, self.experts, self.top = hidden, ff, experts, top
        self.score, self.renorm, self.shared, self.shared_gate = score, renorm, shared, shared_gate and shared is not None
        self.w_router = self.w_gate_up = self.w_down = self.w_sg = None

    def children(self):
        return [] if self.shared is None else [self.shared]

    def set_prefix(self, prefix: str):
        self.prefix = prefix
        if self.shared is not None:
            self.shared.prefix = prefix + "shared."

    def params(self):
        E, W, F = self.experts, self.hidden, self.ff
        ps = [Param("w_router", (Source("router", (E, W)),)),
              Param("w_gate_up", tuple(Source(f"e{e}.{n}", (F, W)) for e in range(E) for n in ("gate", "up"))),
              Param("w_down", tuple(Source(f"e{e}.down", (W, F)) for e in range(E)))]
        if self.shared_gate:
            ps.append(Param("w_sg", (Source("shared.sg", (1, W)),)))
        return ps

    def finalize(self, device, dtype):
        E, F, W = self.experts, self.ff, self.hidden
        self._block = 16 if F % 16 == 0 else None
        if self._block and getattr(self, "_arranged", None) is not self.w_gate_up:
            # as bound: per expert its gate rows, then its up rows. Where the inner size allows it the rows are
            # kept in blocks of 16 gate rows each followed by their 16 up rows, so that a tile of the product
            # holds both halves of its outputs and the kernel can activate in its epilogue. One copy is kept.
            gu = self.w_gate_up.view(E, 2, F // 16, 16, W).permute(0, 2, 1, 3, 4).contiguous()
            self.w_gate_up = self._arranged = gu.view(E * 2 * F, W)
        self._gate_up = self.w_gate_up.view(E, 2 * F, W)
        self._down = self.w_down.view(E, W, F)

    def forward(self, x, ctx, residual=None):
        if residual is not None:
            raise NotImplementedError("GatedRoutedExperts returns its summands; the block adds them")
        be = ctx.backend
        x = x.tensor() if hasattr(x, "tensor") else x
        T = x.shape[0]
        _, _, plan = be.route(be.linear_f32(x, self.w_router, tag="router"), self.top, renorm=self.renorm, score=self.score,
                              tile_rows=be.expert_tile_rows(x, self._gate_up, self._down, T * self.top))
        act = be.experts_gated_up(x, self._gate_up, plan, self._block)        # silu(w g) * (w u), sorted rows
        parts = be.experts_down(act, self._down, plan, T, self.top, scale=False)
        if self.shared is None:
            return Summands(parts)
        return Summands(parts, self.shared.forward(x, ctx, None),
                        be.linear_f32(x, self.w_sg, tag="gate") if self.shared_gate else None)


register_part("ffn", "moe", RoutedExperts)
register_part("ffn", "moe_gated", GatedRoutedExperts)


class GluRoutedExperts(Part):
    """A mixture of gated experts whose weights multiply the experts' *outputs*: expert(h) = W_down act(W_gate h,
    W_up h) without biases, act one of `GluFFN.ACTS` with its `limit` and `alpha`. Router logits z = W_router h
    (+ a bias per expert, tensor `router.b`) in float; `score` "softmax_chosen": the `top` largest logits are chosen
    and their weights are the softmax over the chosen logits only ("softmax" and "sigmoid" as for the other routed
    feed-forwards). `shared`: a dense feed-forward every token uses (its tensors under `shared.`), added as it is.
    Returns `Summands`: one float row per (token, chosen expert) and the shared expert's output; the block adds them."""
    graph_safe = True
    returns_output = True

    def __init__(self, hidden: int, ff: int, experts: int, top: int, act: str = "silu", limit: float = 0.0,
                 alpha: float = 1.0, score: str = "softmax_chosen", renorm: bool = False, router_bias: bool = False,
                 shared: Part | None = None):
        if top > experts:
            raise ValueError(f"top {top} exceeds the {experts} experts")
        self.hidden, self.ff, self.experts, self.top = hidden, ff, experts, top
        self.act, self.limit, self.alpha = act, float(limit), float(alpha)
        self.score, self.renorm, self.router_bias, self.shared = score, renorm, router_bias, shared
        self.w_router = self.b_router = self.w_gate_up = self.w_down = None

    def children(self):
        return [] if self.shared is None else [self.shared]

    def set_prefix(self, prefix: str):
        self.prefix = prefix
        if self.shared is not None:
            self.shared.prefix = prefix + "shared."

    def params(self):
        E, W, F = self.experts, self.hidden, self.ff
        ps = [Param("w_router", (Source("router", (E, W)),)),
              Param("w_gate_up", tuple(Source(f"e{e}.{n}", (F, W)) for e in range(E) for n in ("gate", "up"))),
              Param("w_down", tuple(Source(f"e{e}.down", (W, F)) for e in range(E)))]
        if self.router_bias:
            ps.append(Param("b_router", (Source("router.b", (E,)),), role="vector"))
        return ps

    def finalize(self, device, dtype):
        E, F, W = self.experts, self.ff, self.hidden
        self._block = 16 if F % 16 == 0 else None
        if self._block and getattr(self, "_arranged", None) is not self.w_gate_up:
            # blocks of 16 gate rows each followed by their 16 up rows (as in GatedRoutedExperts): a tile of the
            # product then holds both halves of its outputs and the kernel activates in its epilogue
            gu = self.w_gate_up.view(E, 2, F // 16, 16, W).permute(0, 2, 1, 3, 4).contiguous()
            self.w_gate_up = self._arranged = gu.view(E * 2 * F, W)
        self._gate_up = self.w_gate_up.view(E, 2 * F, W)
        self._down = self.w_down.view(E, W, F)
        self._bias = None if self.b_router is None else self.b_router.float().contiguous()

    def forward(self, x, ctx, residual=None):
        if residual is not None:
            raise NotImplementedError("GluRoutedExperts returns its summands; the block adds them")
        be = ctx.backend
        x = x.tensor() if hasattr(x, "tensor") else x
        T = x.shape[0]
        _, _, plan = be.route(be.linear_f32(x, self.w_router, tag="router"), self.top, renorm=self.renorm, score=self.score,
                              bias=self._bias, tile_rows=be.expert_tile_rows(x, self._gate_up, self._down, T * self.top))
        act = be.experts_glu_up(x, self._gate_up, plan, self.act, self.limit, self.alpha, self._block)
        parts = be.experts_down(act, self._down, plan, T, self.top, scale=True)
        return Summands(parts, None if self.shared is None else self.shared.forward(x, ctx, None))


register_part("ffn", "moe_glu", GluRoutedExperts)
