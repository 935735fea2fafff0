"""Dense feed-forwards as parts. `SwiGLU`: down(silu(gate x) * (up x)). Formula:
src/gpu/cuda/shaders/moe.cu:141-146 and src/model/primitives.rs:557-585 of the reference. Gate and up
weights are stacked so that one product yields both. `ActFFN`: down(act(up x)) with act = relu(.)^2.
`ActFFN` also knows act = gelu in its tanh form. Both add into the residual stream, or return their float output when `residual` is None (for blocks that
norm after the sum)."""
from __future__ import annotations

from .base import Param, Part, Source, register_part


class SwiGLU(Part):
    graph_safe = True
    takes_deferred = True      # x goes to the backend's products as it comes
    returns_output = True

    def __init__(self, hidden: int, intermediate: int,
                 names=("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        self.hidden, self.intermediate, self.names = hidden, intermediate, names
        self.w_gate_up = self.w_down = None

    def params(self):
        H, I = self.hidden, self.intermediate
        g, u, d = self.names
        return [Param("w_gate_up", (Source(g, (I, H)), Source(u, (I, H)))),
                Param("w_down", (Source(d, (H, I)),))]

    def forward(self, x, ctx, residual):
        be = ctx.backend
        act = be.linear_swiglu(x, self.w_gate_up)
        if residual is None:
            return be.linear_f32(act, self.w_down, tag="down")
        be.linear_residual(act, self.w_down, residual)


class ActFFN(Part):
    """down(act(up x)), no biases; act: "relu2" = max(., 0)^2, "gelu_tanh" = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))."""
    graph_safe = True
    returns_output = True
    ACTS = ("relu2", "gelu_tanh")

    def __init__(self, hidden: int, intermediate: int, act: str = "relu2", names=("up", "down")):
        if act not in self.ACTS:
            raise ValueError(f"activation {act!r} is not known (known: {self.ACTS})")
        self.hidden, self.intermediate, self.act, self.names = hidden, intermediate, act, names
        self.w_up = self.w_down = None

    def params(self):
        H, I = self.hidden, self.intermediate
        return [Param("w_up", (Source(self.names[0], (I, H)),)), Param("w_down", (Source(self.names[1], (H, I)),))]

    def forward(self, x, ctx, residual):
        be = ctx.backend
        a = be.linear_act(x, self.w_up, self.act)
        if residual is None:
            return be.linear_f32(a, self.w_down, tag="down")
        be.linear_residual(a, self.w_down, residual)


register_part("ffn", "swiglu", SwiGLU)
register_part("ffn", "act", ActFFN)


class GluFFN(Part):
    """down(act(gate x, up x)), no biases, with the gated activation a constructor argument:
    "silu": silu(g) u; "gelu_tanh": gelu(g) u in its tanh form; "swish_clamped": with g' = min(g, limit) and
    u' = clamp(u, -limit, limit), g' sigmoid(alpha g') (u' + 1). Gate and up weights are stacked so that one product
    yields both; the two halves stay float until the activation has run."""
    graph_safe = True
    returns_output = True
    ACTS = ("silu", "gelu_tanh", "swish_clamped")

    def __init__(self, hidden: int, intermediate: int, act: str = "silu", limit: float = 0.0, alpha: float = 1.0,
                 names=("gate", "up", "down")):
        if act not in self.ACTS:
            raise ValueError(f"activation {act!r} is not known (known: {self.ACTS})")
        self.hidden, self.intermediate, self.act, self.limit, self.alpha = hidden, intermediate, act, float(limit), float(alpha)
        self.names = names
        self.w_gate_up = self.w_down = None

    def params(self):
        H, I = self.hidden, self.intermediate
        g, u, d = self.names
        return [Param("w_gate_up", (Source(g, (I, H)), Source(u, (I, H)))), Param("w_down", (Source(d, (H, I)),))]

    def forward(self, x, ctx, residual):
        be = ctx.backend
        a = be.linear_glu(x, self.w_gate_up, self.act, self.limit, self.alpha)
        if residual is None:
            return be.linear_f32(a, self.w_down, tag="down")
        be.linear_residual(a, self.w_down, residual)


register_part("ffn", "glu", GluFFN)
