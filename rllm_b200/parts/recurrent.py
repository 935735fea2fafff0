"""Recurrent mixers over a per-request state, each with a short causal convolution in front.

Both keep, per request, a float32 state S [heads, dim, vdim] and the last taps - 1 inputs of their convolution
(`StateSpec`), zeroed when the request opens and carried from step to step. The projections run in the run dtype;
convolution, gates, decays, step sizes, unit norms, the recurrence and the norm after it are float.

`StateSpaceMixer` (state-space duality form). W_in h = [z | x | B | C | dt] with inner = heads * vdim channels of z
and x, groups * state of B and C each, one dt per head. x, B and C pass the convolution (with bias) and silu;
dt <- softplus(dt + dt_bias), a = exp(-exp(A_log) dt) per head; per head (B and C shared by the heads of a group)
    S_t = a_t S_(t-1) + dt_t B_t x_t^T,      y_t = S_t^T C_t + D x_t.
y times silu(z), RMS-normed in `norm_groups` equal parts, times `norm`, then W_o.

`DeltaRuleMixer` (gated delta rule). q, k (kv_heads x dim) and v (heads x vdim) each pass a convolution without bias
and silu; q and k become unit vectors per head (q also times dim^-1/2); beta = sigmoid(W_b h) per head; a decay per
head and key channel g = exp(-exp(A_log) softplus(W_a2 (W_a1 h) + dt_bias)); per head
    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.
Each head's o is RMS-normed over vdim with one weight shared by the heads, times sigmoid(W_g2 (W_g1 h)), then W_o.
The widths of the two bottlenecks are sizes of the checkpoint unless given (random-weights mode).

`MinGRUMixer` (a gated recurrence whose gates read only the current token; no convolution, the state one number per
channel). z = sigmoid(W_z h + b_z), u = W_x h + b_x, the candidate c = u + 1/2 where u >= 0 and sigmoid(u) where u < 0;
    S_t = (1 - z_t) S_(t-1) + z_t c_t,
and the output is W_o (S_t * silu(W_g h))."""
from __future__ import annotations

import torch

from .base import Param, Part, Source, StateSpec, register_part


class StateSpaceMixer(Part):
    graph_safe = True
    returns_output = True

    def __init__(self, hidden: int, heads: int, vdim: int, state: int, groups: int = 1, norm_groups: int = 1,
                 taps: int = 4, eps: float = 1e-6):
        if heads % groups or (heads * vdim) % norm_groups:
            raise ValueError(f"{heads} heads of {vdim} do not divide over {groups} groups / {norm_groups} norm parts")
        self.hidden, self.heads, self.vdim, self.state, self.groups = hidden, heads, vdim, state, groups
        self.norm_groups, self.taps, self.eps = norm_groups, taps, float(eps)
        self.inner = heads * vdim
        self.conv_channels = self.inner + 2 * groups * state
        self.w_in = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = self.w_norm = self.w_o = None

    def params(self):
        W, I, C, H = self.hidden, self.inner, self.conv_channels, self.heads
        return [Param("w_in", (Source("in", (2 * I + 2 * self.groups * self.state + H, W)),)),
                Param("conv_w", (Source("conv", (C, self.taps)),), role="vector"),
                Param("conv_b", (Source("conv.b", (C,)),), role="vector"),
                Param("dt_bias", (Source("dt_bias", (H,)),), role="vector"),
                Param("a_log", (Source("A_log", (H,)),), role="vector"),
                Param("skip", (Source("D", (H,), init="norm"),), role="vector"),
                Param("w_norm", (Source("norm", (I,), init="norm"),), role="vector"),
                Param("w_o", (Source("o", (W, I)),))]

    def cache_spec(self):
        return StateSpec((("S", (self.heads, self.state, self.vdim), torch.float32),
                          ("tail", (max(self.taps - 1, 1), self.conv_channels), torch.float32)))

    def finalize(self, device, dtype):
        f32 = lambda t: t.float().contiguous()
        self._conv_w, self._conv_b, self._dt_bias = f32(self.conv_w), f32(self.conv_b), f32(self.dt_bias)
        self._a_log, self._skip, self._norm = f32(self.a_log), f32(self.skip), f32(self.w_norm)

    def forward(self, x, ctx, cache, residual=None):
        be = ctx.backend
        x = x.tensor() if hasattr(x, "tensor") else x
        I, GN, H = self.inner, self.groups * self.state, self.heads
        proj = be.linear(x, self.w_in, tag="in")                                  # [T, z | x | B | C | dt]
        xbc = be.short_conv(proj, I, self.conv_channels, self._conv_w, self._conv_b, ctx, cache.state["tail"])
        step, decay = be.softplus_decay(proj, 2 * I + 2 * GN, H, self._dt_bias, self._a_log, want_step=True)
        y = be.state_scan(xbc[:, I + GN:], self.groups, xbc[:, I: I + GN], self.groups, xbc[:, :I], decay, H, self.state,
                          self.vdim, ctx, cache.state["S"], vscale=step, skip=self._skip)
        g = be.gated_norm(y.view(-1, I), proj, 0, self._norm, self.eps, self.norm_groups, gate_first=True, act="silu")
        if residual is None:
            return be.linear_f32(g, self.w_o, tag="o")
        be.linear_residual(g, self.w_o, residual)
        return None


class DeltaRuleMixer(Part):
    graph_safe = True
    returns_output = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int = 4, eps: float = 1e-6,
                 unit_eps: float = 1e-6, decay_rank: int | None = None, gate_rank: int | None = None):
        if heads % kv_heads:
            raise ValueError(f"heads {heads} must be a multiple of kv_heads {kv_heads}")
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim = hidden, heads, kv_heads, dim, vdim
        self.taps, self.eps, self.unit_eps = taps, float(eps), float(unit_eps)
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        self.qk = kv_heads * dim
        self.conv_channels = 2 * self.qk + heads * vdim
        self.w_in = self.conv_w = self.w_b = self.a_log = self.w_norm = self.w_a2 = self.dt_bias = self.w_g2 = self.w_o = None

    def params(self):
        W, H, QK, V = self.hidden, self.heads, self.qk, self.heads * self.vdim
        ra = -1 if self.decay_rank is None else self.decay_rank
        rg = -1 if self.gate_rank is None else self.gate_rank
        return [Param("w_in", (Source("q", (QK, W)), Source("k", (QK, W)), Source("v", (V, W)), Source("a1", (ra, W)),
                               Source("g1", (rg, W)))),
                Param("conv_w", (Source("q.conv", (QK, self.taps)), Source("k.conv", (QK, self.taps)),
                                 Source("v.conv", (V, self.taps))), role="vector"),
                Param("w_b", (Source("b", (H, W)),)),
                Param("a_log", (Source("A_log", (H,)),), role="vector"),
                Param("w_norm", (Source("norm", (self.vdim,), init="norm"),), role="vector"),
                Param("w_a2", (Source("a2", (H * self.dim, ra)),)),
                Param("dt_bias", (Source("dt_bias", (H * self.dim,)),), role="vector"),
                Param("w_g2", (Source("g2", (V, rg)),)),
                Param("w_o", (Source("o", (W, V)),))]

    def cache_spec(self):
        return StateSpec((("S", (self.heads, self.dim, self.vdim), torch.float32),
                          ("tail", (max(self.taps - 1, 1), self.conv_channels), torch.float32)))

    def finalize(self, device, dtype):
        f32 = lambda t: t.float().contiguous()
        self._conv_w, self._dt_bias, self._a_log, self._norm = f32(self.conv_w), f32(self.dt_bias), f32(self.a_log), f32(self.w_norm)
        self._ra, self._rg = self.w_a2.shape[1], self.w_g2.shape[1]
        if self.w_in.shape[0] != self.conv_channels + self._ra + self._rg:
            raise ValueError(f"{self.prefix}a1 and g1 have {self.w_in.shape[0] - self.conv_channels} rows together, a2 and g2 "
                             f"take {self._ra} and {self._rg}")

    def forward(self, x, ctx, cache, residual=None):
        be = ctx.backend
        x = x.tensor() if hasattr(x, "tensor") else x
        H, G, d, v, C = self.heads, self.kv_heads, self.dim, self.vdim, self.conv_channels
        proj = be.linear(x, self.w_in, tag="in")                                  # [T, q | k | v | a1 | g1]
        beta = be.linear_f32(x, self.w_b, tag="beta")                             # float logits [T, H]
        qkv = be.short_conv(proj, 0, C, self._conv_w, None, ctx, cache.state["tail"])
        be.unit_heads(qkv, 0, G, d, d ** -0.5, self.unit_eps)
        be.unit_heads(qkv, self.qk, G, d, 1.0, self.unit_eps)
        z = be.linear_f32(proj[:, C: C + self._ra], self.w_a2, tag="decay")       # [T, H * dim]
        _, decay = be.softplus_decay(z, 0, H * d, self._dt_bias, self._a_log)
        o = be.state_scan(qkv[:, : self.qk], G, qkv[:, self.qk: 2 * self.qk], G, qkv[:, 2 * self.qk:], decay, H, d, v, ctx,
                          cache.state["S"], beta=beta)
        gate = be.linear_f32(proj[:, C + self._ra:], self.w_g2, tag="gate")       # float logits [T, H * vdim]
        g = be.gated_norm(o.view(-1, H * v), gate, 0, self._norm, self.eps, H, gate_first=False, act="sigmoid")
        if residual is None:
            return be.linear_f32(g, self.w_o, tag="o")
        be.linear_residual(g, self.w_o, residual)
        return None


class MinGRUMixer(Part):
    graph_safe = True
    returns_output = True

    def __init__(self, hidden: int, width: int, names=("z", "x", "g", "o")):
        self.hidden, self.width, self.names = hidden, width, names
        self.w_in = self.b_z = self.b_x = self.w_o = None

    def params(self):
        W, R = self.hidden, self.width
        z, x, g, o = self.names
        return [Param("w_in", (Source(z, (R, W)), Source(x, (R, W)), Source(g, (R, W)))),
                Param("b_z", (Source(z + ".b", (R,)),), role="vector"),
                Param("b_x", (Source(x + ".b", (R,)),), role="vector"),
                Param("w_o", (Source(o, (W, R)),))]

    def cache_spec(self):
        return StateSpec((("S", (self.width,), torch.float32),))

    def finalize(self, device, dtype):
        self._bz, self._bx = self.b_z.float().contiguous(), self.b_x.float().contiguous()

    def forward(self, x, ctx, cache, residual=None):
        be = ctx.backend
        R = self.width
        proj = be.linear_f32(x, self.w_in, tag="in")                                # float [T, z | x | g]
        y = be.mingru_scan(proj, 0, R, 2 * R, R, self._bz, self._bx, ctx, cache.state["S"])
        if residual is None:
            return be.linear_f32(y, self.w_o, tag="o")
        be.linear_residual(y, self.w_o, residual)
        return None


class SideBySideMixer(Part):
    """Two mixers that read the same input; the result is coef * (w_l * l / rms(l) + w_r * r / rms(r)) with plain
    weights `<left name>out` and `<right name>out` of the model's width. Returned as `NormedSum`: the block's sum
    kernel norms and adds the two. Each member has a cache layer of its own. `scales` (a_l, a_r): no norms and no
    weights, the result is a_l * l + a_r * r, returned as `ScaledSum`."""
    graph_safe = True
    returns_output = True

    def __init__(self, hidden: int, left: Part, right: Part, coef: float = 0.5, eps: float = 1e-6,
                 names=("left.", "right."), scales: tuple | None = None):
        self.hidden, self.left, self.right, self.coef, self.eps, self.names = hidden, left, right, float(coef), float(eps), names
        self.scales = None if scales is None else (float(scales[0]), float(scales[1]))
        self.w_left = self.w_right = None

    def children(self):
        return [self.left, self.right]

    def set_prefix(self, prefix: str):
        self.prefix = prefix
        for part, sub in zip(self.children(), self.names):
            part.prefix = prefix + sub

    def params(self):
        if self.scales is not None:
            return []
        return [Param("w_left", (Source(self.names[0] + "out", (self.hidden,), init="norm"),), role="vector"),
                Param("w_right", (Source(self.names[1] + "out", (self.hidden,), init="norm"),), role="vector")]

    def cache_spec(self):
        return (self.left.cache_spec(), self.right.cache_spec())

    def finalize(self, device, dtype):
        if self.scales is None:
            self._wl, self._wr = self.w_left.float().contiguous(), self.w_right.float().contiguous()

    def forward(self, x, ctx, cache, residual=None):
        from .base import NormedSum, ScaledSum
        if residual is not None:
            raise NotImplementedError("SideBySideMixer returns its summands; the block adds them")
        l = self.left.forward(x, ctx, cache[0], None)
        r = self.right.forward(x, ctx, cache[1], None)
        if self.scales is not None:
            return ScaledSum(((l, self.scales[0]), (r, self.scales[1])))
        return NormedSum(((l, self._wl), (r, self._wr)), self.coef, self.eps)


register_part("mixer", "state_space", StateSpaceMixer)
register_part("mixer", "delta_rule", DeltaRuleMixer)
register_part("mixer", "side_by_side", SideBySideMixer)
register_part("mixer", "min_gru", MinGRUMixer)
