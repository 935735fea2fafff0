"""Grouped-query attention over the paged cache, as a mixer part.

Order of operations as in the reference's Llama layer (src/model/registry/llama.rs:168-229):
q, k, v projections (here one product with the three weights stacked), optional bias,
rotation of q and k, write of k and v to the cache, attention with scale head_dim^-1/2
(src/gpu/cuda/shaders/attention.cu:336), output projection added to the residual stream.
A `window` limits each query to the last `window` keys
(src/gpu/cuda/shaders/attention.cu:337-338).
"""
from __future__ import annotations

from .base import KVCacheSpec, Param, Part, Source, register_part


class GQAttention(Part):
    graph_safe = True
    takes_deferred = True      # x goes to the backend's products as it comes

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, position: Part,
                 window: int | None = None, bias: bool = False, scale: float | None = None):
        if heads % kv_heads:
            raise ValueError(f"heads {heads} must be a multiple of kv_heads {kv_heads}")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} must be a multiple of 16, at most 256")
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.position, self.window, self.bias = position, window, bias
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.w_qkv = self.b_qkv = self.w_o = None

    @property
    def q_size(self):
        return self.heads * self.head_dim

    @property
    def kv_size(self):
        return self.kv_heads * self.head_dim

    def children(self):
        return [self.position]

    def params(self):
        H, Q, KV = self.hidden, self.q_size, self.kv_size
        ps = [Param("w_qkv", (Source("q_proj.weight", (Q, H)), Source("k_proj.weight", (KV, H)),
                              Source("v_proj.weight", (KV, H)))),
              Param("w_o", (Source("o_proj.weight", (H, Q)),))]
        if self.bias:
            # random-weights mode draws them like the matrices: a bias of zeros would hide a
            # kernel that drops it
            ps.append(Param("b_qkv", (Source("q_proj.bias", (Q,)), Source("k_proj.bias", (KV,)),
                                      Source("v_proj.bias", (KV,)))))
        return ps

    def cache_spec(self):
        return KVCacheSpec(self.kv_heads, self.head_dim, self.window)

    def forward(self, x, ctx, cache, residual):
        """x: normalised activations [T, hidden]; adds the mixer's output into `residual`."""
        be = ctx.backend
        if hasattr(self.position, "project_rotate_store"):
            qkv = self.position.project_rotate_store(x, self.w_qkv, self.b_qkv, ctx, cache, self.heads,
                                                     self.kv_heads)
        else:
            qkv = be.linear(x, self.w_qkv, bias=self.b_qkv)
            self.position.rotate_and_store(qkv, ctx, cache, self.heads, self.kv_heads)
        q = qkv[:, : self.q_size]
        attn = be.attention(q, cache, ctx, self.heads, self.scale, self.window)
        be.linear_residual(attn, self.w_o, residual)


register_part("mixer", "gqa", GQAttention)


class SinkGQAttention(Part):
    """Grouped-query attention with what some designs put around it, every piece a constructor argument:

    * keys of `head_dim` and values of `v_dim` numbers per head;
    * `qk_norm`: queries and keys divided by their root mean square per head, times a weight of `head_dim`
      numbers shared by all heads (tensors `q.norm`, `k.norm`), before the rotation;
      `qk_norm_weight` False: no weights, queries and keys become vectors of root mean square 1 (a plain factor
      commutes with the rotation, so it is the same norm whether a design names it before or after the rotation);
    * `position`: a rotary part (its `rot_dim` leading dimensions of a head are rotated, the rest pass) or None;
    * the mask: causal, and a `window` (the last `window` positions) and/or a `chunk` (only the positions of the
      query's own block of `chunk` positions, blocks counted from position 0); `keep_first`: the positions below
      this number stay visible to every later query whatever the window says (their pages are never given back);
    * `sink`: one learned number per head (tensor `sink`) whose exponential joins the softmax's denominator;
    * `weights` "sigmoid": no softmax; a visible key's weight is sigmoid(score + b_h) with one learned number per
      head (tensor `score_bias`, None: no bias), not normalised over the keys;
    * `value_mix`: None, or (role, key). The values of the layers that share a `key` are mixed with those of the
      first of them: role "first" keeps its step's values for the others, role "mix" turns its own into
      (1 - lam) v + lam v_first, lam the scalar tensor `vmix`, before they are cached;
    * `gate`: head h's output times sigmoid((W_g x)_h) (tensor `g`, one row per head), before W_o.

    Scores, softmax, norms, rotation and the gate's sigmoid are float. `forward(..., residual=None)` returns
    the float output (for blocks that norm after the sum). `names`: the checkpoint names of q, k, v, o."""
    graph_safe = True
    returns_output = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, v_dim: int | None = None,
                 position: Part | None = None, scale: float | None = None, window: int | None = None,
                 chunk: int | None = None, qk_norm: bool = False, sink: bool = False, gate: bool = False,
                 eps: float = 1e-6, names=("q", "k", "v", "o"), qk_norm_weight: bool = True, keep_first: int = 0,
                 weights: str = "softmax", score_bias: str | None = None, value_mix: tuple | None = None):
        if heads % kv_heads:
            raise ValueError(f"heads {heads} must be a multiple of kv_heads {kv_heads}")
        v_dim = head_dim if v_dim is None else v_dim
        if not 0 < head_dim <= 256 or not 0 < v_dim <= 256:
            raise ValueError(f"head sizes {head_dim} / {v_dim} must lie in 1..256")
        self.hidden, self.heads, self.kv_heads, self.head_dim, self.v_dim = hidden, heads, kv_heads, head_dim, v_dim
        self.position, self.window, self.chunk = position, window, chunk
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.qk_norm, self.sink, self.gate, self.eps, self.names = qk_norm, sink, gate, float(eps), names
        if weights not in ("softmax", "sigmoid"):
            raise ValueError(f"attention weights {weights!r} are not known (known: 'softmax', 'sigmoid')")
        if weights == "sigmoid" and sink:
            raise ValueError("a sink belongs to a softmax; sigmoid weights have none")
        if value_mix is not None and value_mix[0] not in ("first", "mix"):
            raise ValueError(f"value_mix role {value_mix[0]!r} is not known (known: 'first', 'mix')")
        self.qk_norm_weight, self.keep_first, self.weights = qk_norm_weight, int(keep_first or 0), weights
        self.score_bias, self.value_mix = score_bias, value_mix
        self.w_qkv = self.w_o = self.w_g = self.q_norm = self.k_norm = self.sinks = self.bias = self.lam = None

    def children(self):
        return [] if self.position is None else [self.position]

    def params(self):
        W, H, G, D, V = self.hidden, self.heads, self.kv_heads, self.head_dim, self.v_dim
        q, k, v, o = self.names
        ps = [Param("w_qkv", (Source(q, (H * D, W)), Source(k, (G * D, W)), Source(v, (G * V, W)))),
              Param("w_o", (Source(o, (W, H * V)),))]
        if self.qk_norm and self.qk_norm_weight:
            ps += [Param("q_norm", (Source(q + ".norm", (D,), init="norm"),), role="vector"),
                   Param("k_norm", (Source(k + ".norm", (D,), init="norm"),), role="vector")]
        if self.sink:
            ps.append(Param("sinks", (Source("sink", (H,)),), role="vector"))
        if self.weights == "sigmoid" and self.score_bias is not None:
            ps.append(Param("bias", (Source(self.score_bias, (H,)),), role="vector"))
        if self.value_mix is not None:
            # the first layer of a group owns the tensor too (a checkpoint stores it), and has no use for it
            ps.append(Param("lam", (Source("vmix", ()),), role="vector"))
        if self.gate:
            ps.append(Param("w_g", (Source("g", (H, W)),)))
        return ps

    def cache_spec(self):
        return KVCacheSpec(self.kv_heads, self.head_dim, self.window, self.chunk,
                           None if self.v_dim == self.head_dim else self.v_dim, self.keep_first if self.window else 0)

    def finalize(self, device, dtype):
        import torch
        f32 = lambda t: None if t is None else t.float().contiguous()
        self._qn, self._kn, self._sinks = f32(self.q_norm), f32(self.k_norm), f32(self.sinks)
        if self.qk_norm and not self.qk_norm_weight:
            self._qn = self._kn = torch.ones(self.head_dim, dtype=torch.float32, device=device)
        if self.weights == "sigmoid":
            self._sinks = f32(self.bias)
        self._lam = None if self.lam is None else self.lam.float().reshape(1).contiguous()

    def forward(self, x, ctx, cache, residual=None):
        be = ctx.backend
        x = x.tensor() if hasattr(x, "tensor") else x
        H, G, D, V = self.heads, self.kv_heads, self.head_dim, self.v_dim
        proj = be.linear(x, self.w_qkv, tag="qkv")                                  # [T, q | k | v]
        gate = be.linear_f32(x, self.w_g, tag="gate") if self.gate else None         # float logits [T, H]
        pos = self.position
        first = lam = None
        if self.value_mix is not None:
            role, key = self.value_mix
            if role == "first":                  # this step's values, as projected, for the layers that mix them in
                ctx.per_forward[("value_mix", key)] = proj[:, (H + G) * D:]
            else:                                # mixed on their way into the pages, by the kernel that writes them
                first, lam = ctx.per_forward.get(("value_mix", key)), self._lam
                if first is None or first.shape[1] != G * V:
                    raise ValueError(f"{self.prefix}: the values to mix in ({key!r}) are missing or of another size")
        be.qk_norm_rope_store(proj, 0, H * D, (H + G) * D, H, G, D, V, 0 if pos is None else pos.rot_dim,
                              self._qn, self._kn, self.eps, None if pos is None else pos.table(ctx), cache, first, lam)
        att = be.sink_attention(proj[:, : H * D], cache, ctx, H, self.scale, self.window, self.chunk, self._sinks, gate,
                                self.keep_first if self.window else 0, self.weights == "sigmoid")
        if residual is None:
            return be.linear_f32(att, self.w_o, tag="o")
        be.linear_residual(att, self.w_o, residual)
        return None


register_part("mixer", "gqa_sink", SinkGQAttention)


class TalkingHeadsAttention(Part):
    """Grouped-query attention whose heads' softmax weights are mixed by a matrix before they meet the values:

        p_g(i, j) = exp(s_g(i, j)) / (exp(sink) + sum_j' exp(s_g(i, j')))       s_g = scale * q_g . k_c(g)
        w_h(i, j) = sum_g M[h, g] p_g(i, j)            o_h(i) = sum_j w_h(i, j) v_c(h)(j)

    with c(h) the key/value head of query head h and M the tensor `talk` [heads, heads]. Every piece is a constructor
    argument: keys of `head_dim` and values of `v_dim` numbers per head; `bias`: the q, k and v projections have
    biases (`<name>.b`); `value_norm`: each value head is divided by its root mean square (no weight) and cached so;
    the mask is causal with an optional `window` and/or `chunk`; `sink`: a fixed score whose exponential joins every
    head's denominator (None: the plain softmax). Positions do not enter the scores. Scores, softmax, the mix and the
    value norm are float. `forward(..., residual=None)` returns the float output."""
    graph_safe = True
    returns_output = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, v_dim: int | None = None,
                 scale: float | None = None, window: int | None = None, chunk: int | None = None, bias: bool = False,
                 value_norm: bool = False, sink: float | None = None, eps: float = 1e-6,
                 names=("q", "k", "v", "o", "talk")):
        if heads % kv_heads:
            raise ValueError(f"heads {heads} must be a multiple of kv_heads {kv_heads}")
        v_dim = head_dim if v_dim is None else v_dim
        if not 0 < v_dim <= 256 or head_dim <= 0:
            raise ValueError(f"head sizes {head_dim} / {v_dim}: values must lie in 1..256")
        self.hidden, self.heads, self.kv_heads, self.head_dim, self.v_dim = hidden, heads, kv_heads, head_dim, v_dim
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.window, self.chunk, self.bias, self.value_norm = window, chunk, bias, value_norm
        self.sink, self.eps, self.names = sink, float(eps), names
        self.w_qkv = self.b_qkv = self.w_o = self.talk = None

    def params(self):
        W, H, G, D, V = self.hidden, self.heads, self.kv_heads, self.head_dim, self.v_dim
        q, k, v, o, talk = self.names
        ps = [Param("w_qkv", (Source(q, (H * D, W)), Source(k, (G * D, W)), Source(v, (G * V, W)))),
              Param("w_o", (Source(o, (W, H * V)),)),
              Param("talk", (Source(talk, (H, H)),), role="vector")]
        if self.bias:
            ps.append(Param("b_qkv", (Source(q + ".b", (H * D,)), Source(k + ".b", (G * D,)), Source(v + ".b", (G * V,)))))
        return ps

    def cache_spec(self):
        return KVCacheSpec(self.kv_heads, self.head_dim, self.window, self.chunk,
                           None if self.v_dim == self.head_dim else self.v_dim)

    def finalize(self, device, dtype):
        import torch
        self._talk = self.talk.float().contiguous()
        self._sinks = None if self.sink is None else torch.full((self.heads,), float(self.sink), dtype=torch.float32,
                                                                device=device)

    def forward(self, x, ctx, cache, residual=None):
        be = ctx.backend
        x = x.tensor() if hasattr(x, "tensor") else x
        H, G, D, V = self.heads, self.kv_heads, self.head_dim, self.v_dim
        proj = be.linear(x, self.w_qkv, bias=self.b_qkv, tag="qkv")                      # [T, q | k | v]
        be.value_norm_store(proj, H * D, (H + G) * D, G, D, V, self.eps, self.value_norm, cache)
        att = be.talk_attention(proj[:, : H * D], cache, ctx, H, self.scale, self._talk, self.window, self.chunk,
                                self._sinks)
        if residual is None:
            return be.linear_f32(att, self.w_o, tag="o")
        be.linear_residual(att, self.w_o, residual)
        return None


register_part("mixer", "gqa_talk", TalkingHeadsAttention)
