"""Attention over a cache of compressed latents, as a mixer part.

Per token the input h is projected to queries (per head `dim` plain and `rot_dim` rotated
dimensions), to a latent c of `kv_rank` numbers (RMS-normed with a weight) and to one rotated key
part that all heads share; a head's plain key is W_uk c and its value W_uv c. Only c and the rotated
key part are cached (`LatentCacheSpec`: one row of kv_rank + rot_dim numbers a position, keys and
values alike). The up-projections never run over the cache: with
    q . (W_uk c) = (W_uk^T q) . c      and      sum_j p_j (W_uv c_j) = W_uv (sum_j p_j c_j)
W_uk is folded into the query before the attention kernel and W_uv applied to its output, both as
one product per head in one launch. Scores are (plain + rotated part) * `scale`, softmax over the keys
a `window` allows (None: all earlier ones); each head's output is multiplied by sigmoid of a gate
projected from h (`gate` False: there is none); W_o follows. `rot_dim` 0 with `position` None: no rotated part,
positions do not enter the scores. Scores, softmax, the latent's norm and the rotation are float.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import CacheKind, Param, Part, Source, register_cache_kind, register_part


@dataclass(frozen=True)
class LatentCacheSpec:
    """Paged rows of `width` numbers per position (latent, then the shared rotated key part)."""
    width: int
    window: int | None = None


def _allocate(spec, num_pages, page_size, dtype, device):
    return {"kv": torch.zeros((num_pages, page_size, spec.width), dtype=dtype, device=device)}


register_cache_kind(LatentCacheSpec, CacheKind(
    paged=True, allocate=_allocate, window=lambda spec: spec.window,
    page_bytes=lambda spec, page_size, dtype: spec.width * page_size * torch.empty((), dtype=dtype).element_size()))


class LatentAttention(Part):
    graph_safe = True
    takes_deferred = True      # x goes to the backend's products as it comes
    returns_output = True      # forward(..., residual=None) returns the float output instead of adding it

    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float,
                 position: Part | None, window: int | None = None, eps: float = 1e-6, gate: bool = True):
        if (position is None) != (rot_dim == 0):
            raise ValueError("a rotated part needs a position part, and only a rotated part does")
        self.hidden, self.heads, self.dim, self.rot_dim, self.vdim = hidden, heads, dim, rot_dim, vdim
        self.kv_rank, self.scale, self.position, self.window, self.eps = kv_rank, float(scale), position, window, float(eps)
        self.gate = gate
        self.w_in = self.w_latent_norm = self.w_uk = self.w_uv = self.w_o = None

    def children(self):
        return [] if self.position is None else [self.position]

    def params(self):
        H, W = self.heads, self.hidden
        return [Param("w_in", (Source("q", (H * (self.dim + self.rot_dim), W)),
                               Source("dkv", (self.kv_rank + self.rot_dim, W))) + ((Source("g", (H, W)),) if self.gate else ())),
                Param("w_latent_norm", (Source("dkv.norm", (self.kv_rank,), init="norm"),), role="vector"),
                Param("w_uk", (Source("uk", (H * self.dim, self.kv_rank)),)),
                Param("w_uv", (Source("uv", (H * self.vdim, self.kv_rank)),)),
                Param("w_o", (Source("o", (W, H * self.vdim)),))]

    def cache_spec(self):
        return LatentCacheSpec(self.kv_rank + self.rot_dim, self.window)

    def finalize(self, device, dtype):
        H = self.heads
        # per head: [kv_rank, dim] so that the fold is a product with K = dim; [vdim, kv_rank] as stored
        self._uk_t = self.w_uk.view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self._uv = self.w_uv.view(H, self.vdim, self.kv_rank)
        self._norm_f32 = self.w_latent_norm.float().contiguous()

    def forward(self, x, ctx, cache, residual=None):
        be = ctx.backend
        H, dk = self.heads, self.kv_rank + self.rot_dim
        q_cols = H * (self.dim + self.rot_dim)
        proj = be.linear(x, self.w_in)                                   # [T, q | dkv | gate]
        T = proj.shape[0]
        qfull = torch.empty((T, H, dk), dtype=proj.dtype, device=proj.device)
        if self.position is None:
            table, dims = torch.empty((T, 0, 2), dtype=torch.float32, device=proj.device), 0
        else:
            table, dims = self.position.table(ctx), self.position.dims
        writes = cache.writes
        be.latent_prepare(proj, 0, q_cols, H, self.dim, self.rot_dim, self.kv_rank, dims,
                          self._norm_f32, self.eps, table, cache.slots if writes else None,
                          cache.tensors["kv"] if writes else None, qfull)
        be.linear_heads(proj, self.dim + self.rot_dim, self._uk_t, qfull.view(T, H * dk), dk)
        o = be.latent_attention(qfull, cache, ctx, self.kv_rank, self.scale, self.window)
        att = torch.empty((T, H * self.vdim), dtype=proj.dtype, device=proj.device)
        be.linear_heads(o.view(T, H * self.kv_rank), self.kv_rank, self._uv, att, self.vdim,
                        gate=proj[:, q_cols + dk:] if self.gate else None)
        if residual is None:
            return be.linear_f32(att, self.w_o)
        be.linear_residual(att, self.w_o, residual)
        return None


register_part("mixer", "latent_attention", LatentAttention)
