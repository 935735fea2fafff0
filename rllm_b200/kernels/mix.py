"""Python face of the libraries "mix" (sequence mixers other than grouped-query attention: attention
over a cache of compressed latents, gated linear attention as a recurrence over per-request state)
and "experts" (routed feed-forwards: top-k routing with limited groups, the plan of a grouped product,
the grouped product itself, and the norm that follows a sublayer). Like `ops`, every function checks shapes,
dtypes and devices and then calls an `extern "C"` launcher on torch's current stream; there is no
CPU or library path behind them.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong

import torch

from . import ops
from .ops import KernelError, _check, _cuda, _dt, _fn, _ptr, _stream

_P, _LL = ops._P, c_longlong
GEPI_STORE, GEPI_STORE_F32, GEPI_RELU2, GEPI_SILU_GATED = 0, 1, 2, 3

ops.register_signatures("experts", {
    "rllm_grouped_gemm_uniform": [c_int, c_int, _P, _LL, _LL, _P, _LL, _P, _LL, _LL, c_int, c_int, c_int, c_int,
                                  _P, _LL, _P],
    "rllm_grouped_gemm_ragged": [c_int, c_int, _P, _LL, _P, _LL, _P, _LL, c_int, c_int, _P, _P, c_int, c_int, _P, _P, _P,
                                 _P],
    "rllm_grouped_gemm_tile_rows": [c_int, _LL, c_int, c_int],
    "rllm_grouped_gemm_tc_supported": [_LL, c_int, c_int],
    "rllm_grouped_gemm_tc": [c_int, _P, _LL, _LL, _P, c_int, c_int, c_int, _P, _LL, _P, _P, c_int, _P, _P, _P, c_int, c_float,
                             c_float, _P],
    "rllm_gather_rows_bf16": [_P, _LL, _P, _P, c_int, c_int, _P],
    "rllm_moe_topk": [_P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P],
    "rllm_moe_plan": [_P, _P, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P],
    "rllm_rmsnorm_add": [_P, c_int, _P, _P, c_int, c_int, c_float, _P],
    "rllm_add_row": [_P, _P, c_int, c_int, _P],
})
ops.register_signatures("mix", {
    "rllm_latent_prepare": [c_int, _P, _LL, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_float, _P,
                            _P, _P, _P, _P],
    "rllm_latent_attention": [c_int, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                              c_int, _P, c_int, c_int, c_int, c_int, _P, _P, _P],
    "rllm_gla_decay": [_P, _P, c_int, c_int, c_float, _P],
    "rllm_gla_scan": [c_int, _P, _LL, c_int, c_int, c_int, _P, c_float, c_int, c_int, c_int, c_int, c_int, _P, _P, _P,
                      _P, c_int, _P, _P, _P],
    "rllm_gla_finish": [c_int, _P, _P, c_float, _P, _LL, c_int, c_int, c_int, c_int, _P, _P],
})


def _f32(t: torch.Tensor, name: str, shape=None) -> None:
    _cuda(t, name)
    if t.dtype != torch.float32 or not t.is_contiguous() or (shape is not None and tuple(t.shape) != tuple(shape)):
        raise KernelError(f"{name} must be contiguous float32" + (f" {list(shape)}" if shape is not None else "")
                          + f", got {t.dtype} {list(t.shape)}")


def _i32(t: torch.Tensor, name: str, n: int | None = None) -> None:
    _cuda(t, name)
    if t.dtype != torch.int32 or not t.is_contiguous() or (n is not None and t.numel() < n):
        raise KernelError(f"{name} must be a contiguous int32 vector" + (f" of at least {n}" if n is not None else ""))


def _rows(t: torch.Tensor, name: str, cols: int) -> None:
    """[T, >= cols] with unit inner stride."""
    _cuda(t, name)
    if t.dim() != 2 or t.stride(1) != 1 or t.shape[1] < cols:
        raise KernelError(f"{name} must be [T, >= {cols}] with unit inner stride, got {list(t.shape)}")


# --------------------------------------------------------------------------- norm after a sublayer

def rmsnorm_add(residual: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """residual [T, H] += w * s / sqrt(mean(s^2) + eps), s = y[t] ([T, H]) or the sum over p of y[t, p]
    ([T, parts, H]), all float32, in place."""
    _f32(residual, "residual")
    T, H = residual.shape
    parts = 1 if y.dim() == 2 else y.shape[1]
    _f32(y, "y", (T, H) if y.dim() == 2 else (T, parts, H))
    _f32(w, "w", (H,))
    _check(_fn("experts", "rllm_rmsnorm_add")(y.data_ptr(), parts, w.data_ptr(), residual.data_ptr(), T, H, float(eps),
                                          _stream()), "rmsnorm_add")
    return residual


def add_row(h: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """h [T, H] += v [H] on every row, float32, in place."""
    _f32(h, "h")
    _f32(v, "v", (h.shape[1],))
    _check(_fn("experts", "rllm_add_row")(h.data_ptr(), v.data_ptr(), h.shape[0], h.shape[1], _stream()), "add_row")
    return h


# --------------------------------------------------------------------------- grouped products

def grouped_gemm_uniform(a: torch.Tensor, a_gs: int, w: torch.Tensor, out: torch.Tensor, c_gs: int, epilogue: int,
                         gate: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, g * c_gs + n] = sum_k a[t, g * a_gs + k] * w[g, n, k] for every problem g (times
    sigmoid(gate[t, g]) when a gate is given). a [T, >= (G-1) * a_gs + K]; w [G, N, K] contiguous, of a's
    dtype; out [T, >= (G-1) * c_gs + N] float32 for GEPI_STORE_F32, else of a's dtype; gate [T, >= G] of
    a's dtype, unit inner stride."""
    G, N, K = w.shape
    _rows(a, "a", (G - 1) * a_gs + K)
    _rows(out, "out", (G - 1) * c_gs + N)
    _cuda(w, "w")
    if not w.is_contiguous() or w.dtype != a.dtype or a.shape[0] != out.shape[0]:
        raise KernelError("grouped product: w must be contiguous [G, N, K] of a's dtype, out must have a's rows")
    if out.dtype != (torch.float32 if epilogue == GEPI_STORE_F32 else a.dtype):
        raise KernelError(f"grouped product: out has dtype {out.dtype}")
    if gate is not None:
        _rows(gate, "gate", G)
        if gate.dtype != a.dtype or gate.shape[0] != a.shape[0]:
            raise KernelError("grouped product: the gate must have a's dtype and rows")
    _check(_fn("experts", "rllm_grouped_gemm_uniform")(
        _dt(a, "a"), epilogue, a.data_ptr(), a.stride(0), a_gs, w.data_ptr(), N * K, out.data_ptr(), out.stride(0),
        c_gs, a.shape[0], G, N, K, _ptr(gate), 0 if gate is None else gate.stride(0), _stream()), "grouped_gemm_uniform")
    return out


class RoutePlan:
    """What `moe_plan` leaves on the device for the grouped products of one routed feed-forward: per
    sorted row the token it reads (`rows_tok`), the (token, slot) row it writes (`rows_dest`) and its
    weight (`rows_scale`); the tile table and its length."""
    __slots__ = ("rows_tok", "rows_dest", "rows_scale", "tiles", "n_tiles", "max_tiles", "n_rows", "tile_rows")


def tile_rows(dtype: torch.dtype, lda: int, K: int, n_rows: int = 1 << 30) -> int:
    """Rows a plan's tile may have for a ragged product whose input has dtype `dtype`, row stride `lda` and
    depth K, over `n_rows` sorted rows: 128 where the tensor-core kernel takes it (32 for short lists), 64
    for the CUDA-core one. The products that share a plan must agree (take the smallest)."""
    return _fn("experts", "rllm_grouped_gemm_tile_rows")(ops._DT[dtype], int(lda), int(K), int(min(n_rows, 1 << 30)))


SCORE_FNS = {"softmax": 0, "sigmoid": 1, "softmax_chosen": 2}


def moe_topk(logits: torch.Tensor, top: int, groups: int = 1, keep: int = 1,
             renorm: bool = False, score: str = "softmax", bias: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """(chosen experts int32 [T, top], their weights float32 [T, top]) from float32 router logits [T, E];
    `score`: "softmax" over all experts, "sigmoid" of each logit by itself, or "softmax_chosen": the logits are
    ranked as they are and the weights are the softmax over the chosen ones only. `bias` float32 [E] is added to
    the logits first."""
    if bias is not None:
        _f32(bias, "router bias", (logits.shape[1],))
    if score not in SCORE_FNS:
        raise KernelError(f"router score {score!r} has no kernel (known: {sorted(SCORE_FNS)})")
    _f32(logits, "router logits")
    T, E = logits.shape
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    wt = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _check(_fn("experts", "rllm_moe_topk")(logits.data_ptr(), T, E, int(groups), int(keep), int(top), int(bool(renorm)),
                                           SCORE_FNS[score], ops._ptr(bias), idx.data_ptr(), wt.data_ptr(), _stream()), "moe_topk")
    return idx, wt


def moe_plan(idx: torch.Tensor, wt: torch.Tensor, experts: int, rows_per_tile: int = 64) -> RoutePlan:
    _i32(idx, "idx")
    _f32(wt, "wt", idx.shape)
    T, top = idx.shape
    n, dev = T * top, idx.device
    p = RoutePlan()
    p.n_rows, p.tile_rows = n, int(rows_per_tile)
    p.max_tiles = n // p.tile_rows + experts
    p.rows_tok = torch.empty(n, dtype=torch.int32, device=dev)
    p.rows_dest = torch.empty(n, dtype=torch.int32, device=dev)
    p.rows_scale = torch.empty(n, dtype=torch.float32, device=dev)
    p.tiles = torch.empty(3 * p.max_tiles, dtype=torch.int32, device=dev)
    p.n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    _check(_fn("experts", "rllm_moe_plan")(idx.data_ptr(), wt.data_ptr(), T, top, experts, p.tile_rows, p.rows_tok.data_ptr(),
                                       p.rows_dest.data_ptr(), p.rows_scale.data_ptr(), p.tiles.data_ptr(),
                                       p.n_tiles.data_ptr(), _stream()), "moe_plan")
    return p


def grouped_gemm_ragged(a: torch.Tensor, w: torch.Tensor, plan: RoutePlan, out: torch.Tensor, epilogue: int,
                        gather: bool = False, scatter: bool = False, scale: bool = False) -> torch.Tensor:
    """Per sorted row r of the plan, with e its expert: out[r'] = f(sum_k a[r''] * w[e, n, k]) where r'' is
    the row's token (`gather`) or r, r' the row's (token, slot) place (`scatter`) or r, and f the epilogue,
    times the row's weight (`scale`). w [E, N, K] contiguous of a's dtype."""
    E, N, K = w.shape
    _rows(a, "a", K)
    _rows(out, "out", N)
    _cuda(w, "w")
    if not w.is_contiguous() or w.dtype != a.dtype:
        raise KernelError("grouped product: w must be contiguous [E, N, K] of a's dtype")
    if out.dtype != (torch.float32 if epilogue == GEPI_STORE_F32 else a.dtype) or out.shape[0] < plan.n_rows:
        raise KernelError(f"grouped product: out has dtype {out.dtype} and {out.shape[0]} rows")
    if not gather and a.shape[0] < plan.n_rows:
        raise KernelError("grouped product: a has fewer rows than the plan")
    _check(_fn("experts", "rllm_grouped_gemm_ragged")(
        _dt(a, "a"), epilogue, a.data_ptr(), a.stride(0), w.data_ptr(), N * K, out.data_ptr(), out.stride(0), N, K,
        plan.tiles.data_ptr(), plan.n_tiles.data_ptr(), plan.max_tiles, plan.tile_rows,
        plan.rows_tok.data_ptr() if gather else None,
        plan.rows_dest.data_ptr() if scatter else None, plan.rows_scale.data_ptr() if scale else None, _stream()),
        "grouped_gemm_ragged")
    return out


def tc_supported(lda: int, N: int, K: int) -> bool:
    """Does the tcgen05 grouped product take a ragged product with these sizes (bfloat16, tiles of 128 rows)?"""
    return bool(_fn("experts", "rllm_grouped_gemm_tc_supported")(int(lda), int(N), int(K)))


def gather_rows_bf16(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """out[r] = x[idx[r]] for bfloat16 rows (the sorted rows a grouped product reads as one matrix)."""
    _rows(x, "x", x.shape[1])
    _i32(idx, "idx")
    if x.dtype != torch.bfloat16:
        raise KernelError("gather_rows_bf16 takes bfloat16 rows")
    out = torch.empty((idx.numel(), x.shape[1]), dtype=torch.bfloat16, device=x.device)
    _check(_fn("experts", "rllm_gather_rows_bf16")(x.data_ptr(), x.stride(0), idx.data_ptr(), out.data_ptr(), idx.numel(),
                                               x.shape[1], _stream()), "gather_rows_bf16")
    return out


def grouped_gemm_tc(a: torch.Tensor, w: torch.Tensor, plan: RoutePlan, out: torch.Tensor, epilogue: int,
                    scatter: bool = False, scale: bool = False, err: torch.Tensor | None = None, act: int = 0,
                    limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """The ragged product on tcgen05 (csrc/grouped_gemm_tc.cu): a [plan rows, K] bfloat16 in sorted order (no
    gather: see gather_rows_bf16), w [E, N, K]; epilogue GEPI_RELU2 (bfloat16 out, sorted order),
    GEPI_STORE_F32 (float out, `scatter` to the rows' places, `scale` by their weights) or GEPI_SILU_GATED (w's
    rows in blocks of 16 gate rows and their 16 up rows; bfloat16 out [rows, N / 2] = act(f g, f u), f the
    row's weight with `scale`; `act` 0 silu(g) u, 1 gelu_tanh(g) u, 2 the clamped swish with `limit` and `alpha`). The plan must have tiles of 128 rows. `err`: one int32 on the device that records a bounded wait that ran out."""
    E, N, K = w.shape
    _rows(a, "a", K)
    _rows(out, "out", N // 2 if epilogue == GEPI_SILU_GATED else N)
    _cuda(w, "w")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or plan.tile_rows != 128 \
            or a.shape[0] < plan.n_rows or epilogue not in (GEPI_RELU2, GEPI_STORE_F32, GEPI_SILU_GATED):
        raise KernelError("tcgen05 grouped product: bfloat16 operands, a plan with tiles of 128 rows, relu^2, float store or gated silu")
    if epilogue == GEPI_SILU_GATED and (N % 32 or scatter):
        raise KernelError("tcgen05 grouped product: the gated epilogue takes whole blocks of 16 + 16 rows and writes in sorted order")
    if out.dtype != (torch.float32 if epilogue == GEPI_STORE_F32 else torch.bfloat16) or out.shape[0] < plan.n_rows:
        raise KernelError(f"tcgen05 grouped product: out has dtype {out.dtype} and {out.shape[0]} rows")
    _check(_fn("experts", "rllm_grouped_gemm_tc")(
        epilogue, a.data_ptr(), a.stride(0), plan.n_rows, w.data_ptr(), E, N, K, out.data_ptr(), out.stride(0),
        plan.tiles.data_ptr(), plan.n_tiles.data_ptr(), plan.max_tiles, plan.rows_dest.data_ptr() if scatter else None,
        plan.rows_scale.data_ptr() if scale else None, _ptr(err), int(act), float(limit), float(alpha), _stream()),
        "grouped_gemm_tc")
    return out


# --------------------------------------------------------------------------- attention over latents

def latent_prepare(proj: torch.Tensor, q_off: int, dkv_off: int, heads: int, dim: int, rot: int, rank: int,
                   dims: int, wnorm: torch.Tensor, eps: float, table: torch.Tensor, slots: torch.Tensor | None,
                   cache: torch.Tensor | None, qfull: torch.Tensor) -> None:
    """See csrc/latent_attention.cu. proj [T, cols]; table float32 [T, dims/2, 2]; cache [pages, page,
    rank + rot] of proj's dtype (None with slots None: nothing is stored); qfull [T, heads, rank + rot]."""
    T = proj.shape[0]
    _rows(proj, "proj", max(q_off + heads * (dim + rot), dkv_off + rank + rot))
    _f32(wnorm, "latent norm weight", (rank,))
    _f32(table, "rotation table", (T, dims // 2, 2))
    _cuda(qfull, "qfull")
    if qfull.dtype != proj.dtype or tuple(qfull.shape) != (T, heads, rank + rot) or not qfull.is_contiguous():
        raise KernelError(f"qfull must be contiguous [{T}, {heads}, {rank + rot}] of {proj.dtype}")
    if slots is not None:
        _i32(slots, "slots", T)
        if cache is None or cache.dtype != proj.dtype or cache.dim() != 3 or cache.shape[2] != rank + rot \
                or not cache.is_contiguous():
            raise KernelError(f"the latent cache must be contiguous [pages, page, {rank + rot}] of {proj.dtype}")
    _check(_fn("mix", "rllm_latent_prepare")(
        _dt(proj, "proj"), proj.data_ptr(), proj.stride(0), q_off, dkv_off, T, heads, dim, rot, rank, dims,
        wnorm.data_ptr(), float(eps), table.data_ptr(), _ptr(slots), _ptr(cache) if slots is not None else None,
        qfull.data_ptr(), _stream()), "latent_prepare")


def latent_attention(qfull: torch.Tensor, cache: torch.Tensor, token_seq: torch.Tensor, positions: torch.Tensor,
                     block_table: torch.Tensor, rank: int, scale: float, window: int | None,
                     cu_q: torch.Tensor | None = None, num_seqs: int = 0, tensor_cores: bool = True,
                     splits: int = 1, few: bool = False) -> torch.Tensor:
    """qfull [T, heads, dk]; cache [pages, page, dk] -> [T, heads, rank] of qfull's dtype. With `cu_q`
    (int32 [num_seqs + 1], the row range of each sequence) bfloat16 problems of fitting sizes run on the
    tensor cores (`tensor_cores` False: never); `splits` > 1 there deals a row tile's keys out to that many
    CTAs and merges their parts (steps of few rows); `few` asks for the kernel shape with 16 rows a CTA (a
    token or two per sequence; taken where the rank is a multiple of 128)."""
    _cuda(qfull, "qfull"); _cuda(cache, "cache")
    T, H, dk = qfull.shape
    if not qfull.is_contiguous() or not cache.is_contiguous() or cache.dtype != qfull.dtype or cache.dim() != 3 \
            or cache.shape[2] != dk:
        raise KernelError(f"latent attention: cache must be contiguous [pages, page, {dk}] of {qfull.dtype}")
    for t, n in ((token_seq, "token_seq"), (positions, "positions")):
        _i32(t, n, T)
    if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("block_table must be int32 [sequences, pages] with unit inner stride")
    if cu_q is not None:
        _i32(cu_q, "cu_q", num_seqs + 1)
    out = torch.empty((T, H, rank), dtype=qfull.dtype, device=qfull.device)
    pacc = pml = None
    splits = max(1, min(int(splits), 32))
    few = bool(few) and rank % 128 == 0
    if splits > 1 and cu_q is not None:
        rows = 16 if few else 64
        tiles = (T * H + rows - 1) // rows + num_seqs
        pacc = torch.empty((tiles, splits, rows, rank), dtype=torch.float32, device=qfull.device)
        pml = torch.empty((tiles, splits, rows, 2), dtype=torch.float32, device=qfull.device)
    else:
        splits = 1
    _check(_fn("mix", "rllm_latent_attention")(
        _dt(qfull, "qfull"), qfull.data_ptr(), cache.data_ptr(), out.data_ptr(), token_seq.data_ptr(),
        positions.data_ptr(), block_table.data_ptr(), block_table.stride(0), T, H, rank, dk, cache.shape[1],
        float(scale), int(window or 0), _ptr(cu_q), int(num_seqs), int(bool(tensor_cores)), splits, int(few),
        _ptr(pacc), _ptr(pml), _stream()), "latent_attention", 2 if splits > 1 else 1)
    return out


# --------------------------------------------------------------------------- gated linear attention

def gla_decay(z: torch.Tensor, bias: torch.Tensor, tau: float) -> torch.Tensor:
    """z float32 [T, n] -> the decays sigmoid(z + bias)^(1/tau), in place."""
    _f32(z, "decay logits")
    _f32(bias, "decay bias", (z.shape[1],))
    _check(_fn("mix", "rllm_gla_decay")(z.data_ptr(), bias.data_ptr(), z.shape[0], z.shape[1], float(tau), _stream()),
           "gla_decay")
    return z


def gla_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, alpha: torch.Tensor, qscale: float, heads: int,
             dim: int, vdim: int, cu_q: torch.Tensor, num_seqs: int, state_slots: torch.Tensor | None,
             state: torch.Tensor, chunk: int = 0) -> torch.Tensor:
    """See csrc/gla.cu. -> float32 [T, heads, vdim]; `state` float32 [slots, heads, dim, vdim] is updated.
    `chunk` > 0: sequences are cut into chunks of that many tokens that run side by side (long portions)."""
    T = proj.shape[0]
    _rows(proj, "proj", max(q_off + heads * dim, k_off + heads * dim, v_off + heads * vdim))
    _f32(alpha, "decays", (T, heads * dim))
    _f32(state, "state")
    if state.dim() != 4 or tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError(f"state must be [slots, {heads}, {dim}, {vdim}], got {list(state.shape)}")
    _i32(cu_q, "cu_q", num_seqs + 1)
    if state_slots is not None:
        _i32(state_slots, "state_slots", num_seqs)
    out = torch.empty((T, heads, vdim), dtype=torch.float32, device=proj.device)
    cs = cd = None
    if chunk > 0:
        n = T // chunk + num_seqs
        cs = torch.empty((n, heads, dim, vdim), dtype=torch.float32, device=proj.device)
        cd = torch.empty((n, heads, dim), dtype=torch.float32, device=proj.device)
    _check(_fn("mix", "rllm_gla_scan")(
        _dt(proj, "proj"), proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, alpha.data_ptr(), float(qscale), T,
        num_seqs, heads, dim, vdim, cu_q.data_ptr(), _ptr(state_slots), state.data_ptr(), out.data_ptr(), int(chunk),
        _ptr(cs), _ptr(cd), _stream()), "gla_scan", 3 if chunk > 0 else 1)
    return out


def gla_finish(o: torch.Tensor, w: torch.Tensor, eps: float, proj: torch.Tensor, g_off: int) -> torch.Tensor:
    """o float32 [T, heads, vdim] -> [T, heads * vdim] of proj's dtype: per head o / rms(o) * w, times
    silu of the gate at proj[:, g_off + head * vdim + v]."""
    _f32(o, "o")
    T, H, vdim = o.shape
    _f32(w, "w", (vdim,))
    _rows(proj, "proj", g_off + H * vdim)
    out = torch.empty((T, H * vdim), dtype=proj.dtype, device=proj.device)
    _check(_fn("mix", "rllm_gla_finish")(_dt(proj, "proj"), o.data_ptr(), w.data_ptr(), float(eps), proj.data_ptr(),
                                         proj.stride(0), g_off, T, H, vdim, out.data_ptr(), _stream()), "gla_finish")
    return out
