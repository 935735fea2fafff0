"""Python face of the library "sink": grouped-query attention with a per-head norm of queries and keys,
a rotation of part of a head, keys and values of different sizes, a window and/or block mask, a sink in
the softmax and an output gate (csrc/sink_attention.cu), and the row-wise work of layers that norm after
the sum (csrc/stream_ops.cu). Every function checks shapes, dtypes and devices and then calls an
`extern "C"` launcher on torch's current stream; there is no CPU or library path behind them.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong

import torch

from . import ops
from .ops import KernelError, _check, _cuda, _dt, _fn, _ptr, _stream

_P, _LL = ops._P, c_longlong

ops.register_signatures("sink", {
    "rllm_qk_norm_rope_store": [c_int, _P, _LL, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P,
                                c_float, _P, _P, _P, _P, c_int, _P, _LL, _P, _P],
    "rllm_sink_attention_simt": [c_int, _P, _LL, _P, _P, _P, _LL, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_float, c_int, c_int, _P, _P, c_int, c_int, c_int, _P],
    "rllm_sink_attention_mma_supported": [c_int, c_int, c_int, c_int],
    "rllm_sink_attention_mma": [_P, _LL, _P, _P, _P, _LL, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_int, c_float, c_int, c_int, _P, _P, c_int, c_int, _P, _P, c_int, c_int, _P],
    "rllm_postnorm": [_P, _P, c_int, _P, _P, c_int, c_float, _P, c_int, c_int, c_float, _P, c_int, _P],
    "rllm_cast_rows": [_P, _P, _LL, _P],
    "rllm_gated_act": [_P, c_int, _LL, _P, c_int, c_int, c_int, c_int, _P, _P],
    "rllm_relu2": [_P, c_int, _LL, _P],
})


def _f32(t, name, shape=None):
    _cuda(t, name)
    if t.dtype != torch.float32 or not t.is_contiguous() or (shape is not None and tuple(t.shape) != tuple(shape)):
        raise KernelError(f"{name} must be contiguous float32" + (f" {list(shape)}" if shape is not None else "")
                          + f", got {t.dtype} {list(t.shape)}")


def _i32(t, name, n=None):
    _cuda(t, name)
    if t.dtype != torch.int32 or not t.is_contiguous() or (n is not None and t.numel() < n):
        raise KernelError(f"{name} must be a contiguous int32 vector" + (f" of at least {n}" if n is not None else ""))


def _caches(kcache, vcache, dtype, nkv=None):
    for c, n in ((kcache, "kcache"), (vcache, "vcache")):
        _cuda(c, n)
        if c.dtype != dtype or c.dim() != 4 or not c.is_contiguous():
            raise KernelError(f"{n} must be contiguous [pages, kv heads, page, size] of {dtype}")
    if kcache.shape[:3] != vcache.shape[:3] or (nkv is not None and kcache.shape[1] != nkv):
        raise KernelError("key and value pages must agree in pages, kv heads and page size")


def qk_norm_rope_store(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, nh: int, nkv: int, kd: int, vd: int,
                       rot: int, wq: torch.Tensor | None, wk: torch.Tensor | None, eps: float,
                       table: torch.Tensor | None, slots: torch.Tensor | None, kcache: torch.Tensor | None,
                       vcache: torch.Tensor | None, vfirst: torch.Tensor | None = None, lam: torch.Tensor | None = None) -> None:
    """proj [T, cols] holds q (nh heads of kd at q_off), k (nkv of kd at k_off) and v (nkv of vd at v_off). Per
    head: q and k divided by their root mean square times `wq` / `wk` (float [kd]; None: no norm), then the
    first `rot` dimensions rotated (dimension i with i + rot/2) by `table` float [T, rot/2, 2] (cos, sin); q is
    written back in place, k and v go to their pages at `slots` (None, or -1 for a token: not stored). `vfirst` (rows of
    proj's type, [T, nkv * vd], a view with a longer row stride is fine) and `lam` (one float32 on the device): what is
    stored as the value is (1 - lam) v + lam vfirst, formed in float and rounded once; proj keeps v as it was."""
    _cuda(proj, "proj")
    T = proj.shape[0]
    need = max(q_off + nh * kd, k_off + nkv * kd, v_off + nkv * vd)
    if proj.dim() != 2 or proj.stride(1) != 1 or proj.shape[1] < need:
        raise KernelError(f"proj must be [T, >= {need}] with unit inner stride, got {list(proj.shape)}")
    for w, n in ((wq, "query norm weight"), (wk, "key norm weight")):
        if w is not None:
            _f32(w, n, (kd,))
    if rot:
        if table is None:
            raise KernelError("a rotation needs the step's table of cos and sin")
        _f32(table, "rotation table", (T, rot // 2, 2))
    page_size = 1
    if slots is not None:
        _i32(slots, "slots", T)
        _caches(kcache, vcache, proj.dtype, nkv)
        if kcache.shape[3] != kd or vcache.shape[3] != vd:
            raise KernelError(f"pages hold keys of {kcache.shape[3]} and values of {vcache.shape[3]}, not {kd} and {vd}")
        page_size = kcache.shape[2]
    if (vfirst is None) != (lam is None):
        raise KernelError("values are mixed with rows and a coefficient, or not at all")
    if vfirst is not None:
        _cuda(vfirst, "vfirst")
        _f32(lam, "lam")
        if vfirst.dtype != proj.dtype or vfirst.dim() != 2 or vfirst.stride(1) != 1 or tuple(vfirst.shape) != (T, nkv * vd) \
                or lam.numel() != 1:
            raise KernelError(f"vfirst must be [{T}, {nkv * vd}] of {proj.dtype} with unit inner stride, lam one number")
    _check(_fn("sink", "rllm_qk_norm_rope_store")(
        _dt(proj, "proj"), proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, T, nh, nkv, kd, vd, rot, _ptr(wq),
        _ptr(wk), float(eps), _ptr(table) if rot else None, _ptr(slots), _ptr(kcache) if slots is not None else None,
        _ptr(vcache) if slots is not None else None, page_size, _ptr(vfirst), 0 if vfirst is None else vfirst.stride(0),
        _ptr(lam), _stream()), "qk_norm_rope_store")


def _attention_args(q, kcache, vcache, token_seq, positions, block_table, nh, sinks, gate):
    _cuda(q, "q")
    T = q.shape[0]
    _caches(kcache, vcache, q.dtype)
    _, nkv, page_size, kd = kcache.shape
    vd = vcache.shape[3]
    if q.dim() != 2 or q.stride(1) != 1 or q.shape[1] != nh * kd:
        raise KernelError(f"q must be [T, {nh * kd}] with unit inner stride, got {list(q.shape)}")
    if nh % nkv:
        raise KernelError(f"{nh} query heads do not divide over {nkv} kv heads")
    for t, n in ((token_seq, "token_seq"), (positions, "positions")):
        _i32(t, n, T)
    if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("block_table must be int32 [sequences, pages] with unit inner stride")
    if sinks is not None:
        _f32(sinks, "sinks", (nh,))
    if gate is not None:
        _cuda(gate, "gate")
        if gate.dtype != torch.float32 or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < nh:
            raise KernelError(f"the gate must be float32 [T, >= {nh}] with unit inner stride")
    return T, nkv, page_size, kd, vd


def sink_attention_simt(q, kcache, vcache, token_seq, positions, block_table, nh, scale, window=None, chunk=None,
                        sinks=None, gate=None, keep_first: int = 0, sigmoid: bool = False) -> torch.Tensor:
    """Attention of every query row over its sequence's pages, in float on the CUDA cores. q [T, nh * kd] (a view
    with a longer row stride is fine); kcache [pages, nkv, page, kd]; vcache [pages, nkv, page, vd] -> [T, nh * vd]
    of q's dtype. A query at position p sees j <= p with j > p - window (if `window`) and j // chunk == p // chunk
    (if `chunk`), and besides every j <= p below `keep_first`. `sinks` float [nh]: exp(sink) joins the denominator.
    `sigmoid`: no softmax, a visible key's weight is sigmoid(score + sinks[head]) (`sinks` None: no bias). `gate` float
    [T, >= nh]: logits of the output gate."""
    T, nkv, page_size, kd, vd = _attention_args(q, kcache, vcache, token_seq, positions, block_table, nh, sinks, gate)
    out = torch.empty((T, nh * vd), dtype=q.dtype, device=q.device)
    _check(_fn("sink", "rllm_sink_attention_simt")(
        _dt(q, "q"), q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(), out.data_ptr(), out.stride(0),
        token_seq.data_ptr(), positions.data_ptr(), block_table.data_ptr(), block_table.stride(0), T, nh, nkv, kd, vd,
        page_size, float(scale), int(window or 0), int(chunk or 0), _ptr(sinks), _ptr(gate),
        0 if gate is None else gate.stride(0), int(keep_first or 0), int(bool(sigmoid)), _stream()), "sink_attention_simt")
    return out


def mma_supported(dtype: torch.dtype, kd: int, vd: int, page_size: int) -> bool:
    """Does the tensor-core kernel take these sizes (bfloat16; head sizes multiples of 16 up to 128)?"""
    return dtype == torch.bfloat16 and bool(_fn("sink", "rllm_sink_attention_mma_supported")(ops.DT_BF16, kd, vd, page_size))


def sink_attention_mma(q, kcache, vcache, token_seq, positions, block_table, cu_q, num_seqs, max_q_len, nh, scale,
                       window=None, chunk=None, sinks=None, gate=None, splits: int = 1, max_keys: int = 0,
                       keep_first: int = 0, sigmoid: bool = False) -> torch.Tensor:
    """The same attention in bfloat16 on the tensor cores (`mma.sync`, float softmax): row tiles of 64 (query,
    head-of-a-group) rows per sequence and kv head; `splits` > 1 deals a tile's keys out to that many CTAs in
    fixed ranges (steps of few rows) whose parts a second kernel merges in order. `cu_q` int32 [num_seqs + 1];
    `max_keys`: a bound of the keys any query of the step sees (what `splits` cuts up). `keep_first`, `sigmoid`: as in
    `sink_attention_simt`."""
    T, nkv, page_size, kd, vd = _attention_args(q, kcache, vcache, token_seq, positions, block_table, nh, sinks, gate)
    if not mma_supported(q.dtype, kd, vd, page_size):
        raise KernelError(f"sink_attention_mma: bfloat16 with head sizes in steps of 16 up to 128, got {q.dtype} {kd}/{vd}")
    _i32(cu_q, "cu_q", num_seqs + 1)
    out = torch.empty((T, nh * vd), dtype=q.dtype, device=q.device)
    splits = max(1, min(int(splits), 64))
    pacc = pml = None
    if splits > 1:
        pacc = torch.empty((T * nh, splits, vd), dtype=torch.float32, device=q.device)
        pml = torch.empty((T * nh, splits, 2), dtype=torch.float32, device=q.device)
    _check(_fn("sink", "rllm_sink_attention_mma")(
        q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(), out.data_ptr(), out.stride(0),
        positions.data_ptr(), cu_q.data_ptr(), block_table.data_ptr(), block_table.stride(0), int(num_seqs), T,
        int(max_q_len), nh, nkv, kd, vd, page_size, float(scale), int(window or 0), int(chunk or 0), _ptr(sinks),
        _ptr(gate), 0 if gate is None else gate.stride(0), splits, _ptr(pacc), _ptr(pml), int(keep_first or 0),
        int(bool(sigmoid)), _stream()), "sink_attention_mma", 2 if splits > 1 else 1)
    return out


# --------------------------------------------------------------------------- the stream of post-norm layers

def postnorm(h: torch.Tensor, y: torch.Tensor | None, alpha: float, w: torch.Tensor, eps: float,
             y2: torch.Tensor | None = None, y2_gate: torch.Tensor | None = None,
             copy: torch.Tensor | None = None) -> torch.Tensor:
    """h [T, H] float, in place: s = alpha * h + sum over parts of y ([T, H] or [T, parts, H] float, parts added in
    order) + sigmoid(y2_gate[t]) * y2[t] (y2 [T, H] float; y2_gate float [T, >= 1], its first column); then
    h = w * s / sqrt(mean(s^2) + eps). `copy` [T, H] (bfloat16 or float32) also receives the new h."""
    _f32(h, "h")
    T, H = h.shape
    parts = 0
    if y is not None:
        parts = 1 if y.dim() == 2 else y.shape[1]
        _f32(y, "y", (T, H) if y.dim() == 2 else (T, parts, H))
    _f32(w, "w", (H,))
    if y2 is not None:
        _f32(y2, "y2", (T, H))
    if y2_gate is not None:
        _cuda(y2_gate, "y2_gate")
        if y2 is None or y2_gate.dtype != torch.float32 or y2_gate.dim() != 2 or y2_gate.shape[0] != T:
            raise KernelError("postnorm: the gate of the second summand must be float32 [T, >= 1] beside y2")
    if copy is not None:
        _cuda(copy, "copy")
        if tuple(copy.shape) != (T, H) or not copy.is_contiguous():
            raise KernelError(f"postnorm: copy must be contiguous [{T}, {H}]")
    _check(_fn("sink", "rllm_postnorm")(h.data_ptr(), _ptr(y), parts, _ptr(y2), _ptr(y2_gate),
                                        0 if y2_gate is None else y2_gate.stride(0), float(alpha), w.data_ptr(), T, H,
                                        float(eps), _ptr(copy), 0 if copy is None else _dt(copy, "copy"), _stream()),
           "postnorm")
    return h


def cast_rows(h: torch.Tensor) -> torch.Tensor:
    """The float stream as bfloat16 (round to nearest even)."""
    _f32(h, "h")
    out = torch.empty(h.shape, dtype=torch.bfloat16, device=h.device)
    _check(_fn("sink", "rllm_cast_rows")(h.data_ptr(), out.data_ptr(), h.numel(), _stream()), "cast_rows")
    return out


def gated_act(gu: torch.Tensor, out_dtype: torch.dtype, row_scale: torch.Tensor | None = None,
              block: int | None = None) -> torch.Tensor:
    """out[r, i] = silu(f_r * g) * (f_r * u) for gu [R, 2F] (float32 or bfloat16), f_r = row_scale[r] (float [R])
    or 1. The columns of gu: all F gate columns, then all up columns (`block` None), or blocks of `block` gate
    columns each followed by their up columns."""
    _cuda(gu, "gu")
    if gu.dim() != 2 or gu.stride(1) != 1 or gu.shape[1] % 2:
        raise KernelError("gated_act takes [R, 2F] with unit inner stride")
    R, F = gu.shape[0], gu.shape[1] // 2
    if row_scale is not None:
        _f32(row_scale, "row_scale")
        if row_scale.numel() < R:
            raise KernelError("gated_act: one scale per row")
    block = F if block is None else int(block)
    if block <= 0 or F % block:
        raise KernelError(f"gated_act: blocks of {block} do not divide {F} columns")
    out = torch.empty((R, F), dtype=out_dtype, device=gu.device)
    _check(_fn("sink", "rllm_gated_act")(gu.data_ptr(), _dt(gu, "gu"), gu.stride(0), out.data_ptr(), _dt(out, "out"), R, F,
                                         block, _ptr(row_scale), _stream()), "gated_act")
    return out


def relu2_(x: torch.Tensor) -> torch.Tensor:
    """x <- max(x, 0)^2 in place."""
    _cuda(x, "x")
    if not x.is_contiguous():
        raise KernelError("relu2_ takes a contiguous tensor")
    _check(_fn("sink", "rllm_relu2")(x.data_ptr(), _dt(x, "x"), x.numel(), _stream()), "relu2")
    return x
