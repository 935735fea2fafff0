"""Python face of the library "hybrid": recurrent mixers over a per-request state with a short causal
convolution in front (csrc/recurrent.cu), grouped-query attention whose heads' softmax weights are mixed by a
matrix (csrc/talk_attention.cu), and the row-wise work of layers whose sublayers run side by side on one normed
input (csrc/row_mix.cu). Every function checks shapes, dtypes and devices and then calls an `extern "C"`
launcher on torch's current stream; there is no CPU or library path behind them.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong

import torch

from . import ops
from .ops import KernelError, _check, _cuda, _dt, _fn, _ptr, _stream

_P, _LL = ops._P, c_longlong

ops.register_signatures("hybrid", {
    "rllm_pair_embed": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, _P, c_float, _P, c_int, c_int, c_int, c_int, c_int, _LL, _LL,
                        _P, _P],
    "rllm_combine": [_P, _P, _P, _P, _P, c_float, c_float, _P, c_int, _P, c_int, _P, c_int, c_int, c_int, _P],
    "rllm_glu_act": [_P, c_int, _LL, _P, c_int, c_int, c_int, c_int, c_float, c_float, c_int, _P],
    "rllm_add_bias_f32": [_P, _P, c_int, c_int, _P],
    "rllm_short_conv": [c_int, _P, _LL, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P],
    "rllm_unit_heads": [_P, _LL, c_int, c_int, c_int, c_float, c_float, c_int, _P],
    "rllm_softplus_decay": [c_int, _P, _LL, c_int, _P, _P, c_int, c_int, c_int, _P, _P, _P],
    "rllm_state_scan_split": [c_int],
    "rllm_state_scan": [c_int, _P, _LL, c_int, _P, _LL, c_int, _P, _LL, _P, c_int, _P, _LL, _P, _P, c_int, c_int, c_int,
                        c_int, _P, _P, _P, _P, c_int, _P],
    "rllm_gated_norm": [_P, _P, c_int, _LL, _P, c_int, c_float, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P],
    "rllm_value_norm_store": [c_int, _P, _LL, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, _P, _P, _P, c_int, _P],
    "rllm_talk_attention_simt": [c_int, _P, _LL, _P, _P, _P, _P, _P, _LL, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_float, c_int, c_int, _P],
    "rllm_talk_attention_mma_supported": [c_int, c_int, c_int, c_int, c_int],
    "rllm_gated_add": [_P, _P, _LL, _P, _P, c_float, _P, c_float, c_int, c_int, _P],
    "rllm_act_rows": [_P, c_int, _LL, _P, c_int, c_int, c_int, c_int, _P],
    "rllm_mingru_scan": [_P, _LL, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P,
                         _P, _P],
    "rllm_talk_attention_mma": [_P, _LL, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_float, c_int, c_int, _P, _P, _P],
})

GLU_ACTS = {"silu": 0, "gelu_tanh": 1, "swish_clamped": 2}
GATE_ACTS = {"silu": 0, "sigmoid": 1}


def _f32(t, name, shape=None):
    _cuda(t, name)
    if t.dtype != torch.float32 or not t.is_contiguous() or (shape is not None and tuple(t.shape) != tuple(shape)):
        raise KernelError(f"{name} must be contiguous float32" + (f" {list(shape)}" if shape is not None else "")
                          + f", got {t.dtype} {list(t.shape)}")


def _i32(t, name, n=None):
    _cuda(t, name)
    if t.dtype != torch.int32 or not t.is_contiguous() or (n is not None and t.numel() < n):
        raise KernelError(f"{name} must be a contiguous int32 vector" + (f" of at least {n}" if n is not None else ""))


def _rows(t, name, cols):
    _cuda(t, name)
    if t.dim() != 2 or t.stride(1) != 1 or t.shape[1] < cols:
        raise KernelError(f"{name} must be [rows, >= {cols}] with unit inner stride, got {list(t.shape)}")


# --------------------------------------------------------------------------- row-wise

def pair_embed(ids, positions, token_seq, cu_q, num_seqs, state_slots, prev_state, table, pair, buckets, mul_prev, mul_cur,
               norm_w, eps, err=None) -> torch.Tensor:
    """float32 [T, H]: table[id] + pair[hash of the previous token and this one] (row `buckets` for a sequence's first
    token), RMS-normed with `norm_w` (float32 [H]; None: no norm). `prev_state` int32 [slots]: the last token of each
    request's previous portion; updated with this step's last tokens. `pair` None: the table alone."""
    _i32(ids, "ids")
    T = ids.numel()
    for t, n in ((positions, "positions"), (token_seq, "token_seq")):
        _i32(t, n, T)
    _i32(cu_q, "cu_q", num_seqs + 1)
    _cuda(table, "table")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("table must be a contiguous [V, H] matrix")
    V, H = table.shape
    if pair is not None:
        _cuda(pair, "pair table")
        if pair.dtype != table.dtype or not pair.is_contiguous() or tuple(pair.shape) != (buckets + 1, H):
            raise KernelError(f"the pair table must be contiguous [{buckets + 1}, {H}] of {table.dtype}")
        if state_slots is not None:
            _i32(state_slots, "state_slots", num_seqs)
            _i32(prev_state, "previous-token state")
    if norm_w is not None:
        _f32(norm_w, "embedding norm weight", (H,))
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    keeps = pair is not None and state_slots is not None
    _check(_fn("hybrid", "rllm_pair_embed")(
        ids.data_ptr(), positions.data_ptr(), token_seq.data_ptr(), cu_q.data_ptr(), _ptr(state_slots) if keeps else None,
        _ptr(prev_state) if keeps else None, table.data_ptr(), _ptr(pair), _dt(table, "table"), _ptr(norm_w), float(eps),
        out.data_ptr(), T, int(num_seqs), H, V, int(buckets), int(mul_prev), int(mul_cur), _ptr(err), _stream()),
        "pair_embed", 2 if keeps else 1)
    return out


def combine(h, normed=(), coef=1.0, eps=1e-6, plain=()) -> torch.Tensor:
    """h (float32 [T, H], in place) += coef * sum_i w_i * a_i / rms(a_i) over `normed` (up to two (a_i, w_i) pairs,
    float32 [T, H] and [H]) + the `plain` summands (up to three float32 tensors [T, H] or [T, parts, H], each summed
    over parts in order)."""
    _f32(h, "h")
    T, H = h.shape
    if len(normed) > 2 or len(plain) > 3:
        raise KernelError("combine takes up to two normed and three plain summands")
    n = []
    for a, w in normed:
        _f32(a, "normed summand", (T, H))
        _f32(w, "its weight", (H,))
        n += [a.data_ptr(), w.data_ptr()]
    n += [None] * (4 - len(n))
    p = []
    for y in plain:
        _f32(y, "summand")
        if y.shape[0] != T or y.shape[-1] != H or y.dim() not in (2, 3):
            raise KernelError(f"a summand must be [T, H] or [T, parts, H], got {list(y.shape)}")
        p += [y.data_ptr(), 1 if y.dim() == 2 else y.shape[1]]
    p += [None, 0] * (3 - len(plain))
    _check(_fn("hybrid", "rllm_combine")(h.data_ptr(), *n, float(coef), float(eps), *p, T, H, _stream()), "combine")
    return h


def glu_act(gu, out_dtype, act: str, limit: float = 0.0, alpha: float = 1.0, block: int | None = None) -> torch.Tensor:
    """gu [R, 2F] (gate columns, then up columns, or with `block` blocks of that many gate columns each followed by
    their up columns; float32 or the run's type) -> [R, F] of `out_dtype`:
    "silu": silu(g) u; "gelu_tanh": gelu(g) u in its tanh form; "swish_clamped": with g' = min(g, limit) and
    u' = clamp(u, -limit, limit), g' sigmoid(alpha g') (u' + 1)."""
    if act not in GLU_ACTS:
        raise KernelError(f"gated activation {act!r} has no kernel (known: {sorted(GLU_ACTS)})")
    _rows(gu, "gate/up", 2)
    R, F = gu.shape[0], gu.shape[1] // 2
    if gu.shape[1] != 2 * F:
        raise KernelError("gate/up rows must hold an even number of columns")
    out = torch.empty((R, F), dtype=out_dtype, device=gu.device)
    _check(_fn("hybrid", "rllm_glu_act")(gu.data_ptr(), _dt(gu, "gate/up"), gu.stride(0), out.data_ptr(), _dt(out, "out"), R, F,
                                         GLU_ACTS[act], float(limit), float(alpha), int(block or 0), _stream()), "glu_act")
    return out


def add_bias_f32(y, bias) -> torch.Tensor:
    """y float32 [T, N] += bias float32 [N], in place."""
    _f32(y, "y")
    _f32(bias, "bias", (y.shape[1],))
    _check(_fn("hybrid", "rllm_add_bias_f32")(y.data_ptr(), bias.data_ptr(), y.shape[0], y.shape[1], _stream()), "add_bias_f32")
    return y


ROW_ACTS = {"gelu_tanh": 0}


def act_rows(x, out_dtype, act: str) -> torch.Tensor:
    """act(x) element by element for x [R, F] (float32 or the run's type; unit inner stride) -> [R, F] of `out_dtype`;
    the activation runs in float and is rounded once. "gelu_tanh": 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))."""
    if act not in ROW_ACTS:
        raise KernelError(f"activation {act!r} has no kernel (known: {sorted(ROW_ACTS)})")
    _rows(x, "x", 1)
    R, F = x.shape
    out = torch.empty((R, F), dtype=out_dtype, device=x.device)
    _check(_fn("hybrid", "rllm_act_rows")(x.data_ptr(), _dt(x, "x"), x.stride(0), out.data_ptr(), _dt(out, "out"), R, F,
                                          ROW_ACTS[act], _stream()), "act_rows")
    return out


def gated_add(h, gate, bias, terms) -> torch.Tensor:
    """h (float32 [T, W], in place) += sigmoid(gate + bias) * sum_i c_i * y_i, element by element. `gate` float32
    [T, >= W] logits (unit inner stride), `bias` float32 [W] or None, `terms` one or two (y_i float32 [T, W], c_i)."""
    _f32(h, "h")
    T, W = h.shape
    _rows(gate, "gate", W)
    if gate.dtype != torch.float32 or gate.shape[0] != T:
        raise KernelError("the gate's logits must be float32 rows, one per token")
    if bias is not None:
        _f32(bias, "gate bias", (W,))
    if not 1 <= len(terms) <= 2:
        raise KernelError("gated_add takes one or two summands")
    for y, _ in terms:
        _f32(y, "summand", (T, W))
    (y0, c0), (y1, c1) = terms[0], (terms[1] if len(terms) == 2 else (None, 0.0))
    _check(_fn("hybrid", "rllm_gated_add")(h.data_ptr(), gate.data_ptr(), gate.stride(0), _ptr(bias), y0.data_ptr(), float(c0),
                                           _ptr(y1), float(c1), T, W, _stream()), "gated_add")
    return h


# --------------------------------------------------------------------------- recurrent mixers

MINGRU_CHUNK = 32          # tokens a piece of a long portion has; portions of up to twice that run as one piece


def mingru_scan(proj, z_off, x_off, g_off, width, bias_z, bias_x, cu_q, num_seqs, state_slots, state, out_dtype,
                max_q_len: int, chunk: int | None = None) -> torch.Tensor:
    """See csrc/gated_ops.cu. proj float32 [T, cols] with the update gate's, the candidate's and the output gate's
    logits at z_off, x_off, g_off (`width` columns each); biases float32 [width] or None; `state` float32 [slots, width]
    is updated. -> [T, width] of `out_dtype`: S_t * silu(g_t). Portions longer than two chunks are cut into pieces that
    run side by side (`chunk` None: MINGRU_CHUNK; 0: never)."""
    _rows(proj, "proj", max(z_off, x_off, g_off) + width)
    if proj.dtype != torch.float32:
        raise KernelError("mingru_scan takes float32 projections")
    T = proj.shape[0]
    for b, n in ((bias_z, "update bias"), (bias_x, "candidate bias")):
        if b is not None:
            _f32(b, n, (width,))
    _i32(cu_q, "cu_q", num_seqs + 1)
    if state_slots is not None:
        _i32(state_slots, "state_slots", num_seqs)
        _f32(state, "state")
        if state.dim() != 2 or state.shape[1] != width:
            raise KernelError(f"state must be [slots, {width}], got {list(state.shape)}")
    chunk = MINGRU_CHUNK if chunk is None else int(chunk)
    if max_q_len <= 2 * chunk:
        chunk = 0
    ca = cb = s0 = None
    if chunk > 0:
        ca = torch.empty((T // chunk + num_seqs, width), dtype=torch.float32, device=proj.device)
        cb = torch.empty_like(ca)
        s0 = torch.empty((num_seqs, width), dtype=torch.float32, device=proj.device)
    out = torch.empty((T, width), dtype=out_dtype, device=proj.device)
    _check(_fn("hybrid", "rllm_mingru_scan")(
        proj.data_ptr(), proj.stride(0), int(z_off), int(x_off), int(g_off), _ptr(bias_z), _ptr(bias_x), cu_q.data_ptr(),
        _ptr(state_slots), _ptr(state) if state_slots is not None else None, out.data_ptr(), _dt(out, "out"), T, int(num_seqs),
        int(width), chunk, _ptr(ca), _ptr(cb), _ptr(s0), _stream()), "mingru_scan", 2 if chunk > 0 else 1)
    return out

def short_conv(x, col0, channels, w, bias, token_seq, positions, cu_q, num_seqs, state_slots, tail, silu=True) -> torch.Tensor:
    """Causal convolution over time per channel of columns [col0, col0 + channels) of x [T, cols]: float32
    [T, channels], y[t, c] = act(bias[c] + sum_j w[c, j] x[t - (taps - 1 - j), c]). `tail` float32
    [slots, taps - 1, channels]: each request's last inputs, read for the rows before a portion and updated."""
    T = x.shape[0]
    _rows(x, "x", col0 + channels)
    _f32(w, "convolution weight")
    if w.dim() != 2 or w.shape[0] != channels:
        raise KernelError(f"the convolution weight must be [{channels}, taps], got {list(w.shape)}")
    taps = w.shape[1]
    if bias is not None:
        _f32(bias, "convolution bias", (channels,))
    for t, n in ((token_seq, "token_seq"), (positions, "positions")):
        _i32(t, n, T)
    _i32(cu_q, "cu_q", num_seqs + 1)
    if state_slots is not None:
        _i32(state_slots, "state_slots", num_seqs)
        _f32(tail, "convolution tail")
        if taps > 1 and (tail.dim() != 3 or tuple(tail.shape[1:]) != (taps - 1, channels)):
            raise KernelError(f"the convolution tail must be [slots, {taps - 1}, {channels}], got {list(tail.shape)}")
    out = torch.empty((T, channels), dtype=torch.float32, device=x.device)
    keeps = state_slots is not None and taps > 1
    _check(_fn("hybrid", "rllm_short_conv")(
        _dt(x, "x"), x.data_ptr(), x.stride(0), int(col0), int(channels), taps, w.data_ptr(), _ptr(bias), token_seq.data_ptr(),
        positions.data_ptr(), cu_q.data_ptr(), _ptr(state_slots), _ptr(tail) if state_slots is not None else None,
        out.data_ptr(), T, int(num_seqs), int(bool(silu)), _stream()), "short_conv", 2 if keeps else 1)
    return out


def unit_heads(x, col0, heads, dim, scale=1.0, eps=1e-6) -> torch.Tensor:
    """In place on float32 x [T, cols]: each of the `heads` vectors of `dim` numbers from column col0 becomes
    scale * v / sqrt(sum(v^2) + eps)."""
    _cuda(x, "x")
    if x.dtype != torch.float32:
        raise KernelError("unit_heads works on float32 rows")
    _rows(x, "x", col0 + heads * dim)
    _check(_fn("hybrid", "rllm_unit_heads")(x.data_ptr(), x.stride(0), int(col0), int(heads), int(dim), float(scale), float(eps),
                                            x.shape[0], _stream()), "unit_heads")
    return x


def softplus_decay(z, col0, n, bias, a_log, want_step=False):
    """d = softplus(z[:, col0 + c] + bias[c]) and a = exp(-exp(a_log[c // (n / len(a_log))]) d) for c < n, in float.
    Returns (d or None, a), each float32 [T, n]."""
    _rows(z, "z", col0 + n)
    if bias is not None:
        _f32(bias, "step bias", (n,))
    _f32(a_log, "a_log")
    if n % a_log.numel():
        raise KernelError(f"{n} columns do not divide over {a_log.numel()} heads")
    T = z.shape[0]
    step = torch.empty((T, n), dtype=torch.float32, device=z.device) if want_step else None
    decay = torch.empty((T, n), dtype=torch.float32, device=z.device)
    _check(_fn("hybrid", "rllm_softplus_decay")(_dt(z, "z"), z.data_ptr(), z.stride(0), int(col0), _ptr(bias), a_log.data_ptr(), T,
                                                int(n), n // a_log.numel(), _ptr(step), decay.data_ptr(), _stream()),
           "softplus_decay")
    return step, decay


def state_scan(q, q_heads, k, k_heads, v, decay, heads, dim, vdim, cu_q, num_seqs, state_slots, state, beta=None, vscale=None,
               skip=None, channels: int = 0) -> torch.Tensor:
    """See csrc/recurrent.cu. q [T, q_heads * dim], k [T, k_heads * dim], v [T, heads * vdim]: float32 views with unit
    inner stride; decay float32 [T, heads * dim] (per channel) or [T, heads]; beta: logits [T, heads] of the
    projection's type (delta rule) or None (plain); vscale float32 [T, heads]; skip float32 [heads].
    -> float32 [T, heads, vdim]; `state` float32 [slots, heads, dim, vdim] is updated. `channels` (32, 16 or 8): key
    channels a thread where the kernel with compiled sizes runs, for measurements; 0: chosen from the sizes."""
    T = q.shape[0]
    for t, n, c in ((q, "q", q_heads * dim), (k, "k", k_heads * dim), (v, "v", heads * vdim)):
        _rows(t, n, c)
        if t.dtype != torch.float32:
            raise KernelError(f"{n} must be float32")
    _f32(decay, "decays")
    per_channel = tuple(decay.shape) == (T, heads * dim) and dim > 1
    if not per_channel and tuple(decay.shape) != (T, heads):
        raise KernelError(f"decays must be [T, {heads * dim}] or [T, {heads}], got {list(decay.shape)}")
    _f32(state, "state")
    if state.dim() != 4 or tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError(f"state must be [slots, {heads}, {dim}, {vdim}], got {list(state.shape)}")
    _i32(cu_q, "cu_q", num_seqs + 1)
    if state_slots is not None:
        _i32(state_slots, "state_slots", num_seqs)
    if beta is not None:
        _rows(beta, "beta", heads)
    if vscale is not None:
        _f32(vscale, "value scale", (T, heads))
    if skip is not None:
        _f32(skip, "skip", (heads,))
    out = torch.empty((T, heads, vdim), dtype=torch.float32, device=q.device)
    _check(_fn("hybrid", "rllm_state_scan")(
        _dt(beta, "beta") if beta is not None else 0, q.data_ptr(), q.stride(0), int(q_heads), k.data_ptr(), k.stride(0),
        int(k_heads), v.data_ptr(), v.stride(0), decay.data_ptr(), int(per_channel), _ptr(beta),
        beta.stride(0) if beta is not None else 0, _ptr(vscale), _ptr(skip), int(num_seqs), int(heads), int(dim), int(vdim),
        cu_q.data_ptr(), _ptr(state_slots), state.data_ptr(), out.data_ptr(), int(channels), _stream()), "state_scan")
    return out


def gated_norm(y, gate, gate_col0, weight, eps, groups, out_dtype, gate_first: bool, act: str) -> torch.Tensor:
    """y float32 [T, n] in `groups` equal parts, each divided by its own root mean square, times `weight` (float32, of
    n numbers or of one part's size, then shared by the parts). The gate act(gate[:, gate_col0 + c]) multiplies y before
    the norm (`gate_first`) or the result after it; act "silu" or "sigmoid". -> [T, n] of `out_dtype`."""
    _f32(y, "y")
    T, n = y.shape
    if n % groups:
        raise KernelError(f"{n} columns do not form {groups} equal parts")
    _f32(weight, "norm weight")
    if weight.numel() not in (n, n // groups):
        raise KernelError(f"the norm weight must hold {n} or {n // groups} numbers")
    if act not in GATE_ACTS:
        raise KernelError(f"gate activation {act!r} has no kernel (known: {sorted(GATE_ACTS)})")
    g = None
    if gate is not None:
        _rows(gate, "gate", gate_col0 + n)
        g = gate.data_ptr() + gate_col0 * gate.element_size()
    out = torch.empty((T, n), dtype=out_dtype, device=y.device)
    _check(_fn("hybrid", "rllm_gated_norm")(y.data_ptr(), g, _dt(gate, "gate") if gate is not None else 0,
                                            gate.stride(0) if gate is not None else 0, weight.data_ptr(), weight.numel(),
                                            float(eps), out.data_ptr(), _dt(out, "out"), T, int(groups), n // groups,
                                            int(bool(gate_first)), GATE_ACTS[act], _stream()), "gated_norm")
    return out


# --------------------------------------------------------------------------- attention with mixed heads

def _caches(kcache, vcache, dtype, nkv):
    for c, n in ((kcache, "kcache"), (vcache, "vcache")):
        _cuda(c, n)
        if c.dtype != dtype or c.dim() != 4 or not c.is_contiguous():
            raise KernelError(f"{n} must be contiguous [pages, kv heads, page, size] of {dtype}")
    if kcache.shape[:3] != vcache.shape[:3] or kcache.shape[1] != nkv:
        raise KernelError("key and value pages must agree in pages, kv heads and page size")


def value_norm_store(proj, k_off, v_off, nkv, kd, vd, eps, norm, slots, kcache, vcache) -> None:
    """Keys (nkv heads of kd at column k_off of proj) as they are and values (nkv of vd at v_off), each value head
    divided by its root mean square if `norm`, into their pages at `slots` (-1 for a token: not stored)."""
    _rows(proj, "proj", max(k_off + nkv * kd, v_off + nkv * vd))
    if slots is None:
        return
    _i32(slots, "slots", proj.shape[0])
    _caches(kcache, vcache, proj.dtype, nkv)
    if kcache.shape[3] != kd or vcache.shape[3] != vd:
        raise KernelError(f"pages hold keys of {kcache.shape[3]} and values of {vcache.shape[3]}, not {kd} and {vd}")
    _check(_fn("hybrid", "rllm_value_norm_store")(_dt(proj, "proj"), proj.data_ptr(), proj.stride(0), int(k_off), int(v_off),
                                                  proj.shape[0], nkv, kd, vd, float(eps), int(bool(norm)), slots.data_ptr(),
                                                  kcache.data_ptr(), vcache.data_ptr(), kcache.shape[2], _stream()),
           "value_norm_store")


def talk_attention_simt(q, kcache, vcache, token_seq, positions, block_table, nh, scale, mix, window=None, chunk=None,
                        sinks=None) -> torch.Tensor:
    """Attention of every query row over its sequence's pages with the heads' softmax weights mixed by `mix` (float32
    [nh, nh]: row h holds head h's share of every head's weights), in float on the CUDA cores. q [T, nh * kd] (a view
    with a longer row stride is fine) -> [T, nh * vd] of q's dtype. `sinks` float32 [nh]: exp(sink) joins each head's
    denominator."""
    _cuda(q, "q")
    T = q.shape[0]
    nkv = kcache.shape[1]
    _caches(kcache, vcache, q.dtype, nkv)
    _, _, page_size, kd = kcache.shape
    vd = vcache.shape[3]
    if q.dim() != 2 or q.stride(1) != 1 or q.shape[1] != nh * kd:
        raise KernelError(f"q must be [T, {nh * kd}] with unit inner stride, got {list(q.shape)}")
    for t, n in ((token_seq, "token_seq"), (positions, "positions")):
        _i32(t, n, T)
    if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("block_table must be int32 [sequences, pages] with unit inner stride")
    _f32(mix, "head mix", (nh, nh))
    if sinks is not None:
        _f32(sinks, "sinks", (nh,))
    out = torch.empty((T, nh * vd), dtype=q.dtype, device=q.device)
    _check(_fn("hybrid", "rllm_talk_attention_simt")(
        _dt(q, "q"), q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(), token_seq.data_ptr(), positions.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), mix.data_ptr(), _ptr(sinks), out.data_ptr(), T, nh, nkv, kd, vd, page_size,
        float(scale), int(window or 0), int(chunk or 0), _stream()), "talk_attention_simt")
    return out


def talk_mma_supported(dtype, nh, kd, vd, page_size) -> bool:
    return bool(_fn("hybrid", "rllm_talk_attention_mma_supported")(_dt_of(dtype), nh, kd, vd, page_size))


def _dt_of(dtype) -> int:
    return {torch.float32: ops.DT_F32, torch.bfloat16: ops.DT_BF16}.get(dtype, -1)


def talk_attention_mma(q, kcache, vcache, token_seq, positions, block_table, cu_q, num_seqs, max_q_len, nh, scale, mix,
                       window=None, chunk=None, sinks=None) -> torch.Tensor:
    """The same attention in bfloat16 on the tensor cores (`mma.sync`, float softmax). The mix is applied after the
    values: a first kernel leaves, as floats, every head's weights summed over every kv head's values ([T, nh, nkv,
    vd], one pass with a running softmax), a second one adds them by `mix` and rounds once. `cu_q` int32
    [num_seqs + 1]: each sequence's rows; `max_q_len`: the longest portion of the step."""
    _cuda(q, "q")
    T = q.shape[0]
    nkv = kcache.shape[1]
    _caches(kcache, vcache, q.dtype, nkv)
    _, _, page_size, kd = kcache.shape
    vd = vcache.shape[3]
    if q.dim() != 2 or q.stride(1) != 1 or q.shape[1] != nh * kd:
        raise KernelError(f"q must be [T, {nh * kd}] with unit inner stride, got {list(q.shape)}")
    if not talk_mma_supported(q.dtype, nh, kd, vd, page_size):
        raise KernelError(f"talk_attention_mma: bfloat16 with head sizes in steps of 16 up to 128, got {q.dtype} {kd}/{vd}")
    _i32(positions, "positions", T)
    _i32(cu_q, "cu_q", num_seqs + 1)
    if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("block_table must be int32 [sequences, pages] with unit inner stride")
    _f32(mix, "head mix", (nh, nh))
    if sinks is not None:
        _f32(sinks, "sinks", (nh,))
    parts = torch.empty((T, nh, nkv, vd), dtype=torch.float32, device=q.device)
    out = torch.empty((T, nh * vd), dtype=q.dtype, device=q.device)
    _check(_fn("hybrid", "rllm_talk_attention_mma")(
        q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(), out.data_ptr(), parts.data_ptr(), positions.data_ptr(),
        cu_q.data_ptr(), block_table.data_ptr(), block_table.stride(0), int(num_seqs), T, int(max_q_len), nh, nkv, kd, vd,
        page_size, float(scale), int(window or 0), int(chunk or 0), mix.data_ptr(), _ptr(sinks), _stream()),
        "talk_attention_mma", 2)
    return out
