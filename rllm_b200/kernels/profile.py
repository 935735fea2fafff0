"""Per-operation timing of the launch-by-launch path, switched on with RLLM_B200_PROFILE=1.

Every backend operation (embedding, norm, the q/k/v product with rotation and cache write,
attention, the output, gate/up and down products, the head, sampling) is bracketed by a pair of
CUDA events on the launching stream; the pairs are read when a report is asked for, so that no
operation waits for a measurement. With the switch on, decode steps do not replay CUDA graphs
(events cannot sit inside a replayed graph), so the step times are those of the launch-by-launch
path: the shares say where a step's time goes, the absolute times are not the serving path's.
A report lists, per class, calls, mean microseconds, the bytes and FLOPs the operation has to move
and do (counted from its operands' shapes) and what fraction of the measured copy bandwidth or
tensor throughput that is.

The counterpart of the reference's RLLM_PROFILE timers (src/model/profile.rs:19-100, call sites
src/model/registry/llama.rs:159-258), which bracket the same classes with a device synchronize.
"""
from __future__ import annotations

import json
import os
import sys
from collections import OrderedDict

import torch


def enabled() -> bool:
    return os.environ.get("RLLM_B200_PROFILE") == "1"


def _peaks() -> tuple[float, float]:
    """(copy bandwidth in bytes/s, bf16 tensor throughput in FLOP/s): the measured ones if the file
    with them lies beside the package, else the nominal 7.7 TB/s and 2.25 PFLOP/s."""
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        return m["hbm_gbs"] * 1e9, m["bf16_tflops"] * 1e12
    except (OSError, KeyError, ValueError):
        return 7.7e12, 2.25e15


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if isinstance(t, torch.Tensor))


class OpProfile:
    """Wraps a `Backend`: the same methods, each timed under a class name."""

    # backend method -> (class name, function of (args, kwargs, result) -> (bytes, flops))
    def __init__(self, backend):
        self._be = backend
        self.classes: OrderedDict[str, list] = OrderedDict()     # name -> [calls, bytes, flops, [event pairs]]
        self._free: list = []
        self.tokens = 0

    def __getattr__(self, name):
        return getattr(self._be, name)

    # ---- bookkeeping
    def _timed(self, cls: str, nbytes: int, flops: int, fn, *a, **k):
        if torch.cuda.is_current_stream_capturing():
            return fn(*a, **k)
        e0, e1 = self._free.pop() if self._free else (torch.cuda.Event(enable_timing=True),
                                                      torch.cuda.Event(enable_timing=True))
        e0.record()
        out = fn(*a, **k)
        e1.record()
        rec = self.classes.setdefault(cls, [0, 0, 0, [], 0.0])
        rec[0] += 1; rec[1] += nbytes; rec[2] += flops; rec[3].append((e0, e1))
        return out

    def _settle(self) -> None:
        torch.cuda.synchronize(self._be.device)
        for rec in self.classes.values():
            for e0, e1 in rec[3]:
                rec[4] += e0.elapsed_time(e1) * 1e3           # microseconds
                self._free.append((e0, e1))
            rec[3] = []

    def report(self, file=None, reset: bool = True) -> dict:
        """Print the table (to stderr by default) and return it as a dict."""
        self._settle()
        bw, tf = _peaks()
        total = sum(r[4] for r in self.classes.values()) or 1.0
        out = {}
        lines = [f"[rllm profile] {'class':<12}{'calls':>8}{'mean us':>10}{'share':>8}{'GB/s':>9}{'of copy':>9}"
                 f"{'TFLOP/s':>9}{'of peak':>9}"]
        for name, (calls, nbytes, flops, _, us) in self.classes.items():
            if not calls:
                continue
            sec = us * 1e-6
            gbs, tfl = nbytes / sec / 1e9 if sec else 0.0, flops / sec / 1e12 if sec else 0.0
            out[name] = {"calls": calls, "mean_us": us / calls, "share": us / total, "gbs": gbs, "hbm_frac": gbs * 1e9 / bw,
                         "tflops": tfl, "tensor_frac": tfl * 1e12 / tf}
            lines.append(f"[rllm profile] {name:<12}{calls:>8}{us / calls:>10.1f}{us / total:>8.1%}{gbs:>9.0f}"
                         f"{gbs * 1e9 / bw:>9.2f}{tfl:>9.1f}{tfl * 1e12 / tf:>9.3f}")
        print("\n".join(lines), file=file or sys.stderr, flush=True)
        if reset:
            self.classes.clear()
        return out

    # ---- the backend's operations
    def embed(self, ids, table, err=None, scale=1.0):
        return self._timed("embed", ids.numel() * table.shape[1] * (table.element_size() + 4), 0,
                           self._be.embed, ids, table, err=err, scale=scale)

    def rmsnorm(self, x, w, eps, out_dtype=None, rows=None):
        T = x.shape[0] if rows is None else rows.numel()
        return self._timed("norm", T * x.shape[1] * 6, 0, self._be.rmsnorm, x, w, eps, out_dtype, rows)

    def _product(self, cls, x, w, fn, *a, **k):
        T = x.shape[0]
        return self._timed(cls, _nbytes(w) + T * (w.shape[0] + w.shape[1]) * 2, 2 * T * w.shape[0] * w.shape[1],
                           fn, *a, **k)

    def linear(self, x, w, bias=None, tag=None):
        return self._product(tag or "linear", x, w, self._be.linear, x, w, bias=bias)

    def linear_f32(self, x, w, tag=None):
        return self._product(tag or "head", x, w, self._be.linear_f32, x, w)

    def linear_residual(self, x, w, residual):
        cls = "o" if w.shape[0] >= w.shape[1] else "down"       # a square or widening product: the mixer's output
        return self._product(cls, x, w, self._be.linear_residual, x, w, residual)

    def linear_swiglu(self, x, w_gate_up):
        return self._product("gate_up", x, w_gate_up, self._be.linear_swiglu, x, w_gate_up)

    def qkv_rope_cache_write(self, x, w_qkv, *a, **k):
        return self._product("qkv+rope", x, w_qkv, self._be.qkv_rope_cache_write, x, w_qkv, *a, **k)

    def rope_cache_write(self, qkv, *a, **k):
        return self._timed("rope", 2 * _nbytes(qkv), 0, self._be.rope_cache_write, qkv, *a, **k)

    def attention(self, q, cache, ctx, nh, scale, window):
        hd = q.shape[1] // nh
        nkv = cache.k.shape[1] if cache.k is not None else nh
        lens, qs = ctx.kv_lens_host, ctx.q_lens_host
        if lens is None:
            lens, qs = [ctx.max_kv_len] * ctx.num_seqs, [1] * ctx.num_seqs
        seen = [min(L, window + q - 1) if window else L for L, q in zip(lens, qs)]
        pairs = sum(q * (s - q) + q * (q + 1) // 2 for s, q in zip(seen, qs))
        nbytes = sum(seen) * nkv * hd * 2 * cache.k.element_size() + 2 * _nbytes(q)
        return self._timed("attention", nbytes, 4 * nh * hd * pairs, self._be.attention, q, cache, ctx, nh, scale, window)

    # ---- mixers with latents or a recurrent state, routed feed-forwards
    def rmsnorm_add(self, residual, y, w, eps):
        return self._timed("norm+add", _nbytes(y) + 2 * _nbytes(residual), 0, self._be.rmsnorm_add, residual, y, w, eps)

    def linear_heads(self, a, a_gs, w, out, c_gs, f32=False, gate=None):
        T, (G, N, K) = a.shape[0], w.shape
        return self._timed("heads", _nbytes(w) + T * G * (N + K) * a.element_size(), 2 * T * G * N * K,
                           self._be.linear_heads, a, a_gs, w, out, c_gs, f32=f32, gate=gate)

    def expert_tile_rows(self, *a):
        return self._be.expert_tile_rows(*a)

    def route(self, logits, *a, **k):
        return self._timed("route", 2 * _nbytes(logits), 0, self._be.route, logits, *a, **k)

    def experts_up(self, x, w_up, plan, act="relu2"):
        E, F, W = w_up.shape
        return self._timed("experts_up", _nbytes(w_up) + plan.n_rows * (F + W) * x.element_size(), 2 * plan.n_rows * F * W,
                           self._be.experts_up, x, w_up, plan, act)

    def experts_down(self, a, w_down, plan, T, top, scale=True):
        E, W, F = w_down.shape
        return self._timed("experts_down", _nbytes(w_down) + plan.n_rows * (F * a.element_size() + 4 * W),
                           2 * plan.n_rows * F * W, self._be.experts_down, a, w_down, plan, T, top, scale)

    def experts_gated_up(self, x, w_gate_up, plan, block=None):
        E, F2, W = w_gate_up.shape
        return self._timed("experts_up", _nbytes(w_gate_up) + plan.n_rows * (F2 // 2 + W) * x.element_size(),
                           2 * plan.n_rows * F2 * W, self._be.experts_gated_up, x, w_gate_up, plan, block)

    # ---- layers that norm after the sum, attention with sink, gate and block mask
    def stream_copy(self, h):
        return self._timed("cast", 6 * h.numel(), 0, self._be.stream_copy, h)

    def postnorm(self, h, y, *a, **k):
        parts = y.parts if hasattr(y, "parts") else y
        return self._timed("add+norm", _nbytes(parts, getattr(y, "extra", None)) + 10 * h.numel(), 0, self._be.postnorm, h, y, *a, **k)

    def linear_act(self, x, w, act):
        return self._product("up", x, w, self._be.linear_act, x, w, act)

    def qk_norm_rope_store(self, proj, *a, **k):
        return self._timed("qk_norm+rope", 2 * _nbytes(proj), 0, self._be.qk_norm_rope_store, proj, *a, **k)

    def sink_attention(self, q, cache, ctx, nh, scale, window, chunk, sinks, gate, keep_first=0, sigmoid=False):
        kd, vd, nkv = cache.k.shape[3], cache.v.shape[3], cache.k.shape[1]
        lens, qs = ctx.kv_lens_host, ctx.q_lens_host
        if lens is None:
            lens, qs = [ctx.max_kv_len] * ctx.num_seqs, [1] * ctx.num_seqs
        pairs = seen_keys = 0
        for n, ql in zip(lens, qs):
            first = n
            for pos in range(n - ql, n):
                lo = max(0, pos - window + 1) if window else 0
                if chunk:
                    lo = max(lo, pos // chunk * chunk)
                pairs += pos - lo + 1 + min(keep_first, lo)
                first = min(first, lo)
            seen_keys += n - first + min(keep_first, first)
        nbytes = seen_keys * nkv * (kd + vd) * cache.k.element_size() + _nbytes(q) + q.shape[0] * nh * vd * q.element_size()
        return self._timed("sigmoid_attention" if sigmoid else "attention", nbytes, 2 * nh * (kd + vd) * pairs,
                           self._be.sink_attention, q, cache, ctx, nh, scale, window, chunk, sinks, gate, keep_first, sigmoid)

    def latent_prepare(self, proj, *a, **k):
        return self._timed("latent_prepare", 2 * _nbytes(proj), 0, self._be.latent_prepare, proj, *a, **k)

    def latent_attention(self, qfull, cache, ctx, rank, scale, window):
        T, H, dk = qfull.shape
        lens, qs = ctx.kv_lens_host, ctx.q_lens_host
        if lens is None:
            lens, qs = [ctx.max_kv_len] * ctx.num_seqs, [1] * ctx.num_seqs
        seen = [min(L, window + q - 1) if window else L for L, q in zip(lens, qs)]
        pairs = sum(q * (s - q) + q * (q + 1) // 2 for s, q in zip(seen, qs))
        nbytes = sum(seen) * dk * qfull.element_size() + _nbytes(qfull) + T * H * rank * qfull.element_size()
        return self._timed("latent_attention", nbytes, 2 * H * (dk + rank) * pairs, self._be.latent_attention,
                           qfull, cache, ctx, rank, scale, window)

    def gla_decay(self, z, bias, tau):
        return self._timed("gla_decay", 2 * _nbytes(z), 0, self._be.gla_decay, z, bias, tau)

    def gla_scan(self, proj, q_off, k_off, v_off, alpha, qscale, heads, dim, vdim, cu_q, num_seqs, slots, state, chunk=0):
        T = proj.shape[0]
        nbytes = T * heads * (2 * dim + vdim) * proj.element_size() + _nbytes(alpha) + T * heads * vdim * 4 \
            + 2 * num_seqs * heads * dim * vdim * 4
        return self._timed("gla_scan", nbytes, 5 * T * heads * dim * vdim, self._be.gla_scan, proj, q_off, k_off, v_off,
                           alpha, qscale, heads, dim, vdim, cu_q, num_seqs, slots, state, chunk)

    def gla_finish(self, o, *a, **k):
        return self._timed("gla_finish", 2 * _nbytes(o), 0, self._be.gla_finish, o, *a, **k)

    # ---- library "hybrid"
    def pair_embed(self, ctx, table, *a, **k):
        return self._timed("embed", ctx.token_ids.numel() * table.shape[1] * (2 * table.element_size() + 4), 0,
                           self._be.pair_embed, ctx, table, *a, **k)

    def combine(self, h, *outputs):
        n = 2
        for y in outputs:
            n += len(y.terms) if hasattr(y, "terms") else 0 if y is None else 1
        return self._timed("norm+add", n * _nbytes(h), 0, self._be.combine, h, *outputs)

    def linear_glu(self, x, w_gate_up, act, limit=0.0, alpha=1.0):
        return self._product("gate_up+act", x, w_gate_up, self._be.linear_glu, x, w_gate_up, act, limit, alpha)

    def experts_glu_up(self, x, w_gate_up, plan, act, limit=0.0, alpha=1.0, block=None):
        rows, (E, F2, K) = plan.n_rows, w_gate_up.shape
        return self._timed("experts_up", _nbytes(w_gate_up) + rows * (K * 2 + F2 * 4 + F2), 2 * rows * F2 * K,
                           self._be.experts_glu_up, x, w_gate_up, plan, act, limit, alpha, block)

    def short_conv(self, x, col0, channels, *a, **k):
        return self._timed("short_conv", x.shape[0] * channels * (x.element_size() + 4), 0, self._be.short_conv, x, col0,
                           channels, *a, **k)

    def unit_heads(self, x, col0, heads, dim, *a, **k):
        return self._timed("scan_gates", x.shape[0] * heads * dim * 8, 0, self._be.unit_heads, x, col0, heads, dim, *a, **k)

    def softplus_decay(self, z, col0, n, *a, **k):
        return self._timed("scan_gates", z.shape[0] * n * (z.element_size() + 4), 0, self._be.softplus_decay, z, col0, n, *a, **k)

    def state_scan(self, q, q_heads, k, k_heads, v, decay, heads, dim, vdim, ctx, state, beta=None, vscale=None, skip=None):
        T = q.shape[0]
        nbytes = T * (heads * (2 * dim + 2 * vdim) * 4) + _nbytes(decay) + 2 * ctx.num_seqs * heads * dim * vdim * 4
        flops = (7 if beta is not None else 5) * T * heads * dim * vdim
        return self._timed("state_scan", nbytes, flops, self._be.state_scan, q, q_heads, k, k_heads, v, decay, heads, dim,
                           vdim, ctx, state, beta, vscale, skip)

    def gated_norm(self, y, *a, **k):
        return self._timed("gated_norm", _nbytes(y) * 7 // 4, 0, self._be.gated_norm, y, *a, **k)

    def value_norm_store(self, proj, k_off, v_off, nkv, kd, vd, *a, **k):
        return self._timed("value_norm", 2 * proj.shape[0] * nkv * (kd + vd) * proj.element_size(), 0,
                           self._be.value_norm_store, proj, k_off, v_off, nkv, kd, vd, *a, **k)

    def talk_attention(self, q, cache, ctx, nh, scale, mix, window, chunk, sinks):
        kd, vd, nkv = cache.k.shape[3], cache.v.shape[3], cache.k.shape[1]
        lens, qs = ctx.kv_lens_host, ctx.q_lens_host
        if lens is None:
            lens, qs = [ctx.max_kv_len] * ctx.num_seqs, [1] * ctx.num_seqs
        seen = [min(L, window + n - 1) if window else L for L, n in zip(lens, qs)]
        pairs = sum(n * (s - n) + n * (n + 1) // 2 for s, n in zip(seen, qs))
        nbytes = sum(seen) * nkv * (kd + vd) * cache.k.element_size() + _nbytes(q) + q.shape[0] * nh * vd * q.element_size()
        return self._timed("talk_attention", nbytes, 2 * nh * (kd + vd) * pairs, self._be.talk_attention, q, cache, ctx, nh,
                           scale, mix, window, chunk, sinks)

    def gated_add(self, h, gate, bias, y):
        n = 3 + (len(y.terms) if hasattr(y, "terms") else 1)       # the stream read and written, the gate, the summands
        return self._timed("gate+add", n * _nbytes(h), 0, self._be.gated_add, h, gate, bias, y)

    def mingru_scan(self, proj, z_off, x_off, g_off, width, bias_z, bias_x, ctx, state):
        T = proj.shape[0]
        pieces = 2 if ctx.max_q_len > 64 else 1                    # long portions read the gates' logits twice
        nbytes = T * width * (4 * (1 + 2 * pieces) + self._be.dtype.itemsize) + 8 * ctx.num_seqs * width
        return self._timed("gru_scan", nbytes, 0, self._be.mingru_scan, proj, z_off, x_off, g_off, width, bias_z, bias_x, ctx,
                           state)

    def argmax(self, logits):
        return self._timed("sample", _nbytes(logits), 0, self._be.argmax, logits)

    def sample(self, logits, *a, **k):
        return self._timed("sample", _nbytes(logits), 0, self._be.sample, logits, *a, **k)

    def logprobs(self, logits, *a, **k):
        return self._timed("sample", _nbytes(logits), 0, self._be.logprobs, logits, *a, **k)
