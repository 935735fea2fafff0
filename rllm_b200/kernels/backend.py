"""Chooses the kernel for each operation of a run.

`Backend(torch.float32)` is the true 32-bit path: float storage everywhere and
FMA kernels only. `Backend(torch.bfloat16)` is the serving path: bfloat16
weights, activations and cache, float residual stream and logits; it sends
matrix products to the tcgen05 kernel and attention to the tiled kernels when
those take the sizes at hand, and to the generic CUDA-core kernels otherwise.
Both are hand-written CUDA; there is nothing else to fall back to.
"""
from __future__ import annotations

import os

import torch

from . import ops


class Normed:
    """An RMSNorm that has not run yet: rows of the float residual stream, the norm's weight and
    eps. A product that can take the norm in front of it in one kernel consumes it as it is;
    everything else calls `tensor()`, which runs the norm kernel once and keeps the result."""

    def __init__(self, backend, h, weight, eps, rows=None):
        self.backend, self.h, self.weight, self.eps, self.rows = backend, h, weight, float(eps), rows
        self._tensor = None

    @property
    def shape(self):
        return (self.h.shape[0] if self.rows is None else self.rows.numel(), self.h.shape[1])

    def tensor(self):
        if self._tensor is None:
            self._tensor = self.backend.rmsnorm(self.h, self.weight, self.eps, rows=self.rows)
        return self._tensor


class Backend:
    def __init__(self, dtype: torch.dtype, device: torch.device | str = "cuda:0"):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"run dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ops.KernelError("the engine runs on a CUDA device only (there is no CPU path)")
        self.fast = dtype == torch.bfloat16 and os.environ.get("RLLM_B200_GENERIC_ONLY") != "1"
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._sm100 = None
        if self.fast:
            from . import sm100          # builds/loads the tcgen05 library, or raises
            self._sm100 = sm100
            sm100.init(self.device)

    # ---- element-wise / row-wise
    def embed(self, ids, table, err=None, scale=1.0):
        return ops.embed(ids, table, err=err, scale=scale)

    def rmsnorm(self, x, w, eps, out_dtype=None, rows=None):
        return ops.rmsnorm(x, w, eps, out_dtype or self.dtype, rows=rows)

    def normed(self, h, weight, eps, rows=None):
        """rmsnorm(h[rows]) for a consumer that may fuse it: deferred on the serving path, computed
        at once on the 32-bit path."""
        n = Normed(self, h, weight, eps, rows)
        return n if self._sm100 is not None else n.tensor()

    def _fused_norm(self, x, w, gate_up=False):
        """Take the norm into the product? Every CTA of the product then normalises its own slice of
        the rows, which pays while the weight has no more 128-row tiles than the GPU has SMs; a
        wider weight (the output head) gets the norm from its own kernel, once. So does a gate/up
        pair from 33 tokens on: its faster kernel there (tokens on the accumulator's rows, no ranges
        of K to merge) takes no norm in front (64 tokens: 14.8 us + the norm's 2 against 19.4)."""
        if gate_up and isinstance(x, Normed) and x.shape[0] > 32:
            return False
        if not (isinstance(x, Normed) and x._tensor is None and self._sm100 is not None and w.shape[0] % 4 == 0
                and os.environ.get("RLLM_B200_NO_NORM_FUSION") != "1"
                and self._sm100.norm_supported(x.h, x.weight, w, x.rows)):
            return False
        # the kernel for steps of at most 8 tokens builds the normalised rows once per CTA whatever
        # the width (a CTA walks many slabs of the weight)
        return (w.shape[0] + 127) // 128 <= self._sm100.init(self.device).sm_count or \
            self._sm100.stream_supported(ops.EPI_STORE_F32, True, x.shape[0], w.shape[0], w.shape[1])

    def gather_rows(self, x, rows):
        return ops.gather_rows(x, rows)

    def add_into(self, residual, delta):
        return ops.add_into(residual, delta)

    # ---- matrix products: y = x W^T
    def _tc(self, x, w):
        # weights whose height is no multiple of 4 (a gate row per head, say) stay on the CUDA cores
        return self._sm100 is not None and w.shape[0] % 4 == 0 and self._sm100.gemm_supported(x, w)

    def linear(self, x, w, bias=None, tag=None):
        # `tag` names the product for per-operation timing (kernels/profile.py); it changes nothing here
        if bias is None and self._fused_norm(x, w):
            return self._sm100.gemm_norm(x.h, x.weight, x.eps, w, ops.EPI_STORE, rows=x.rows)
        x = x.tensor() if isinstance(x, Normed) else x
        if self._tc(x, w):
            # a bias is added after the product (a small kernel): the product stays on the tensor cores
            y = self._sm100.gemm(x, w, ops.EPI_STORE)
            return y if bias is None else ops.add_bias(y, bias)
        return ops.gemm_simt(x, w, ops.EPI_STORE, bias=bias)

    def linear_f32(self, x, w, tag=None):
        if w.shape[0] <= ops.SKINNY_MAX:         # a gate row, a handful of heads: a warp a token
            return ops.gemm_skinny(x.tensor() if isinstance(x, Normed) else x, w)
        if self._fused_norm(x, w):
            return self._sm100.gemm_norm(x.h, x.weight, x.eps, w, ops.EPI_STORE_F32, rows=x.rows)
        x = x.tensor() if isinstance(x, Normed) else x
        if self._tc(x, w):
            return self._sm100.gemm(x, w, ops.EPI_STORE_F32)
        return ops.gemm_simt(x, w, ops.EPI_STORE_F32)

    def linear_residual(self, x, w, residual):
        """residual (float32, in place) += x W^T"""
        x = x.tensor() if isinstance(x, Normed) else x
        if self._tc(x, w):
            return self._sm100.gemm(x, w, ops.EPI_ACCUM_F32, out=residual)
        return ops.gemm_simt(x, w, ops.EPI_ACCUM_F32, out=residual)

    def linear_swiglu(self, x, w_gate_up):
        """silu(x Wg^T) * (x Wu^T) with w_gate_up = [Wg; Wu]"""
        if self._fused_norm(x, w_gate_up, gate_up=True):
            return self._sm100.gemm_norm(x.h, x.weight, x.eps, w_gate_up, ops.EPI_SWIGLU, rows=x.rows)
        x = x.tensor() if isinstance(x, Normed) else x
        if self._tc(x, w_gate_up):
            return self._sm100.gemm(x, w_gate_up, ops.EPI_SWIGLU)
        return ops.gemm_simt(x, w_gate_up, ops.EPI_SWIGLU)

    # ---- position encoding + cache write, attention
    def rope_table(self, ctx, positions, inv_freq, rot_dim, key=None):
        """The step's (cos, sin) table for one rotation rule, made at its first use in a forward
        pass and shared by the layers with the same rule (`key`)."""
        if ctx is None:
            return None
        tables = ctx.per_forward.setdefault("rope_tables", {})
        key = key if key is not None else (inv_freq.data_ptr(), rot_dim)
        t = tables.get(key)
        if t is None:
            t = tables[key] = ops.rope_table(positions, inv_freq[: rot_dim // 2].contiguous(), ctx.num_tokens)
        return t

    def qkv_rope_cache_write(self, x, w_qkv, bias, positions, inv_freq, cache, nh, nkv, hd, rot_dim=None,
                             ctx=None, key=None):
        """qkv = x w_qkv^T (+ bias), q and k rotated, k and v written to the cache. One kernel when
        the tensor-core product takes the sizes, else the product followed by the rotation kernel."""
        rot_dim = hd if rot_dim is None else rot_dim
        table = self.rope_table(ctx, positions, inv_freq, rot_dim, key)
        kc = cache.k if cache.writes else None
        if bias is None and self._fused_norm(x, w_qkv) and x.rows is None and 128 % hd == 0 and \
                (kc is None or kc.dtype == torch.bfloat16):
            writes = cache.writes
            return self._sm100.gemm_qkv_rope(None, w_qkv, positions, inv_freq, cache.slots if writes else None,
                                             kc, cache.v if writes else None, nh, nkv, hd, cache.page_size,
                                             rot_dim, norm=(x.h, x.weight, x.eps), table=table)
        x = x.tensor() if isinstance(x, Normed) else x
        if bias is None and self._sm100 is not None and \
                self._sm100.qkv_rope_supported(x, w_qkv, cache.k if cache.writes else None, hd, rot_dim):
            writes = cache.writes
            return self._sm100.gemm_qkv_rope(x, w_qkv, positions, inv_freq, cache.slots if writes else None,
                                             cache.k if writes else None, cache.v if writes else None,
                                             nh, nkv, hd, cache.page_size, rot_dim, table=table)
        qkv = self.linear(x, w_qkv, bias=bias)
        self.rope_cache_write(qkv, positions, inv_freq, cache, nh, nkv, hd, rot_dim, ctx=ctx, key=key)
        return qkv

    def rope_cache_write(self, qkv, positions, inv_freq, cache, nh, nkv, hd, rot_dim=None, ctx=None, key=None):
        writes = cache.writes
        rot_dim = hd if rot_dim is None else rot_dim
        table = self.rope_table(ctx, positions, inv_freq, rot_dim, key)
        ops.rope_cache_write(qkv, positions, inv_freq, cache.slots if writes else None,
                             cache.k if writes else None, cache.v if writes else None,
                             nh, nkv, hd, cache.page_size, rot_dim, table=table)

    def attention(self, q, cache, ctx, nh, scale, window):
        if self._sm100 is not None:
            out = self._sm100.attention(q, cache, ctx, nh, scale, window)
            if out is not None:
                return out
        return ops.paged_attention_simt(q, cache.k, cache.v, ctx.token_seq, ctx.positions,
                                        cache.block_table, nh, scale, window)

    # ---- mixers with a cache of latents or a recurrent state, routed feed-forwards (library "mix")
    @property
    def _mix(self):
        from . import mix
        return mix

    def rmsnorm_add(self, residual, y, w, eps):
        """residual += rmsnorm(y) * w (y [T, H], or [T, parts, H] summed over parts first), in float."""
        return self._mix.rmsnorm_add(residual, y, w, eps)

    def add_row(self, h, v):
        return self._mix.add_row(h, v)

    def linear_heads(self, a, a_gs, w, out, c_gs, f32=False, gate=None):
        """One product per head in one launch: out[:, g*c_gs + n] = a[:, g*a_gs : g*a_gs + K] w[g]^T."""
        return self._mix.grouped_gemm_uniform(a, a_gs, w, out, c_gs,
                                              self._mix.GEPI_STORE_F32 if f32 else self._mix.GEPI_STORE, gate=gate)

    def expert_tile_rows(self, x, w_up, w_down, n_rows):
        """Rows per tile of a plan that the up and the down product of a routed feed-forward share."""
        up = self._mix.tile_rows(x.dtype, x.stride(0), w_up.shape[2], n_rows)
        down = self._mix.tile_rows(x.dtype, w_down.shape[2], w_down.shape[2], n_rows)
        return up if up == down else 64         # one of them stays on the CUDA cores: both take its tiles

    def route(self, logits, top, groups=1, keep=1, renorm=False, tile_rows=64, score="softmax", bias=None):
        """Router logits (plus a float bias per expert) -> the plan of the experts' grouped products (all on the device)."""
        idx, wt = self._mix.moe_topk(logits, top, groups, keep, renorm, score, bias)
        return idx, wt, self._mix.moe_plan(idx, wt, logits.shape[1], tile_rows)

    def _tc_experts(self, a, w, plan):
        """Long row lists in bfloat16 go to the tcgen05 grouped product (RLLM_B200_NO_TC_EXPERTS=1: never)."""
        return self._sm100 is not None and plan.tile_rows == 128 and a.dtype == torch.bfloat16 \
            and os.environ.get("RLLM_B200_NO_TC_EXPERTS") != "1" and self._mix.tc_supported(a.stride(0), w.shape[1], w.shape[2])

    def experts_up(self, x, w_up, plan, act="relu2"):
        """act(x[token of row] W_up[expert of row]^T) for every sorted row of the plan."""
        if act != "relu2":
            raise ops.KernelError(f"expert activation {act!r} has no kernel")
        out = torch.empty((plan.n_rows, w_up.shape[1]), dtype=x.dtype, device=x.device)
        if self._tc_experts(x, w_up, plan):
            rows = self._mix.gather_rows_bf16(x, plan.rows_tok)       # the sorted rows as a matrix of their own: TMA boxes
            return self._mix.grouped_gemm_tc(rows, w_up, plan, out, self._mix.GEPI_RELU2,
                                             err=self._sm100.init(self.device).err)
        return self._mix.grouped_gemm_ragged(x, w_up, plan, out, self._mix.GEPI_RELU2, gather=True)

    def experts_gated_up(self, x, w_gate_up, plan, block=None):
        """silu(f g) * (f u) for every sorted row of the plan, with g and u the row's token times the gate and up
        rows of the row's expert and f the row's weight: the weight on the expert's input, applied in float to the
        two linear projections. W [E, 2F, K]: an expert's gate rows, then its up rows (`block` None), or blocks of
        `block` gate rows each followed by their up rows (16: the tcgen05 kernel then activates in its epilogue)."""
        F2 = w_gate_up.shape[1]
        if self._tc_experts(x, w_gate_up, plan):
            rows = self._mix.gather_rows_bf16(x, plan.rows_tok)
            if block == 16:
                out = torch.empty((plan.n_rows, F2 // 2), dtype=torch.bfloat16, device=x.device)
                return self._mix.grouped_gemm_tc(rows, w_gate_up, plan, out, self._mix.GEPI_SILU_GATED, scale=True,
                                                 err=self._sm100.init(self.device).err)
            gu = torch.empty((plan.n_rows, F2), dtype=torch.float32, device=x.device)
            self._mix.grouped_gemm_tc(rows, w_gate_up, plan, gu, self._mix.GEPI_STORE_F32,
                                      err=self._sm100.init(self.device).err)
        else:
            gu = torch.empty((plan.n_rows, F2), dtype=torch.float32, device=x.device)
            self._mix.grouped_gemm_ragged(x, w_gate_up, plan, gu, self._mix.GEPI_STORE_F32, gather=True)
        return self._sink.gated_act(gu, x.dtype, plan.rows_scale, block)

    def experts_down(self, a, w_down, plan, T, top, scale=True):
        """(weight of row, if `scale`) * (a[row] W_down[expert of row]^T), stored at the row's (token, slot):
        float [T, top, width], every place written exactly once."""
        out = torch.empty((T * top, w_down.shape[1]), dtype=torch.float32, device=a.device)
        if self._tc_experts(a, w_down, plan):
            self._mix.grouped_gemm_tc(a, w_down, plan, out, self._mix.GEPI_STORE_F32, scatter=True, scale=scale,
                                      err=self._sm100.init(self.device).err)
        else:
            self._mix.grouped_gemm_ragged(a, w_down, plan, out, self._mix.GEPI_STORE_F32, scatter=True, scale=scale)
        return out.view(T, top, w_down.shape[1])

    # ---- layers that norm after the sum; attention with query/key norm, sink, gate and block mask (library "sink")
    @property
    def _sink(self):
        from . import sink
        return sink

    def stream_copy(self, h):
        """The float stream in the run's storage type: what a sublayer that reads the stream itself multiplies."""
        return h if self.dtype == torch.float32 else self._sink.cast_rows(h)

    def postnorm(self, h, y, alpha, w, eps):
        """h <- w * s / rms(s), s = alpha h + y, in float and in place; y a float tensor [T, H] / [T, parts, H] or
        `Summands`. Returns the new stream in the run's storage type (h itself in the 32-bit run)."""
        parts, extra, gate = (y.parts, y.extra, y.extra_gate) if hasattr(y, "parts") else (y, None, None)
        copy = None if self.dtype == torch.float32 else torch.empty(h.shape, dtype=self.dtype, device=h.device)
        self._sink.postnorm(h, parts, alpha, w, eps, extra, gate, copy)
        return h if copy is None else copy

    def linear_act(self, x, w, act):
        """act(x W^T) in the run dtype; act "relu2" = max(., 0)^2, "gelu_tanh" = gelu in its tanh form (on the float
        product, rounded once)."""
        if act not in ("relu2", "gelu_tanh"):
            raise ops.KernelError(f"activation {act!r} has no kernel")
        fuse = os.environ.get("RLLM_B200_NO_ACT_FUSION") != "1"
        if fuse and self._fused_norm(x, w):                                  # the norm in front, the activation behind
            return self._sm100.gemm_norm(x.h, x.weight, x.eps, w, ops.EPI_STORE, rows=x.rows, act=act)
        x = x.tensor() if isinstance(x, Normed) else x
        if self._tc(x, w) and fuse:
            return self._sm100.gemm(x, w, ops.EPI_STORE, act=act)            # in the product's store epilogue
        if act == "gelu_tanh":
            return self._hy.act_rows(self.linear_f32(x, w, tag="up"), self.dtype, act)
        if self._tc(x, w):
            return self._sink.relu2_(self._sm100.gemm(x, w, ops.EPI_STORE))
        return ops.gemm_simt(x, w, ops.EPI_RELU2)

    def qk_norm_rope_store(self, proj, q_off, k_off, v_off, nh, nkv, kd, vd, rot, wq, wk, eps, table, cache, vfirst=None,
                           lam=None):
        """`vfirst`, `lam`: the values are cached as (1 - lam) v + lam vfirst (another layer's values of the same tokens)."""
        writes = cache.writes
        self._sink.qk_norm_rope_store(proj, q_off, k_off, v_off, nh, nkv, kd, vd, rot, wq, wk, eps, table,
                                      cache.slots if writes else None, cache.k if writes else None,
                                      cache.v if writes else None, vfirst if writes else None, lam if writes else None)

    def sink_attention(self, q, cache, ctx, nh, scale, window, chunk, sinks, gate, keep_first=0, sigmoid=False):
        """Attention with a window and/or block mask, a sink and an output gate over pages whose keys and values
        may differ in size: bfloat16 on the tensor cores where the kernel takes the sizes, else (and in the
        32-bit run) in float on the CUDA cores. `keep_first`: positions below it are seen whatever the window says.
        `sigmoid`: no softmax, a visible key's weight is sigmoid(score + sinks[head])."""
        sk = self._sink
        kd, vd, nkv = cache.k.shape[3], cache.v.shape[3], cache.k.shape[1]
        tc = self.fast and os.environ.get("RLLM_B200_NO_TC_ATTENTION") != "1"
        # keys a query of this step can see at most, known without a device read (graph captures included)
        keys = ctx.max_kv_len
        if window:
            keys = min(keys, window + ctx.max_q_len + keep_first)
        if chunk:
            keys = min(keys, chunk)
        G = nh // nkv
        if tc and kd == vd and self._sm100.attention_supported(q, cache.k):
            # equal head sizes of 64 or 128: the kernels of plain grouped-query attention take the mask, the sink
            # and the gate as well (the clusters of the decode kernel, tcgen05 for long portions); kept first keys and
            # sigmoid weights only the tcgen05 kernel does
            sm = self._sm100
            if ctx.max_q_len == 1 and not keep_first and not sigmoid and sm.decode_supported(q, cache.k, nh):
                return sm.attention_decode(q, cache.k, cache.v, ctx.kv_lens, cache.block_table, nh, scale, window, keys,
                                           chunk=chunk, sinks=sinks, gate=gate)
            lens = ctx.q_lens_host
            if ctx.max_q_len * G >= 128 and ctx.max_kv_len >= sm.TC_ATTENTION_MIN_KEYS and sm.prefill_tc_supported(q, cache.k) \
                    and lens is not None and min(lens) * G >= 128:
                return sm.attention_prefill_tc(q, cache.k, cache.v, ctx.cu_q, ctx.kv_lens, cache.block_table, ctx.max_q_len,
                                               nh, scale, window, chunk=chunk, sinks=sinks, gate=gate, keep_first=keep_first,
                                               sigmoid=sigmoid)
        if tc and sk.mma_supported(q.dtype, kd, vd, cache.page_size):
            tiles = 0
            for ql in (ctx.q_lens_host if not ctx.graph_safe else [1] * ctx.num_seqs):
                tiles += (ql * G + 63) // 64
            tiles *= nkv
            # ranges of keys per row tile: up to four CTAs an SM are resident, a range is at least 128 keys
            splits = max(1, min(16, 4 * self.sm_count // max(tiles, 1), keys // 128))
            return sk.sink_attention_mma(q, cache.k, cache.v, ctx.token_seq, ctx.positions, cache.block_table, ctx.cu_q,
                                         ctx.num_seqs, ctx.max_q_len, nh, scale, window, chunk, sinks, gate, splits, keys,
                                         keep_first, sigmoid)
        return sk.sink_attention_simt(q, cache.k, cache.v, ctx.token_seq, ctx.positions, cache.block_table, nh, scale,
                                      window, chunk, sinks, gate, keep_first, sigmoid)

    def latent_prepare(self, *a, **k):
        return self._mix.latent_prepare(*a, **k)

    def latent_attention(self, qfull, cache, ctx, rank, scale, window):
        # Steps of few rows (decoding) have fewer row tiles than the GPU has SMs: the keys of a tile are then
        # dealt out to several CTAs, at least four key tiles (128 keys) each; steps of a token or two per
        # sequence take the kernel shape with 16 rows a CTA. Everything this depends on is known when a decode
        # graph is captured (rows, sequences, the longest portion, the bound of the key count).
        T, H = qfull.shape[0], qfull.shape[1]
        few = ctx.max_q_len <= 2 and rank % 128 == 0
        rows = 16 if few else 64
        tiles = max(1, T * H // rows)               # row tiles the step has at least
        keys = min(window, ctx.max_kv_len) if window else ctx.max_kv_len
        splits = max(1, min(16, self.sm_count // tiles, keys // 128))
        return self._mix.latent_attention(qfull, cache.tensors["kv"], ctx.token_seq, ctx.positions,
                                          cache.block_table, rank, scale, window, cu_q=ctx.cu_q, num_seqs=ctx.num_seqs,
                                          tensor_cores=self.fast and os.environ.get("RLLM_B200_NO_TC_ATTENTION") != "1",
                                          splits=splits, few=few)

    def gla_decay(self, z, bias, tau):
        return self._mix.gla_decay(z, bias, tau)

    def gla_scan(self, *a, **k):
        return self._mix.gla_scan(*a, **k)

    def gla_finish(self, *a, **k):
        return self._mix.gla_finish(*a, **k)

    # ---- recurrent mixers with a short convolution, attention with mixed heads, layers whose sublayers run side by
    # side (library "hybrid")
    @property
    def _hy(self):
        from . import hybrid
        return hybrid

    def pair_embed(self, ctx, table, pair, buckets, mul_prev, mul_cur, norm_w, eps, prev_state):
        """The embedded rows plus the rows of a table addressed by a hash of each token and the one before it, normed."""
        return self._hy.pair_embed(ctx.token_ids, ctx.positions, ctx.token_seq, ctx.cu_q, ctx.num_seqs,
                                   ctx.state_slots if prev_state is not None else None, prev_state, table, pair, buckets,
                                   mul_prev, mul_cur, norm_w, eps, err=ctx.extras.get("err_flag"))

    def combine(self, h, *outputs):
        """h += the sublayers' outputs, in float and in one pass. An output is a float tensor [T, H] / [T, parts, H],
        `Summands` (parts and an ungated second summand) or `NormedSum` (summands that are RMS-normed first)."""
        normed, plain, coef, eps = [], [], 1.0, 1e-6
        for y in outputs:
            if y is None:
                continue
            if hasattr(y, "terms"):
                if normed:
                    raise ops.KernelError("combine takes the normed summands of one sublayer")
                normed, coef, eps = list(y.terms), y.coef, y.eps
            elif hasattr(y, "parts"):
                if y.extra_gate is not None:
                    raise ops.KernelError("combine takes no gated summand")
                plain += [t for t in (y.parts, y.extra) if t is not None]
            else:
                plain.append(y)
        return self._hy.combine(h, normed, coef, eps, plain)

    def linear_glu(self, x, w_gate_up, act, limit=0.0, alpha=1.0):
        """act(x Wg^T, x Wu^T) with w_gate_up = [Wg; Wu] in the run dtype; the two products stay float until the
        activation has run."""
        if act == "silu":
            return self.linear_swiglu(x, w_gate_up)
        return self._hy.glu_act(self.linear_f32(x, w_gate_up, tag="gate_up"), self.dtype, act, limit, alpha)

    def experts_glu_up(self, x, w_gate_up, plan, act, limit=0.0, alpha=1.0, block=None):
        """act(g, u) for every sorted row of the plan, g and u the row's token times the gate and the up rows of the
        row's expert. W [E, 2F, K]: an expert's gate rows, then its up rows (`block` None), or blocks of `block` gate
        rows each followed by their up rows (16: the tcgen05 kernel then activates in its epilogue)."""
        F2 = w_gate_up.shape[1]
        if self._tc_experts(x, w_gate_up, plan):
            rows = self._mix.gather_rows_bf16(x, plan.rows_tok)
            if block == 16:
                out = torch.empty((plan.n_rows, F2 // 2), dtype=torch.bfloat16, device=x.device)
                return self._mix.grouped_gemm_tc(rows, w_gate_up, plan, out, self._mix.GEPI_SILU_GATED,
                                                 err=self._sm100.init(self.device).err, act=self._hy.GLU_ACTS[act],
                                                 limit=limit, alpha=alpha)
            gu = torch.empty((plan.n_rows, F2), dtype=torch.float32, device=x.device)
            self._mix.grouped_gemm_tc(rows, w_gate_up, plan, gu, self._mix.GEPI_STORE_F32,
                                      err=self._sm100.init(self.device).err)
        else:
            gu = torch.empty((plan.n_rows, F2), dtype=torch.float32, device=x.device)
            self._mix.grouped_gemm_ragged(x, w_gate_up, plan, gu, self._mix.GEPI_STORE_F32, gather=True)
        return self._hy.glu_act(gu, x.dtype, act, limit, alpha, block)

    def add_bias_f32(self, y, bias):
        return self._hy.add_bias_f32(y, bias)

    def gated_add(self, h, gate, bias, y):
        """h += sigmoid(gate + bias) * y, in float and in one pass; y a float tensor [T, H] or `ScaledSum` (one or two
        float tensors with a coefficient each)."""
        terms = list(y.terms) if hasattr(y, "terms") else [(y, 1.0)]
        return self._hy.gated_add(h, gate, bias, terms)

    def mingru_scan(self, proj, z_off, x_off, g_off, width, bias_z, bias_x, ctx, state):
        return self._hy.mingru_scan(proj, z_off, x_off, g_off, width, bias_z, bias_x, ctx.cu_q, ctx.num_seqs,
                                    ctx.state_slots, state, self.dtype, ctx.max_q_len)

    def short_conv(self, x, col0, channels, w, bias, ctx, tail, silu=True):
        return self._hy.short_conv(x, col0, channels, w, bias, ctx.token_seq, ctx.positions, ctx.cu_q, ctx.num_seqs,
                                   ctx.state_slots, tail, silu)

    def unit_heads(self, *a, **k):
        return self._hy.unit_heads(*a, **k)

    def softplus_decay(self, *a, **k):
        return self._hy.softplus_decay(*a, **k)

    def state_scan(self, q, q_heads, k, k_heads, v, decay, heads, dim, vdim, ctx, state, beta=None, vscale=None, skip=None):
        return self._hy.state_scan(q, q_heads, k, k_heads, v, decay, heads, dim, vdim, ctx.cu_q, ctx.num_seqs,
                                   ctx.state_slots, state, beta, vscale, skip)

    def gated_norm(self, y, gate, gate_col0, weight, eps, groups, gate_first, act):
        return self._hy.gated_norm(y, gate, gate_col0, weight, eps, groups, self.dtype, gate_first, act)

    def value_norm_store(self, proj, k_off, v_off, nkv, kd, vd, eps, norm, cache):
        if cache.writes:
            self._hy.value_norm_store(proj, k_off, v_off, nkv, kd, vd, eps, norm, cache.slots, cache.k, cache.v)

    def talk_attention(self, q, cache, ctx, nh, scale, mix, window, chunk, sinks):
        """Attention whose heads' softmax weights are mixed by `mix` before they meet the values: bfloat16 on the
        tensor cores where the kernel takes the sizes, else (and in the 32-bit run) in float on the CUDA cores."""
        hy = self._hy
        kd, vd = cache.k.shape[3], cache.v.shape[3]
        if self.fast and os.environ.get("RLLM_B200_NO_TC_ATTENTION") != "1" \
                and hy.talk_mma_supported(q.dtype, nh, kd, vd, cache.page_size):
            return hy.talk_attention_mma(q, cache.k, cache.v, ctx.token_seq, ctx.positions, cache.block_table, ctx.cu_q,
                                         ctx.num_seqs, ctx.max_q_len, nh, scale, mix, window, chunk, sinks)
        return hy.talk_attention_simt(q, cache.k, cache.v, ctx.token_seq, ctx.positions, cache.block_table, nh, scale,
                                            mix, window, chunk, sinks)

    # ---- selection
    def argmax(self, logits):
        return ops.argmax(logits)

    def add_at(self, logits, rows, cols, vals):
        return ops.add_at(logits, rows, cols, vals)

    def logprobs(self, logits, temperature, top_k, chosen, rows, n_top):
        return ops.logprobs(logits, temperature, top_k, chosen, rows, n_top)

    def sample(self, logits, temperature, uniform, top_k=None, top_p=None, min_p=None, out=None):
        return ops.sample(logits, temperature, uniform, top_k, top_p, min_p, out=out)
