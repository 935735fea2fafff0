"""Times one kernel at a time at given sizes: the tool the launch choices (token tile, ranges of K,
ranges of keys) were tuned with, and the small case a profiler is pointed at.

    python -m rllm_b200.kernels.microbench gemm --shape gateup --tokens 1,8,64
    python -m rllm_b200.kernels.microbench gemm --n 3072 --k 2048 --epilogue store --tokens 2048
    python -m rllm_b200.kernels.microbench attn-decode --batch 64 --context 3000 --splits 1,2,3
    python -m rllm_b200.kernels.microbench attn-prefill --tokens 2048 --kernel tc
    python -m rllm_b200.kernels.microbench sample --rows 8 --top-p 0.9
    python -m rllm_b200.kernels.microbench experts --tokens 8,2048 --width 2048 --ff 2048 --experts 16 --top 6
    python -m rllm_b200.kernels.microbench latent-attn --heads 16 --rank 512 --rot 64 --tokens 2048
    python -m rllm_b200.kernels.microbench latent-attn --heads 16 --rank 512 --rot 64 --batch 8 --context 1024
    python -m rllm_b200.kernels.microbench gla --heads 16 --dim 128 --vdim 128 --tokens 2048 [--batch 8]
    python -m rllm_b200.kernels.microbench sink --heads 32 --kv-heads 8 --dim 64 --vdim 48 --tokens 2048 --batch 8,64 --context 1024
    ... --plain 3      # no timing: three plain launches and a synchronize (for ncu -k ... -c ...)

Timing: the kernel runs back to back over `--copies` distinct weight (or cache) tensors, larger
together than the 126 MB L2, captured in a CUDA graph and replayed; CUDA events bracket five
replays. Back-to-back launches of one kernel overlap through programmatic dependent launch as
they do inside a decode step. Sizes default to the Llama 3.2 1B shapes.
"""
from __future__ import annotations

import argparse
import sys

import torch

from . import ops, sm100

DEV = "cuda:0"
SHAPES = {   # name -> (output features, inner size, epilogue)
    "qkv": (3072, 2048, "store"), "o": (2048, 2048, "accum"), "gateup": (8192, 2048, "swiglu"),
    "down": (2048, 8192, "accum"), "head": (128256, 2048, "store_f32"),
    "qkv-rope": (3072, 2048, "rope"),     # 32 + 2 x 8 heads of 64, rotated and written to a paged cache in the epilogue
}
EPI = {"store": ops.EPI_STORE, "store_f32": ops.EPI_STORE_F32, "accum": ops.EPI_ACCUM_F32,
       "swiglu": ops.EPI_SWIGLU}


def timed(fns, reps: int = 5) -> float:
    """Microseconds per call of the callables in `fns`, replayed as one CUDA graph."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(fns))


def run(fns, plain: int, label: str, nbytes: float = 0.0, flops: float = 0.0) -> None:
    if plain:
        for _ in range(plain):
            fns[0]()
        torch.cuda.synchronize()
        print(f"{label}: {plain} plain launches done")
        return
    us = timed(fns)
    extra = ""
    if nbytes:
        extra += f"  {nbytes / us / 1e3:7.0f} GB/s"
    if flops:
        extra += f"  {flops / us / 1e6:7.1f} TFLOP/s"
    print(f"{label}: {us:8.2f} us{extra}", flush=True)


def cmd_gemm(a) -> None:
    if a.shape:
        N, K, epi_name = SHAPES[a.shape]
    else:
        N, K, epi_name = a.n, a.k, a.epilogue
    sm100.set_pairs(a.pairs)
    sm100.set_token_rows(not a.weight_rows)
    if epi_name == "rope":
        return cmd_gemm_rope(a, N, K)
    epi = EPI[epi_name]
    rows = 2 * N if epi == ops.EPI_SWIGLU else N
    copies = max(1, min(a.copies, int(2e9 // (rows * K * 2)) or 1))
    ws = [torch.randn(rows, K, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    split = a.ranges if a.ranges > 1 else not a.no_split      # a number: that many ranges of K (tcgen05 small tiles)
    for T in a.tokens:
        out = torch.zeros(T, N, device=DEV, dtype=torch.float32) if epi == ops.EPI_ACCUM_F32 else None
        if a.norm:
            h = torch.randn(T, K, device=DEV)
            g = torch.ones(K, device=DEV)
            fns = [(lambda w=w: sm100.gemm_norm(h, g, 1e-5, w, epi, split=split)) for w in ws]
        else:
            x = torch.randn(T, K, device=DEV, dtype=torch.bfloat16)
            fns = [(lambda w=w: sm100.gemm(x, w, epi, out=out, split=split)) for w in ws]
        bn, sp = sm100.plan(epi, T, N, K, split=split)
        run(fns, a.plain, f"gemm {epi_name} T={T} N={N} K={K} tile={bn} ranges={sp}" + (" norm" if a.norm else ""),
            nbytes=rows * K * 2, flops=2.0 * T * rows * K)
    sm100.check_error(DEV)


def cmd_gemm_rope(a, N: int, K: int) -> None:
    """The q/k/v product with rotation and cache write in its epilogue (heads of 64, a quarter of them k and v each)."""
    hd, page = 64, 16
    nkv = N // hd // 6
    nh = N // hd - 2 * nkv
    copies = max(1, min(a.copies, int(2e9 // (N * K * 2)) or 1))
    ws = [torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, hd, 2, device=DEV, dtype=torch.float32) / hd))).contiguous()
    for T in a.tokens:
        pages = (T + page - 1) // page
        kc = torch.zeros(pages, nkv, page, hd, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        pos = torch.arange(T, device=DEV, dtype=torch.int32)
        slots = torch.arange(T, device=DEV, dtype=torch.int32)
        table = ops.rope_table(pos, inv_freq, T)
        split = a.ranges if a.ranges > 1 else not a.no_split
        if a.norm:
            h = torch.randn(T, K, device=DEV)
            g = torch.ones(K, device=DEV)
            x, norm = None, (h, g, 1e-5)
        else:
            x, norm = torch.randn(T, K, device=DEV, dtype=torch.bfloat16), None
        fns = [(lambda w=w: sm100.gemm_qkv_rope(x, w, pos, inv_freq, slots, kc, vc, nh, nkv, hd, page, hd,
                                                split=split, table=table, norm=norm)) for w in ws]
        run(fns, a.plain, f"gemm qkv+rope T={T} N={N} K={K} heads {nh}/{nkv} of {hd}" + (" norm" if a.norm else "")
            + (f" ranges asked {a.ranges}" if a.ranges > 1 else ""), nbytes=N * K * 2, flops=2.0 * T * N * K)
    sm100.check_error(DEV)


def cmd_attn_decode(a) -> None:
    nh, nkv, hd, page = a.heads, a.kv_heads, a.head_dim, a.page
    pages_per = (a.context + page - 1) // page
    used = a.batch * pages_per
    npages = max(used, a.pool_pages)          # a pool larger than what the sequences hold spreads their pages
    per_copy = npages * nkv * page * hd * 2 * 2
    copies = max(1, min(a.copies, int(4e9 // per_copy) or 1))
    caches = [(torch.randn(npages, nkv, page, hd, device=DEV, dtype=torch.bfloat16),
               torch.randn(npages, nkv, page, hd, device=DEV, dtype=torch.bfloat16)) for _ in range(copies)]
    if a.page_order == "random":              # a sequence's pages anywhere in the pool
        order = torch.randperm(npages, device=DEV)[:used]
    elif a.page_order == "reversed":          # each sequence a run of neighbouring pages, falling
        order = torch.arange(used - 1, -1, -1, device=DEV)
    else:                                     # each sequence a run of neighbouring pages, rising
        order = torch.arange(used, device=DEV)
    bt = order.to(torch.int32).view(a.batch, pages_per).contiguous()
    lens = torch.full((a.batch,), a.context, dtype=torch.int32, device=DEV)
    q = torch.randn(a.batch, nh * hd, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    nbytes = a.batch * a.context * nkv * hd * 2 * 2
    auto = sm100.decode_splits(a.batch, nkv, a.context, sm100.init(DEV).sm_count)
    for sp in (a.splits or [auto]):
        fns = [(lambda kc=kc, vc=vc: sm100.attention_decode(q, kc, vc, lens, bt, nh, hd ** -0.5, None, a.context,
                                                            splits=sp, out=out)) for kc, vc in caches]
        run(fns, a.plain, f"attn-decode B={a.batch} ctx={a.context} hd={hd} page={page} pages {a.page_order} of {npages} "
            f"ranges={sp} (auto {auto})",
            nbytes=nbytes)


def cmd_attn_prefill(a) -> None:
    nh, nkv, hd, page = a.heads, a.kv_heads, a.head_dim, a.page
    T = a.tokens[0]
    pages_per = (T + page - 1) // page
    kc = torch.randn(pages_per, nkv, page, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.randn(pages_per, nkv, page, hd, device=DEV, dtype=torch.bfloat16)
    bt = torch.arange(pages_per, device=DEV, dtype=torch.int32).view(1, pages_per)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    cu, lens = i32([0, T]), i32([T])
    q = torch.randn(T, nh * hd, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    if a.kernel == "tc":
        f = lambda: sm100.attention_prefill_tc(q, kc, vc, cu, lens, bt, T, nh, hd ** -0.5, None, out=out)
    else:
        f = lambda: sm100.attention_fa(q, kc, vc, cu, lens, bt, T, T, T, nh, hd ** -0.5, None, splits=1, out=out)
    run([f] * 4, a.plain, f"attn-prefill ({a.kernel}) T={T} heads={nh}/{nkv} hd={hd}",
        flops=4.0 * nh * hd * T * (T + 1) / 2)
    sm100.check_error(DEV)


def cmd_sample(a) -> None:
    R, V = a.rows, a.vocab
    logits = torch.randn(R, V, device=DEV) * 3
    vec = lambda v, dt=torch.float32: torch.full((R,), v, dtype=dt, device=DEV)
    u = torch.rand(R, device=DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    if a.temperature <= 0:
        f = lambda: ops.argmax(logits, out=out)
        what = "argmax"
    else:
        kw = dict(top_k=vec(a.top_k, torch.int32) if a.top_k > 0 else None, top_p=vec(a.top_p) if a.top_p < 1 else None,
                  min_p=vec(a.min_p) if a.min_p > 0 else None)
        temp = vec(a.temperature)
        f = lambda: ops.sample(logits, temp, u, out=out, **kw)
        what = f"temperature {a.temperature} top-k {a.top_k} top-p {a.top_p} min-p {a.min_p}"
    run([f] * 4, a.plain, f"sample rows={R} vocab={V} {what}", nbytes=R * V * 4)


def cmd_experts(a) -> None:
    """The two grouped products of a routed feed-forward (bfloat16) over a plan from random router logits."""
    from . import mix
    W, F, E, top = a.width, a.ff, a.experts, a.top
    ups = [torch.randn(E, F, W, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(a.copies)]
    downs = [torch.randn(E, W, F, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(a.copies)]
    for T in a.tokens:
        x = torch.randn(T, W, device=DEV, dtype=torch.bfloat16)
        logits = torch.randn(T, E, device=DEV)
        per_tile = mix.tile_rows(torch.bfloat16, W, W, T * top) if W % 8 == 0 and F % 8 == 0 else 64
        idx, wt = mix.moe_topk(logits, top, a.groups, a.keep)
        plan = mix.moe_plan(idx, wt, E, per_tile)
        act = torch.empty(T * top, F, device=DEV, dtype=torch.bfloat16)
        out = torch.empty(T * top, W, device=DEV, dtype=torch.float32)
        used = int(torch.unique(idx).numel())
        run([lambda: (mix.moe_topk(logits, top, a.groups, a.keep), mix.moe_plan(idx, wt, E, per_tile))], a.plain,
            f"route+plan T={T}")
        tc = per_tile == 128 and not a.mma and mix.tc_supported(W, F, W) and mix.tc_supported(F, W, F)
        if tc:
            err = sm100.init(DEV).err
            run([lambda: mix.gather_rows_bf16(x, plan.rows_tok)], a.plain, f"gather rows T={T}", 2 * T * top * W * 2)
            rows = mix.gather_rows_bf16(x, plan.rows_tok)
            up_fn = lambda u: mix.grouped_gemm_tc(rows, u, plan, act, mix.GEPI_RELU2, err=err)
            down_fn = lambda d: mix.grouped_gemm_tc(act, d, plan, out, mix.GEPI_STORE_F32, scatter=True, scale=True, err=err)
        else:
            up_fn = lambda u: mix.grouped_gemm_ragged(x, u, plan, act, mix.GEPI_RELU2, gather=True)
            down_fn = lambda d: mix.grouped_gemm_ragged(act, d, plan, out, mix.GEPI_STORE_F32, scatter=True, scale=True)
        kind = "tcgen05" if tc else "mma.sync"
        run([lambda u=u: up_fn(u) for u in ups], a.plain,
            f"experts_up T={T} ({used} experts used, {kind})", used * F * W * 2 + T * top * (F + W) * 2, 2.0 * T * top * F * W)
        run([lambda d=d: down_fn(d) for d in downs], a.plain, f"experts_down T={T} ({kind})",
            used * F * W * 2 + T * top * (2 * F + 4 * W), 2.0 * T * top * F * W)
        if tc:
            sm100.check_error(DEV)


def _paged(batch: int, context: int, new: int, page: int):
    """Block tables, positions and row ranges of `batch` sequences that hold `context` keys, the last `new` of
    them this step's tokens; pages handed out in a random order."""
    per = (context + page - 1) // page
    perm = torch.randperm(batch * per, dtype=torch.int32).view(batch, per)
    pos = torch.arange(context - new, context, dtype=torch.int32).repeat(batch)
    seq = torch.arange(batch, dtype=torch.int32).repeat_interleave(new)
    cu = torch.arange(batch + 1, dtype=torch.int32) * new
    return perm.to(DEV), pos.to(DEV), seq.to(DEV), cu.to(DEV), batch * per


def cmd_latent_attn(a) -> None:
    from . import mix
    H, rank, dk, page = a.heads, a.rank, a.rank + a.rot, a.page
    cases = [(1, T, T) for T in a.tokens] if a.batch == 0 else [(a.batch, a.context, 1)]
    for batch, context, new in cases:
        bt, pos, seq, cu, pages = _paged(batch, context, new, page)
        caches = [torch.randn(pages, page, dk, device=DEV, dtype=torch.bfloat16) for _ in range(a.copies)]
        q = torch.randn(batch * new, H, dk, device=DEV, dtype=torch.bfloat16)
        few = new <= 2 and rank % 128 == 0 and not a.wide
        rows = 16 if few else 64
        tiles = max(1, batch * new * H // rows)
        keys = min(a.window, context) if a.window else context
        splits = a.splits or max(1, min(16, torch.cuda.get_device_properties(0).multi_processor_count // tiles, keys // 128))
        seen = sum(min(p + 1, a.window or p + 1) for p in range(context - new, context)) * batch
        run([lambda c=c: mix.latent_attention(q, c, seq, pos, bt, rank, dk ** -0.5, a.window or None, cu_q=cu,
                                              num_seqs=batch, tensor_cores=not a.simt, splits=splits, few=few) for c in caches],
            a.plain, f"latent attention {batch} x {new} tokens, context {context}, {H} heads, splits {splits}, rows a CTA {rows}",
            batch * min(context, keys + new) * dk * 2 + 2 * q.numel() * 2, 2.0 * H * (dk + rank) * seen)


def cmd_gla(a) -> None:
    from . import mix
    H, d, v = a.heads, a.dim, a.vdim
    cases = [(1, T) for T in a.tokens] if a.batch == 0 else [(a.batch, 1)]
    for batch, new in cases:
        T = batch * new
        cols = 2 * H * d + H * v
        proj = torch.randn(T, cols, device=DEV, dtype=torch.bfloat16) * 0.3
        alpha = torch.rand(T, H * d, device=DEV) * 0.1 + 0.9
        cu = (torch.arange(batch + 1, dtype=torch.int32) * new).to(DEV)
        slots = torch.arange(batch, dtype=torch.int32).to(DEV)
        states = [torch.zeros(batch, H, d, v, device=DEV) for _ in range(a.copies if new == 1 else 1)]
        chunk = a.chunk if new >= 3 * a.chunk else 0
        run([lambda s=s: mix.gla_scan(proj, 0, H * d, 2 * H * d, alpha, d ** -0.5, H, d, v, cu, batch, slots, s, chunk)
             for s in states], a.plain, f"gla scan {batch} x {new} tokens, {H} heads of {d} x {v}, chunk {chunk}",
            T * (cols * 2 + H * d * 4 + H * v * 4) + 2 * batch * H * d * v * 4, (5.0 if chunk == 0 else 8.0) * T * H * d * v)


def cmd_sink(a) -> None:
    """The kernels of attention with sink, gate and block mask and of layers that norm after the sum, each beside
    the like kernel of plain grouped-query attention at the same sizes."""
    from . import sink
    nh, nkv, kd, vd, page, W = a.heads, a.kv_heads, a.dim, a.vdim, a.page, a.width
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    bf = lambda *shape: torch.randn(*shape, device=DEV, dtype=torch.bfloat16)
    sinks, scale = torch.randn(nh, device=DEV), kd ** -0.5
    for T in a.tokens:                                   # one prompt of T tokens
        pages = (T + page - 1) // page
        kc, vc, ve = bf(pages, nkv, page, kd), bf(pages, nkv, page, vd), bf(pages, nkv, page, kd)
        bt, cu, lens = torch.arange(pages, device=DEV, dtype=torch.int32).view(1, pages), i32([0, T]), i32([T])
        q, gate = bf(T, nh * kd), torch.randn(T, nh, device=DEV)
        pos, seq = torch.arange(T, device=DEV, dtype=torch.int32), torch.zeros(T, device=DEV, dtype=torch.int32)
        pairs = T * (T + 1) / 2
        run([lambda: sink.sink_attention_mma(q, kc, vc, seq, pos, bt, cu, 1, T, nh, scale, None, a.chunk or None, sinks, gate)] * 4,
            a.plain, f"sink attention (mma.sync) T={T} heads={nh}/{nkv} of {kd}/{vd}", flops=2.0 * nh * (kd + vd) * pairs)
        if a.plain:
            return
        if kd in (64, 128):
            out = torch.empty_like(q)
            run([lambda: sm100.attention_fa(q, kc, ve, cu, lens, bt, T, T, T, nh, scale, None, splits=1, out=out)] * 4, 0,
                f"  like: plain attention (mma.sync) T={T} heads of {kd}", flops=4.0 * nh * kd * pairs)
            run([lambda: sm100.attention_prefill_tc(q, kc, ve, cu, lens, bt, T, nh, scale, None, out=out, chunk=a.chunk or None,
                                                    sinks=sinks, gate=gate)] * 4, 0,
                f"  equal head sizes: tcgen05 kernel with mask, sink and gate T={T}", flops=4.0 * nh * kd * pairs)
        # query/key norm + rotation + cache write beside the plain rotation + cache write; sum-and-norm beside the plain norm
        rot = kd // 2
        proj = bf(T, (nh + nkv) * kd + nkv * vd)
        wn, table = torch.ones(kd, device=DEV), torch.randn(T, rot // 2, 2, device=DEV)
        slots = torch.arange(T, device=DEV, dtype=torch.int32)
        run([lambda: sink.qk_norm_rope_store(proj, 0, nh * kd, (nh + nkv) * kd, nh, nkv, kd, vd, rot, wn, wn, 1e-6, table, slots,
                                             kc, vc)] * 4, 0, f"query/key norm + rotation + cache write T={T}",
            nbytes=proj.numel() * 2 + T * (nh * kd + nkv * (kd + vd)) * 2)
        if kd in (64, 128):
            qkv, inv = bf(T, (nh + 2 * nkv) * kd), torch.rand(kd // 2, device=DEV)
            tb = ops.rope_table(pos, inv, T)
            run([lambda: ops.rope_cache_write(qkv, pos, inv, slots, kc, ve, nh, nkv, kd, page, table=tb)] * 4, 0,
                f"  like: rotation + cache write T={T}", nbytes=qkv.numel() * 2 + T * (nh + 2 * nkv) * kd * 2)
        h, y, w = torch.randn(T, W, device=DEV), torch.randn(T, W, device=DEV), torch.ones(W, device=DEV)
        copy = torch.empty(T, W, device=DEV, dtype=torch.bfloat16)
        run([lambda: sink.postnorm(h, y, 2.0, w, 1e-6, copy=copy)] * 4, 0, f"sum + norm (float stream, bfloat16 copy) T={T} width={W}",
            nbytes=T * W * 14)
        run([lambda: ops.rmsnorm(h, w, 1e-6, torch.bfloat16, out=copy)] * 4, 0, f"  like: norm T={T}", nbytes=T * W * 6)
    for B in a.batch:                                    # B single tokens at context C
        C = a.context
        pages = (C + page - 1) // page
        copies = max(1, min(8, int(2e9 // (B * pages * nkv * page * (kd + vd) * 2))))
        caches = [(bf(B * pages, nkv, page, kd), bf(B * pages, nkv, page, vd), bf(B * pages, nkv, page, kd)) for _ in range(copies)]
        bt = torch.randperm(B * pages, device=DEV).to(torch.int32).view(B, pages).contiguous()
        lens, pos, seq, cu = i32([C] * B), i32([C - 1] * B), torch.arange(B, device=DEV, dtype=torch.int32), torch.arange(B + 1, device=DEV, dtype=torch.int32)
        q, gate = bf(B, nh * kd), torch.randn(B, nh, device=DEV)
        tiles = B * nkv * ((nh // nkv + 63) // 64)
        sp = max(1, min(16, 4 * sm100.init(DEV).sm_count // tiles, C // 128))
        run([(lambda c=c: sink.sink_attention_mma(q, c[0], c[1], seq, pos, bt, cu, B, 1, nh, scale, None, a.chunk or None, sinks, gate,
                                                  sp, C)) for c in caches], 0,
            f"sink attention (mma.sync) {B} x 1 token, {C} keys, heads of {kd}/{vd}, ranges={sp}", nbytes=B * C * nkv * (kd + vd) * 2)
        if kd in (64, 128):
            out = torch.empty_like(q)
            run([(lambda c=c: sm100.attention_decode(q, c[0], c[2], lens, bt, nh, scale, None, C, out=out)) for c in caches], 0,
                f"  like: plain decode attention {B} x 1 token, {C} keys, heads of {kd}", nbytes=B * C * nkv * kd * 4)
    sm100.check_error(DEV)


def cmd_talk(a) -> None:
    """Attention with mixed heads: one prompt of T tokens, then B single tokens at context C."""
    from . import hybrid
    nh, nkv, kd, vd, page = a.heads, a.kv_heads, a.dim, a.vdim, a.page
    bf = lambda *shape: torch.randn(*shape, device=DEV, dtype=torch.bfloat16)
    mixm, sinks, scale = torch.randn(nh, nh, device=DEV) * 0.2 + torch.eye(nh, device=DEV), torch.zeros(nh, device=DEV), kd ** -0.5
    for T in a.tokens:
        bt, pos, seq, cu, pages = _paged(1, T, T, page)
        kc, vc, q = bf(pages, nkv, page, kd), bf(pages, nkv, page, vd), bf(T, nh * kd)
        pairs = sum(min(p + 1, a.window or p + 1) for p in range(T))
        if a.simt:
            fn = lambda: hybrid.talk_attention_simt(q, kc, vc, seq, pos, bt, nh, scale, mixm, a.window or None, None, sinks)
        else:
            fn = lambda: hybrid.talk_attention_mma(q, kc, vc, seq, pos, bt, cu, 1, T, nh, scale, mixm, a.window or None, None, sinks)
        run([fn] * 2, a.plain, f"mixed-heads attention ({'CUDA cores' if a.simt else 'mma.sync'}) T={T} heads={nh}/{nkv} of {kd}/{vd}",
            flops=2.0 * nh * (kd + vd) * pairs)
        if a.plain:
            return
    for B in a.batch:
        C = a.context
        bt, pos, seq, cu, pages = _paged(B, C, 1, page)
        copies = max(1, min(8, int(2e9 // (pages * nkv * page * (kd + vd) * 2))))
        caches = [(bf(pages, nkv, page, kd), bf(pages, nkv, page, vd)) for _ in range(copies)]
        q = bf(B, nh * kd)
        keys = min(C, a.window or C)
        run([(lambda c=c: hybrid.talk_attention_mma(q, c[0], c[1], seq, pos, bt, cu, B, 1, nh, scale, mixm, a.window or None, None,
                                                    sinks)) for c in caches], 0,
            f"mixed-heads attention (mma.sync) {B} x 1 token, {C} keys, heads={nh}/{nkv} of {kd}/{vd}",
            nbytes=B * keys * nkv * (kd + vd) * 2)


def cmd_scan(a) -> None:
    """The recurrence over a per-request state, plain or delta rule: one prompt of T tokens, then B single tokens."""
    from . import hybrid
    H, d, v = a.heads, a.dim, a.vdim
    cases = [(1, T) for T in a.tokens] + [(B, 1) for B in a.batch]
    for batch, new in cases:
        T = batch * new
        q, k = torch.randn(T, H * d, device=DEV) * d ** -0.5, torch.nn.functional.normalize(torch.randn(T, H, d, device=DEV), dim=-1).view(T, H * d)
        x = torch.randn(T, H * v, device=DEV)
        decay = torch.rand(T, H * d if a.delta else H, device=DEV) * 0.1 + 0.9
        beta = torch.randn(T, H, device=DEV, dtype=torch.bfloat16) if a.delta else None
        cu = (torch.arange(batch + 1, dtype=torch.int32) * new).to(DEV)
        slots = torch.arange(batch, dtype=torch.int32).to(DEV)
        states = [torch.zeros(batch, H, d, v, device=DEV) for _ in range(a.copies if new == 1 else 1)]
        run([lambda s=s: hybrid.state_scan(q, H, k, H, x, decay, H, d, v, cu, batch, slots, s, beta, channels=a.channels) for s in states], a.plain,
            f"state scan ({'delta rule' if a.delta else 'plain'}) {batch} x {new} tokens, {H} heads of {d} x {v}",
            T * H * (2 * d + 2 * v) * 4 + decay.numel() * 4 + 2 * batch * H * d * v * 4, (7.0 if a.delta else 5.0) * T * H * d * v)
        if a.plain:
            return


def cmd_gated(a) -> None:
    """The kernels of layers whose sublayers are gated into the stream, each beside its like kernel at the same sizes:
    attention with sigmoid weights and with kept first keys beside the softmax and the window alone (one kernel, other
    branches), the gated recurrence beside the state scan, the gated sum beside the sum of a layer's terms, the gelu in
    a product's epilogue beside relu squared there."""
    from . import hybrid, sink
    nh, nkv, kd, vd, page, W = a.heads, a.kv_heads, a.dim, a.vdim, a.page, a.width
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    bf = lambda *shape: torch.randn(*shape, device=DEV, dtype=torch.bfloat16)
    bias, scale = torch.randn(nh, device=DEV) - 2, kd ** -0.5
    for T in a.tokens:                                   # one prompt of T tokens
        pages = (T + page - 1) // page
        kc, vc = bf(pages, nkv, page, kd), bf(pages, nkv, page, vd)
        bt, cu = torch.arange(pages, device=DEV, dtype=torch.int32).view(1, pages), i32([0, T])
        q = bf(T, nh * kd)
        pos, seq = torch.arange(T, device=DEV, dtype=torch.int32), torch.zeros(T, device=DEV, dtype=torch.int32)
        pairs = T * (T + 1) / 2
        if a.plain and a.tcgen05:
            lens, out = i32([T]), torch.empty(T, nh * vd, device=DEV, dtype=torch.bfloat16)
            run([lambda: sm100.attention_prefill_tc(q, kc, vc, cu, lens, bt, T, nh, scale, None, out=out, sinks=bias, sigmoid=True)],
                a.plain, f"sigmoid attention (tcgen05) T={T} heads of {kd}")
            sm100.check_error(DEV)
            return
        run([lambda: sink.sink_attention_mma(q, kc, vc, seq, pos, bt, cu, 1, T, nh, scale, None, None, bias, None, 1, T, 0, True)] * 4,
            a.plain, f"sigmoid attention (mma.sync) T={T} heads={nh}/{nkv} of {kd}/{vd}", flops=2.0 * nh * (kd + vd) * pairs)
        if a.plain:
            return
        run([lambda: sink.sink_attention_mma(q, kc, vc, seq, pos, bt, cu, 1, T, nh, scale, None, None, None, None, 1, T)] * 4, 0,
            f"  like: softmax attention, the same kernel T={T}", flops=2.0 * nh * (kd + vd) * pairs)
        win, kept = a.window, a.keep_first
        wpairs = sum(min(i + 1, win) + min(kept, max(0, i + 1 - win)) for i in range(T))
        run([lambda: sink.sink_attention_mma(q, kc, vc, seq, pos, bt, cu, 1, T, nh, scale, win, None, None, None, 1, T, kept)] * 4, 0,
            f"windowed attention with kept first keys T={T} window={win} kept={kept}", flops=2.0 * nh * (kd + vd) * wpairs)
        run([lambda: sink.sink_attention_mma(q, kc, vc, seq, pos, bt, cu, 1, T, nh, scale, win, None, None, None, 1, T)] * 4, 0,
            f"  like: the window alone T={T}", flops=2.0 * nh * (kd + vd) * sum(min(i + 1, win) for i in range(T)))
        if kd == vd and kd in (64, 128):                 # equal head sizes: long portions take the tcgen05 kernel
            lens, out = i32([T]), torch.empty(T, nh * vd, device=DEV, dtype=torch.bfloat16)
            run([lambda: sm100.attention_prefill_tc(q, kc, vc, cu, lens, bt, T, nh, scale, None, out=out, sinks=bias, sigmoid=True)] * 4, 0,
                f"sigmoid attention (tcgen05) T={T} heads of {kd}", flops=4.0 * nh * kd * pairs)
            run([lambda: sm100.attention_prefill_tc(q, kc, vc, cu, lens, bt, T, nh, scale, None, out=out)] * 4, 0,
                f"  like: softmax attention (tcgen05) T={T}", flops=4.0 * nh * kd * pairs)
            run([lambda: sm100.attention_prefill_tc(q, kc, vc, cu, lens, bt, T, nh, scale, win, out=out, keep_first=kept)] * 4, 0,
                f"windowed attention with kept first keys (tcgen05) T={T} window={win} kept={kept}", flops=4.0 * nh * kd * wpairs)
            run([lambda: sm100.attention_prefill_tc(q, kc, vc, cu, lens, bt, T, nh, scale, win, out=out)] * 4, 0,
                f"  like: the window alone (tcgen05) T={T}", flops=4.0 * nh * kd * sum(min(i + 1, win) for i in range(T)))
        # the gated recurrence beside the state scan over as many channels (heads of 128 x 64 hold 64 times the state)
        R = a.channels or W
        proj, bz, bx = torch.randn(T, 3 * R, device=DEV), torch.randn(R, device=DEV), torch.randn(R, device=DEV)
        st, slots = torch.zeros(1, R, device=DEV), i32([0])
        run([lambda: hybrid.mingru_scan(proj, 0, R, 2 * R, R, bz, bx, cu, 1, slots, st, torch.bfloat16, T)] * 4, 0,
            f"gated recurrence T={T} channels={R}", nbytes=T * R * (5 * 4 + 2))
        H, d, v = max(1, R // 64), 128, 64
        sq, sk = torch.randn(T, H * d, device=DEV) * d ** -0.5, torch.randn(T, H * d, device=DEV) * d ** -0.5
        sx, decay, S = torch.randn(T, H * v, device=DEV), torch.rand(T, H, device=DEV) * 0.1 + 0.9, torch.zeros(1, H, d, v, device=DEV)
        run([lambda: hybrid.state_scan(sq, H, sk, H, sx, decay, H, d, v, cu, 1, slots, S)] * 4, 0,
            f"  like: state scan T={T}, {H} heads of {d} x {v}", nbytes=T * H * (2 * d + 2 * v) * 4 + decay.numel() * 4)
        # the gated sum beside the sum of a layer's terms
        h, g, b, y0, y1 = (torch.randn(T, W, device=DEV) for _ in range(5))
        run([lambda: hybrid.gated_add(h, g, b[0].contiguous(), [(y0, 0.5), (y1, 0.5)])] * 4, 0,
            f"gated sum into the stream, two summands T={T} width={W}", nbytes=T * W * 4 * 5)
        wl = torch.ones(W, device=DEV)
        run([lambda: hybrid.combine(h, [(y0, wl), (y1, wl)], 0.5, 1e-6, [g])] * 4, 0, f"  like: sum of a layer's terms T={T}",
            nbytes=T * W * 4 * 5)
        # gelu in the epilogue of the up product beside relu squared there, and beside the float product with a pass after it
        x, wu = bf(T, W), bf(4 * W, W)
        for act in ("gelu_tanh", "relu2"):
            run([lambda act=act: sm100.gemm(x, wu, ops.EPI_STORE, act=act)] * 4, 0,
                f"{'  like: ' if act == 'relu2' else ''}up product with {act} in its epilogue T={T} {W} -> {4 * W}", flops=2.0 * T * W * 4 * W)
        run([lambda: hybrid.act_rows(sm100.gemm(x, wu, ops.EPI_STORE_F32), torch.bfloat16, "gelu_tanh")] * 4, 0,
            f"  the float product and a pass for the gelu T={T}", flops=2.0 * T * W * 4 * W)
    for B in a.batch:                                    # B single tokens at context C
        C = a.context
        pages = (C + page - 1) // page
        copies = max(1, min(8, int(2e9 // (B * pages * nkv * page * (kd + vd) * 2))))
        caches = [(bf(B * pages, nkv, page, kd), bf(B * pages, nkv, page, vd)) for _ in range(copies)]
        bt = torch.randperm(B * pages, device=DEV).to(torch.int32).view(B, pages).contiguous()
        pos, seq, cu = i32([C - 1] * B), torch.arange(B, device=DEV, dtype=torch.int32), torch.arange(B + 1, device=DEV, dtype=torch.int32)
        q = bf(B, nh * kd)
        tiles = B * nkv * ((nh // nkv + 63) // 64)
        sp = max(1, min(16, 4 * sm100.init(DEV).sm_count // tiles, C // 128))
        for sig in (True, False):
            run([(lambda c=c: sink.sink_attention_mma(q, c[0], c[1], seq, pos, bt, cu, B, 1, nh, scale, None, None, bias if sig else None,
                                                      None, sp, C, 0, sig)) for c in caches], 0,
                f"{'sigmoid attention' if sig else '  like: softmax attention'} {B} x 1 token, {C} keys, heads of {kd}/{vd}, ranges={sp}",
                nbytes=B * C * nkv * (kd + vd) * 2)
        R = a.channels or W
        proj, bz, bx = torch.randn(B, 3 * R, device=DEV), torch.randn(R, device=DEV), torch.randn(R, device=DEV)
        states = [torch.zeros(B, R, device=DEV) for _ in range(8)]
        run([lambda s=s: hybrid.mingru_scan(proj, 0, R, 2 * R, R, bz, bx, cu, B, seq, s, torch.bfloat16, 1) for s in states], 0,
            f"gated recurrence {B} x 1 token, channels={R}", nbytes=B * R * (3 * 4 + 2 + 8))
    sm100.check_error(DEV)


def main(argv=None) -> int:
    ints = lambda s: [int(x) for x in s.split(",")]
    ap = argparse.ArgumentParser(prog="python -m rllm_b200.kernels.microbench", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("sample")
    p.add_argument("--plain", type=int, default=0, help="N plain launches instead of timing")
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--vocab", type=int, default=128256)
    p.add_argument("--temperature", type=float, default=0.8, help="0: the argmax kernel")
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--min-p", type=float, default=0.0)
    p = sub.add_parser("experts")
    p.add_argument("--plain", type=int, default=0)
    p.add_argument("--copies", type=int, default=4)
    p.add_argument("--tokens", type=ints, default=[8, 2048])
    for k, v in (("width", 2048), ("ff", 2048), ("experts", 16), ("top", 6), ("groups", 1), ("keep", 1)):
        p.add_argument("--" + k, type=int, default=v)
    p.add_argument("--mma", action="store_true", help="long row lists on the mma.sync kernel instead of tcgen05")
    p = sub.add_parser("latent-attn")
    p.add_argument("--plain", type=int, default=0)
    p.add_argument("--copies", type=int, default=4)
    p.add_argument("--tokens", type=ints, default=[2048])
    for k, v in (("heads", 16), ("rank", 512), ("rot", 64), ("page", 16), ("batch", 0), ("context", 1024), ("window", 0),
                 ("splits", 0)):
        p.add_argument("--" + k, type=int, default=v)
    p.add_argument("--simt", action="store_true", help="the CUDA-core kernel")
    p.add_argument("--wide", action="store_true", help="64 rows a CTA also for single tokens")
    p = sub.add_parser("gla")
    p.add_argument("--plain", type=int, default=0)
    p.add_argument("--copies", type=int, default=8)
    p.add_argument("--tokens", type=ints, default=[2048])
    for k, v in (("heads", 16), ("dim", 128), ("vdim", 128), ("batch", 0), ("chunk", 128)):
        p.add_argument("--" + k, type=int, default=v)
    p = sub.add_parser("sink")
    p.add_argument("--plain", type=int, default=0, help="N plain launches of the prompt attention kernel instead of timing")
    p.add_argument("--tokens", type=ints, default=[2048])
    p.add_argument("--batch", type=ints, default=[8, 64])
    for k, v in (("heads", 32), ("kv-heads", 8), ("dim", 64), ("vdim", 32), ("page", 16), ("context", 1024), ("chunk", 0),
                 ("width", 2048)):
        p.add_argument("--" + k, type=int, default=v)
    p = sub.add_parser("gated")
    p.add_argument("--plain", type=int, default=0, help="N plain launches of the sigmoid attention kernel instead of timing")
    p.add_argument("--tcgen05", action="store_true", help="with --plain: the tcgen05 kernel (equal head sizes of 64 or 128)")
    p.add_argument("--tokens", type=ints, default=[2048])
    p.add_argument("--batch", type=ints, default=[8, 64])
    for k, v in (("heads", 16), ("kv-heads", 4), ("dim", 128), ("vdim", 128), ("page", 16), ("context", 1024), ("window", 1024),
                 ("keep-first", 64), ("width", 2048), ("channels", 0)):
        p.add_argument("--" + k, type=int, default=v)
    p = sub.add_parser("talk")
    p.add_argument("--plain", type=int, default=0, help="N plain launches of the prompt kernel instead of timing")
    p.add_argument("--tokens", type=ints, default=[2048])
    p.add_argument("--batch", type=ints, default=[8, 64])
    p.add_argument("--simt", action="store_true", help="the CUDA-core kernel (prompts only)")
    for k, v in (("heads", 16), ("kv-heads", 4), ("dim", 128), ("vdim", 128), ("page", 16), ("context", 1024), ("window", 0)):
        p.add_argument("--" + k, type=int, default=v)
    p = sub.add_parser("scan")
    p.add_argument("--plain", type=int, default=0)
    p.add_argument("--copies", type=int, default=8)
    p.add_argument("--tokens", type=ints, default=[2048])
    p.add_argument("--batch", type=ints, default=[8, 64])
    p.add_argument("--delta", action="store_true", help="the delta rule with a decay per channel (default: plain, a decay per head)")
    for k, v in (("heads", 16), ("dim", 128), ("vdim", 128), ("channels", 0)):
        p.add_argument("--" + k, type=int, default=v)
    for name in ("gemm", "attn-decode", "attn-prefill"):
        p = sub.add_parser(name)
        p.add_argument("--plain", type=int, default=0, help="N plain launches instead of timing")
        p.add_argument("--copies", type=int, default=8, help="distinct weight / cache tensors to cycle through")
        if name == "gemm":
            p.add_argument("--shape", choices=sorted(SHAPES))
            p.add_argument("--n", type=int, default=2048)
            p.add_argument("--k", type=int, default=2048)
            p.add_argument("--epilogue", choices=sorted(EPI), default="store")
            p.add_argument("--tokens", type=ints, default=[1, 8, 64, 2048])
            p.add_argument("--norm", action="store_true", help="RMSNorm in front, in the same kernel")
            p.add_argument("--no-split", action="store_true")
            p.add_argument("--weight-rows", action="store_true",
                           help="gate/up of long portions with the weight rows on the accumulator's rows (default: the tokens)")
            p.add_argument("--pairs", action="store_true", help="long portions on pairs of CTAs (tcgen05.mma.cta_group::2)")
            p.add_argument("--ranges", type=int, default=0, help="ranges of K to force on the tcgen05 small-tile kernel")
        else:
            p.add_argument("--heads", type=int, default=32)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=64)
            p.add_argument("--page", type=int, default=16)
            if name == "attn-decode":
                p.add_argument("--batch", type=int, default=8)
                p.add_argument("--context", type=int, default=3000)
                p.add_argument("--splits", type=ints, default=None)
                p.add_argument("--page-order", choices=["random", "rising", "reversed"], default="random")
                p.add_argument("--pool-pages", type=int, default=0, help="pages of the pool (at least what the sequences hold)")
            else:
                p.add_argument("--tokens", type=ints, default=[2048])
                p.add_argument("--kernel", choices=["tc", "fa"], default="tc",
                               help="tc: tcgen05 kernel (head sizes 64 and 128); fa: mma.sync kernel")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench: no CUDA device", file=sys.stderr)
        return 1
    {"gemm": cmd_gemm, "attn-decode": cmd_attn_decode, "attn-prefill": cmd_attn_prefill, "sample": cmd_sample,
     "experts": cmd_experts, "latent-attn": cmd_latent_attn, "gla": cmd_gla, "sink": cmd_sink, "talk": cmd_talk,
     "scan": cmd_scan, "gated": cmd_gated}[a.cmd](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
