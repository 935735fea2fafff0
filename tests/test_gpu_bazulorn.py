"""Bazulorn on the GPU against the plain implementation (tests/plain_bazulorn.py): each mechanism alone, then
whole models through the step function, the scheduler and the trace program; prompts whole, in portions down
to two tokens, decoded token by token, and in mixed batches with pages and slots used again. Where random inputs
would hide a fault the inputs are made so that it shows: the input at one position is scaled up so that its key
wins every score it takes part in (a window's edge that is one off, a far key that is lost, the first tokens),
scores are small enough for the sink to hold a visible share of every softmax, and decays are near one so that
the first token is still felt at the end."""
import itertools
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import bazulorn_tiny as B
import plain_bazulorn as P
import replay
from test_gpu_zukotar import SCHEDULES, Harness, bind, check, cut, rel, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


def as_stored(weights, dtype):
    return {k: (v.to(DT[dtype]) if v.is_floating_point() else v).to(F64) for k, v in weights.items()}


def stored_as(dtype):
    """What a run of this type does to the activations it keeps between two kernels."""
    return P.exact if dtype == "float32" else (lambda x: x.to(torch.bfloat16).to(F64))


def close(got, want, dtype):
    """Against the plain implementation with the run's own roundings of stored activations put in: in bfloat16 a
    projection's output is rounded to 8 bits of mantissa before it enters a recurrence, and a step size or a decay
    that such a rounding moves is felt by every later token of its head, so against exact arithmetic single rows
    lie several percent off by rounding alone. With the same roundings on both sides what is left is the order of
    sums and numbers that fall on the other side of a rounding's edge."""
    return rel(got, want) < (3e-5 if dtype == "float32" else 1.5e-2)


def strip(w, prefix="x."):
    return {k[len(prefix):]: v for k, v in w.items()}


class TwoLayers(Harness):
    """A harness whose part is made of two mixers: it gets a tuple of two cache layers."""

    def run(self, entries, fn):
        from rllm_b200.engine import Entry
        entries = [Entry(r, [0] * n, []) for r, n in entries]
        rcs = self.engine.prepare(entries)
        ctx, _ = self.engine.build_context(entries, rcs)
        out = fn(ctx, (self.cache.layer_view(0, ctx, True), self.cache.layer_view(1, ctx, True)))
        for e, rc in zip(entries, rcs):
            self.cache.commit(rc, rc.num_tokens + len(e.tokens))
        return out


# ------------------------------------------------------------------ small kernels

@pytest.mark.parametrize("buckets,mp,mc", [(211, 31, 5), (7919, 77, 1), (5, 0, 1), (64, 1, 0)])
def test_pair_embedding_over_portions(buckets, mp, mc):
    """The row of the pair table depends on the token before: it is kept per request, so a prompt cut anywhere
    (also into single tokens, also beside another request) gives the same rows; a sequence's first token takes
    the last row of the table."""
    from rllm_b200.parts import PairEmbedding
    V, W = 90, 40
    w = {"embed": rnd(V, W, seed=1), "bigram": rnd(buckets + 1, W, seed=2), "embed.norm": rnd(W, seed=3) + 1}
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}, "norm": {"eps": 1e-5}}
    emb = PairEmbedding(V, W, buckets, mp, mc, eps=1e-5)
    bind(emb, w, "float32")
    ids = {"a": B.random_prompt(37, V, 5), "b": B.random_prompt(12, V, 6)}
    want = {k: P.embed(cfg, {k_: v.double() for k_, v in w.items()}, t) for k, t in ids.items()}
    assert P.pair_rows(ids["a"], cfg["embedding"]["bigram"])[0] == buckets
    hs = Harness("float32", [emb.cache_spec()], slots=2)

    def step(entries):
        from rllm_b200.engine import Entry
        es = [Entry(r, toks, []) for r, toks in entries]
        rcs = hs.engine.prepare(es)
        ctx, _ = hs.engine.build_context(es, rcs)
        out = emb.forward(ctx, hs.cache.layer_view(0, ctx, True))
        for e, rc in zip(es, rcs):
            hs.cache.commit(rc, rc.num_tokens + len(e.tokens))
        return out
    a, b = ids["a"], ids["b"]
    got_a = [step([("a", a[:9])])]
    y = step([("b", b[:2]), ("a", a[9:11])])
    got_b = [y[:2]]; got_a.append(y[2:])
    for i in range(11, 20):
        got_a.append(step([("a", a[i: i + 1])]))
    y = step([("a", a[20:]), ("b", b[2:])])
    got_a.append(y[:17]); got_b.append(y[17:])
    assert rel(torch.cat(got_a), want["a"]) < 2e-6 and rel(torch.cat(got_b), want["b"]) < 2e-6
    hs.engine.end(["a", "b"])
    again = step([("c", b)])            # a slot that was used: the token it kept is not this request's
    assert rel(again, want["b"]) < 2e-6


@pytest.mark.parametrize("H", [40, 96, 100, 1024, 2500])
def test_sum_of_normed_and_plain_summands_in_float(H):
    from rllm_b200.kernels import hybrid
    T = 9
    h, a, b = rnd(T, H, seed=1), rnd(T, H, seed=2, scale=3.0), rnd(T, H, seed=3, scale=0.2)
    wa, wb = rnd(H, seed=4) + 1, rnd(H, seed=5) + 1
    parts, extra = rnd(T, 3, H, seed=6), rnd(T, H, seed=7)
    want = h.double() + 0.5 * (P.rms_norm(a.double(), wa.double(), 1e-5) + P.rms_norm(b.double(), wb.double(), 1e-5))
    hd = h.to(DEV)
    hybrid.combine(hd, [(a.to(DEV), wa.to(DEV)), (b.to(DEV), wb.to(DEV))], 0.5, 1e-5)
    assert rel(hd, want) < 2e-6
    hd = h.to(DEV)
    hybrid.combine(hd, [(a.to(DEV), wa.to(DEV)), (b.to(DEV), wb.to(DEV))], 0.5, 1e-5, [parts.to(DEV), extra.to(DEV)])
    assert rel(hd, want + parts.double().sum(1) + extra.double()) < 2e-6
    hd = h.to(DEV)
    hybrid.combine(hd, [], 1.0, 1e-5, [extra.to(DEV)])
    assert rel(hd, h.double() + extra.double()) < 2e-6


@pytest.mark.parametrize("dtype", list(DT))
def test_gated_activations(dtype):
    """The clamps bite on both sides: the inputs reach several times the limit."""
    from rllm_b200.kernels import hybrid
    gu = rnd(37, 2 * 24, seed=1, scale=3.0)
    g, u = gu[:, :24].double(), gu[:, 24:].double()
    tol = 2e-6 if dtype == "float32" else 8e-3
    want = P.gelu_tanh(g) * u
    got = hybrid.glu_act(gu.to(DEV), DT[dtype], "gelu_tanh")
    assert got.dtype == DT[dtype] and rel(got, want) < tol
    for limit, alpha in ((1.25, 1.702), (0.5, 1.0), (7.0, 1.702)):
        gc, uc = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
        want = gc * torch.sigmoid(alpha * gc) * (uc + 1)
        assert float((g > limit).sum()) > 0 and float((u < -limit).sum()) > 0 or limit == 7.0
        assert rel(hybrid.glu_act(gu.to(DEV), DT[dtype], "swish_clamped", limit, alpha), want) < tol


@pytest.mark.parametrize("E,top", [(8, 1), (6, 2), (7, 3), (64, 8), (4, 4), (12, 4)])
def test_router_softmax_over_the_chosen_logits(E, top):
    from rllm_b200.kernels import mix
    z, b = rnd(41, E, seed=E + top, scale=2.0), rnd(E, seed=E, scale=1.5)
    idx, wt = P.route(z.double() + b.double(), top)
    gi, gw = mix.moe_topk(z.to(DEV), top, score="softmax_chosen", bias=b.to(DEV))
    assert torch.equal(gi.cpu().long(), idx) and rel(gw, wt) < 1e-6
    assert rel(gw.sum(1), torch.ones(41)) < 1e-6          # a distribution over the chosen experts
    idx0, _ = P.route(z.double(), top)
    assert not torch.equal(idx0, idx)                      # the bias does change the choice


@pytest.mark.parametrize("F,T", [(64, 700), (48, 700), (40, 700), (40, 90), (32, 90)])
def test_clamped_experts_long_and_short_row_lists(F, T):
    """1,400 (token, expert) rows take the tcgen05 grouped products: with an inner size in steps of 16 the gate/up
    product activates in its epilogue on weights kept in blocks of 16 + 16 rows; other inner sizes and short row
    lists activate in a pass of their own, on either layout. A small limit, so that the clamps bite."""
    from rllm_b200.parts import GluRoutedExperts
    W, E, top, limit = 64, 5, 2, 0.6
    w = {"x.router": rnd(E, W, seed=1, scale=0.5), "x.router.b": rnd(E, seed=2, scale=0.5)}
    for e in range(E):
        w[f"x.e{e}.gate"], w[f"x.e{e}.up"], w[f"x.e{e}.down"] = (rnd(F, W, seed=10 + e, scale=0.3), rnd(F, W, seed=40 + e, scale=0.3),
                                                              rnd(W, F, seed=70 + e, scale=0.3))
    ffn = GluRoutedExperts(W, F, E, top, act="swish_clamped", limit=limit, alpha=P.SWISH_ALPHA, router_bias=True)
    bind(ffn, w, "bfloat16", "x.")
    x = rnd(T, W, seed=3).bfloat16()
    mlp = {"kind": "moe", "expert": {"ff": F, "limit": limit}, "router": {"experts": E, "top": top}}
    want = P.feed_forward(x.double(), as_stored(w, "bfloat16"), "x.", mlp)
    assert rel(P.feed_forward(x.double(), as_stored(w, "bfloat16"), "x.", dict(mlp, expert={"ff": F, "limit": 9.0})), want) > 1e-2

    class Ctx:
        backend = Harness("bfloat16", []).backend
    be, seen = Ctx.backend, []
    orig = be._mix.grouped_gemm_tc
    be._mix.grouped_gemm_tc = lambda *a, **k: (seen.append(a[4]), orig(*a, **k))[1]
    try:
        out = ffn.forward(x.to(DEV), Ctx)
    finally:
        be._mix.grouped_gemm_tc = orig
    if seen:          # the down product joins where its inner size allows
        assert seen[0] == (be._mix.GEPI_SILU_GATED if F % 16 == 0 else be._mix.GEPI_STORE_F32)
    assert (F, T) != (64, 700) or seen == [be._mix.GEPI_SILU_GATED, be._mix.GEPI_STORE_F32]
    assert rel(out.parts.sum(1), want) < 2e-2


@pytest.mark.parametrize("taps", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("dtype", list(DT))
def test_short_convolution_over_portions(dtype, taps):
    """Portions shorter than the taps, single tokens, two requests side by side, a slot that was used."""
    from rllm_b200.kernels import hybrid
    from rllm_b200.parts import StateSpec
    C, col0, n = 37, 5, 29
    x = {"a": rnd(n, col0 + C + 3, seed=taps), "b": rnd(11, col0 + C + 3, seed=taps + 10)}
    w, b = rnd(C, taps, seed=3), rnd(C, seed=4)
    xs = {k: v.to(DT[dtype]) for k, v in x.items()}
    want = {k: P.silu(P.short_conv(v[:, col0: col0 + C].double(), w.double(), b.double())) for k, v in xs.items()}
    spec = StateSpec((("tail", (max(taps - 1, 1), C), torch.float32),))
    hs = Harness(dtype, [spec], slots=2)
    dev = {k: v.to(DEV) for k, v in xs.items()}

    def conv(rows):
        return lambda ctx, cache: hybrid.short_conv(rows, col0, C, w.to(DEV), b.to(DEV), ctx.token_seq, ctx.positions, ctx.cu_q,
                                                    ctx.num_seqs, ctx.state_slots, cache.state["tail"])
    got_a = [hs.run([("a", 1)], conv(dev["a"][:1])), hs.run([("a", 2)], conv(dev["a"][1:3]))]
    y = hs.run([("b", 5), ("a", 1)], conv(torch.cat([dev["b"][:5], dev["a"][3:4]])))
    got_b = [y[:5]]; got_a.append(y[5:])
    y = hs.run([("a", n - 4), ("b", 6)], conv(torch.cat([dev["a"][4:], dev["b"][5:]])))
    got_a.append(y[: n - 4]); got_b.append(y[n - 4:])
    assert rel(torch.cat(got_a), want["a"]) < 2e-6 and rel(torch.cat(got_b), want["b"]) < 2e-6
    hs.engine.end(["a", "b"])
    assert rel(hs.run([("c", 11)], conv(dev["b"])), want["b"]) < 2e-6
    # no bias, no activation
    hs = Harness(dtype, [spec], slots=1)
    y = hs.run([("a", n)], lambda ctx, cache: hybrid.short_conv(dev["a"], col0, C, w.to(DEV), None, ctx.token_seq, ctx.positions,
                                                                ctx.cu_q, ctx.num_seqs, ctx.state_slots, cache.state["tail"], silu=False))
    assert rel(y, P.short_conv(xs["a"][:, col0: col0 + C].double(), w.double())) < 2e-6


def test_unit_vectors_steps_and_decays():
    from rllm_b200.kernels import hybrid
    x = rnd(13, 3 + 4 * 33 + 2, seed=1)
    x[2] *= 1e-4                                            # the eps inside the root matters here
    v = x[:, 3: 3 + 4 * 33].double().view(13, 4, 33)
    want = v / torch.sqrt((v * v).sum(-1, keepdim=True) + 1e-6) * 33 ** -0.5
    xd = x.to(DEV)
    hybrid.unit_heads(xd, 3, 4, 33, 33 ** -0.5, 1e-6)
    assert rel(xd[:, 3: 3 + 4 * 33], want.view(13, -1)) < 2e-6
    assert torch.equal(xd[:, :3].cpu(), x[:, :3]) and torch.equal(xd[:, -2:].cpu(), x[:, -2:])
    # steps far above 20 are themselves (no clamp), far below -20 are exp of themselves
    for dtype in DT:
        z = (rnd(17, 2 + 12, seed=2, scale=3.0) * torch.tensor([1.0] * 8 + [15.0] * 6)).to(DT[dtype])
        bias, a_log = rnd(12, seed=3), rnd(4, seed=4)
        d = P.softplus(z[:, 2:].double() + bias.double())
        a = torch.exp(-torch.exp(a_log.double()).repeat_interleave(3) * d)
        step, decay = hybrid.softplus_decay(z.to(DEV), 2, 12, bias.to(DEV), a_log.to(DEV), want_step=True)
        assert float(d.max()) > 30 and rel(step, d) < 2e-6 and float((decay.cpu().double() - a).abs().max()) < 2e-6


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("n,groups,shared_w", [(48, 1, False), (48, 4, False), (120, 5, True), (36, 2, False), (256, 2, True)])
def test_norm_in_parts_with_a_gate_before_or_after(dtype, n, groups, shared_w):
    from rllm_b200.kernels import hybrid
    T = 11
    y, gate = rnd(T, n, seed=1, scale=2.0), rnd(T, 7 + n, seed=2).to(DT[dtype])
    w = rnd(n // groups if shared_w else n, seed=3) + 1
    wf = w.double().repeat(groups) if shared_w else w.double()
    g = gate[:, 7:].double()
    tol = 2e-6 if dtype == "float32" else 8e-3
    before = P.rms_norm((y.double() * P.silu(g)).view(T, groups, -1), None, 1e-5).reshape(T, n) * wf
    got = hybrid.gated_norm(y.to(DEV), gate.to(DEV), 7, w.to(DEV), 1e-5, groups, DT[dtype], True, "silu")
    assert got.dtype == DT[dtype] and rel(got, before) < tol
    after = P.rms_norm(y.double().view(T, groups, -1), None, 1e-5).reshape(T, n) * wf * torch.sigmoid(g)
    got = hybrid.gated_norm(y.to(DEV), gate.to(DEV), 7, w.to(DEV), 1e-5, groups, DT[dtype], False, "sigmoid")
    assert rel(got, after) < tol
    assert rel(before, after) > 1e-2                       # the order of gate and norm is not a matter of taste


# ------------------------------------------------------------------ attention with mixed heads, over steps

def talk_weights(W, m, seed):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    shapes = {"q": (H * D, W), "k": (G * D, W), "v": (G * V, W), "q.b": (H * D,), "k.b": (G * D,), "v.b": (G * V,),
              "talk": (H, H), "o": (W, H * V)}
    w = {"x." + k: rnd(*s, seed=seed + i, scale=0.25) for i, (k, s) in enumerate(shapes.items())}
    w["x.talk"] = w["x.talk"] * 2 + torch.eye(H)       # far from the identity: a mix that is left out or transposed shows
    return w


def make_talk(W, m, eps=1e-5):
    from rllm_b200.config.bazulorn import TalkAttentionConfig
    from rllm_b200.parts import TalkingHeadsAttention
    c = TalkAttentionConfig.from_dict(m, "mixer")
    return TalkingHeadsAttention(W, c.heads, c.kv_heads, c.dim, c.vdim, scale=c.scale, window=c.window, bias=True,
                                 value_norm=True, sink=0.0, eps=eps)


TALKS = [
    (B.talk(4, 2, 32, 16, 0.2, 21), 4),       # a window over several pages, heads that share keys
    (B.talk(4, 4, 16, 32, 0.3, 16), 16),      # window = page, as many key/value heads as heads
    (B.talk(6, 1, 24, 40, 0.17, 3), 8),       # a window shorter than a page, one key/value head
    (B.talk(2, 2, 48, 48, 0.125, None), 8),   # every key seen
    (B.talk(3, 1, 20, 12, 0.25, 33), 16),     # nothing a multiple of 8
    (B.talk(16, 4, 64, 32, 0.11, 64), 16),    # many heads
    (B.talk(2, 2, 128, 128, 0.09, 50), 16),   # large heads
    (B.talk(8, 4, 16, 16, 0.25, 1), 4),       # a window of the query alone
    (B.talk(1, 1, 40, 24, 0.2, 40), 16),      # one head: the mix is a factor
]


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("m,page", TALKS)
def test_talk_attention_over_steps(dtype, m, page):
    """Inputs at the first positions, at page borders, far back and just inside and just outside the windows of
    queries 96 and 70 are scaled up: their keys then win the scores of the queries that see them. The scores are
    small enough for the sink to hold a good share of every row."""
    W, n = 40, 97
    w = talk_weights(W, m, seed=m["heads"])
    h = rnd(n, W, seed=9)
    size = (m.get("mask") or {"size": 30})["size"]
    special = {0, 1, page - 1, page, 2 * page + 1, 50}
    for qpos in (96, 70):
        special |= {max(0, qpos - size), max(0, qpos - size + 1)}
    for p in special:
        h[p] *= 5.0
    stored = as_stored(strip(w), dtype)
    want = P.talk_attention(h.to(DT[dtype]).double(), stored, "", m, 1e-5)
    # the sink's share is visible, and so are the window's edge and the mix
    assert rel(P.talk_attention(h.to(DT[dtype]).double(), stored, "", m, 1e-5, sink=None), want) > 1e-2
    if m.get("mask") and size > 1:
        off = dict(m, mask={"size": size + 1})
        assert rel(P.talk_attention(h.to(DT[dtype]).double(), stored, "", off, 1e-5), want) > 1e-3
    part = make_talk(W, m)
    bind(part, w, dtype, "x.")
    hd = h.to(DT[dtype]).to(DEV)
    tol = 2e-5 if dtype == "float32" else 4e-2
    outs = {}
    for name, sched in SCHEDULES.items():
        hs = Harness(dtype, [part.cache_spec()], page_size=page, pages=2 + (n + page - 1) // page)
        got, i = [], 0
        for q in cut(n, sched(n)):
            got.append(hs.run([("a", q)], lambda ctx, cache: part.forward(hd[i: i + q], ctx, cache)))
            i += q
            hs.cache.check()
        outs[name] = torch.cat(got)
        assert outs[name].dtype == torch.float32 and rel(outs[name], want) < tol, name
    if dtype == "float32":       # the same numbers however the tokens were cut
        assert all(rel(o, outs["whole"]) < 2e-6 for o in outs.values())
    # two requests in one step, unequal portions beside single tokens; then a third on pages that were used
    hb = rnd(47, W, seed=10)
    hb[3] *= 5.0
    want_b = P.talk_attention(hb.to(DT[dtype]).double(), stored, "", m, 1e-5)
    hbd = hb.to(DT[dtype]).to(DEV)
    hs = Harness(dtype, [part.cache_spec()], page_size=page, pages=4 + (n + 47 + 2 * page - 1) // page)
    got_a, got_b, ia, ib = [], [], 0, 0
    for qa, qb in ((30, 5), (1, 40), (66, 2)):
        y = hs.run([("a", qa), ("b", qb)], lambda ctx, cache: part.forward(
            torch.cat([hd[ia: ia + qa], hbd[ib: ib + qb]]), ctx, cache))
        got_a.append(y[:qa]); got_b.append(y[qa:])
        ia += qa; ib += qb
        hs.cache.check()
    assert rel(torch.cat(got_a), want) < tol and rel(torch.cat(got_b), want_b) < tol
    hs.engine.end(["a", "b"])
    again = hs.run([("c", 47)], lambda ctx, cache: part.forward(hbd, ctx, cache))
    assert rel(again, want_b) < tol


@pytest.mark.parametrize("window", [None, 77, 300])
def test_talk_attention_far_keys_in_long_contexts(window):
    """Contexts of up to 2,048 keys over scattered pages, single query tokens and a portion: one far key, one key
    just inside the window and one just outside are made to stand out. Against the plain implementation on the
    same keys and values."""
    from rllm_b200.kernels import hybrid
    g = torch.Generator().manual_seed(5)
    nh, nkv, kd, vd, page, n_pages = 8, 2, 64, 48, 16, 130
    lens = [1500, 333, 2048, 1]
    S = len(lens)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        k = [(torch.randn(n, nkv, kd, generator=g) * 0.5).to(dtype) for n in lens]
        v = [torch.randn(n, nkv, vd, generator=g).to(dtype) for n in lens]
        qlens = [1, 1, 40, 1]
        q = [torch.randn(ql, nh, kd, generator=g).to(dtype) for ql in qlens]
        for far in ((0, 1499 - (window or 1400) + 1, 1499 - (window or 1400)) if window else (0, 99)):
            k[0][far] = q[0][0].view(nh, kd)[::4] * 3
        mix = (torch.randn(nh, nh, generator=g) * 0.5 + torch.eye(nh))
        kc = torch.zeros(n_pages * S, nkv, page, kd, dtype=dtype)
        vc = torch.zeros(n_pages * S, nkv, page, vd, dtype=dtype)
        bt = torch.randperm(n_pages * S, generator=g).int().view(S, n_pages)
        for s in range(S):
            for p in range(lens[s]):
                kc[bt[s, p // page], :, p % page], vc[bt[s, p // page], :, p % page] = k[s][p], v[s][p]
        want = []
        for s in range(S):
            for r in range(qlens[s]):
                i = lens[s] - qlens[s] + r
                lo = 0 if window is None else max(0, i - window + 1)
                sc = torch.einsum("hd,jhd->hj", q[s][r].double(), k[s][lo: i + 1].double().repeat_interleave(nh // nkv, 1)) * 0.11
                p = torch.exp(sc) / (1 + torch.exp(sc).sum(1, keepdim=True))
                p = mix.double() @ p
                want.append(torch.einsum("hj,jhv->hv", p, v[s][lo: i + 1].double().repeat_interleave(nh // nkv, 1)).reshape(-1))
        want = torch.stack(want)
        pos = torch.cat([torch.arange(n - ql, n) for n, ql in zip(lens, qlens)]).int().to(DEV)
        seq = torch.cat([torch.full((ql,), i) for i, ql in enumerate(qlens)]).int().to(DEV)
        qd = torch.cat([x.reshape(-1, nh * kd) for x in q]).to(DEV)
        got = hybrid.talk_attention_simt(qd, kc.to(DEV), vc.to(DEV), seq, pos, bt.to(DEV), nh, 0.11, mix.to(DEV), window, None,
                                         torch.zeros(nh, device=DEV))
        assert rel(got, want) < tol, dtype
        if dtype == torch.bfloat16:          # the tensor-core kernel: decoded tokens and a portion in one launch, then tokens alone
            assert hybrid.talk_mma_supported(dtype, nh, kd, vd, page)
            cu = torch.tensor([0] + list(itertools.accumulate(qlens)), dtype=torch.int32, device=DEV)
            got = hybrid.talk_attention_mma(qd, kc.to(DEV), vc.to(DEV), seq, pos, bt.to(DEV), cu, S, max(qlens), nh, 0.11,
                                            mix.to(DEV), window, None, torch.zeros(nh, device=DEV))
            assert rel(got, want) < tol
            one = [0, 1, 42]
            cu1 = torch.arange(4, dtype=torch.int32, device=DEV)
            got1 = hybrid.talk_attention_mma(qd[one], kc.to(DEV), vc.to(DEV), seq[one], pos[one], bt[[0, 1, 3]].to(DEV), cu1, 3, 1,
                                             nh, 0.11, mix.to(DEV), window, None, torch.zeros(nh, device=DEV))
            assert rel(got1, want[one]) < tol


# ------------------------------------------------------------------ the recurrent mixers, over steps and slots

def ssm_weights(W, m, seed):
    H, Pd, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    I, C = H * Pd, H * Pd + 2 * G * N
    shapes = {"in": (2 * I + 2 * G * N + H, W), "conv": (C, taps), "conv.b": (C,), "dt_bias": (H,), "A_log": (H,), "D": (H,),
              "norm": (I,), "o": (W, I)}
    w = {"x." + k: rnd(*s, seed=seed + i, scale=0.25) for i, (k, s) in enumerate(shapes.items())}
    w["x.norm"], w["x.D"] = w["x.norm"] + 1, w["x.D"] + 1
    w["x.A_log"] = w["x.A_log"] - 3.0              # decays near one: the first tokens stay in the state
    w["x.conv"] = w["x.conv"] + 0.5
    return w


def delta_weights(W, m, seed):
    H, G, D, V, taps, ra, rg = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], m["decay_rank"], m["gate_rank"]
    shapes = {"q": (G * D, W), "k": (G * D, W), "v": (H * V, W), "q.conv": (G * D, taps), "k.conv": (G * D, taps),
              "v.conv": (H * V, taps), "b": (H, W), "a1": (ra, W), "a2": (H * D, ra), "dt_bias": (H * D,), "A_log": (H,),
              "g1": (rg, W), "g2": (H * V, rg), "norm": (V,), "o": (W, H * V)}
    w = {"x." + k: rnd(*s, seed=seed + i, scale=0.25) for i, (k, s) in enumerate(shapes.items())}
    w["x.norm"] = w["x.norm"] + 1
    w["x.A_log"] = w["x.A_log"] - 3.5
    w["x.b"] = w["x.b"] * 0.3                      # small writes: the state keeps what the first tokens wrote
    for c in ("q.conv", "k.conv", "v.conv"):
        w["x." + c] = w["x." + c] + 0.5
    return w


def make_recurrent(kind, W, m, eps=1e-5):
    from rllm_b200.parts import DeltaRuleMixer, StateSpaceMixer
    if kind == "ssm":
        return StateSpaceMixer(W, m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"], m["conv"], eps=eps)
    return DeltaRuleMixer(W, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], eps=eps, unit_eps=1e-6)


RECURRENT = [
    ("ssm", B.ssm(4, 12, 20, 2, 2, 3)),
    ("ssm", B.ssm(3, 24, 8, 1, 1, 2)),             # one group, one part
    ("ssm", B.ssm(2, 36, 44, 2, 4, 4)),            # more parts than heads
    ("ssm", B.ssm(6, 8, 12, 3, 1, 1)),             # one tap: no convolution state
    ("ssm", B.ssm(5, 6, 14, 5, 5, 5)),             # a group per head
    ("ssm", B.ssm(2, 64, 128, 1, 2, 4)),           # a large state
    ("ssm", B.ssm(3, 20, 32, 3, 1, 2)),            # a warp's lanes a state
    ("delta", B.delta(4, 2, 20, 24, 4, 8, 12, None)["mixer"]),
    ("delta", B.delta(1, 1, 64, 72, 2, 16, 4, None)["mixer"]),
    ("delta", B.delta(6, 3, 8, 8, 5, 4, 20, None)["mixer"]),
    ("delta", B.delta(2, 2, 130, 20, 1, 8, 8, None)["mixer"]),     # key channels beyond a warp's lanes, one tap
    ("delta", B.delta(2, 1, 128, 128, 3, 8, 8, None)["mixer"]),    # a large state
    ("delta", B.delta(2, 2, 256, 24, 2, 8, 8, None)["mixer"]),     # eight lanes a value column
]


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("kind,m", RECURRENT)
def test_recurrent_mixers_over_steps_and_slots(dtype, kind, m):
    """Decays near one keep the first tokens in the state for the whole sequence; a request that takes over a
    slot must not see what its predecessor left there (neither the state nor the convolution's last inputs)."""
    W, n = 48, 83
    w = (ssm_weights if kind == "ssm" else delta_weights)(W, m, seed=m["heads"] + m["vdim"])
    plain = P.state_space if kind == "ssm" else P.delta_rule
    part = make_recurrent(kind, W, m)
    bind(part, w, dtype, "x.")
    seqs = {"a": rnd(n, W, seed=20), "b": rnd(31, W, seed=21), "c": rnd(n, W, seed=22)}
    seqs["a"][0] *= 6.0                      # the first token must still be felt at the end
    stored = as_stored(strip(w), dtype)
    want = {k: plain(x.to(DT[dtype]).double(), stored, "", m, 1e-5, stored_as(dtype)) for k, x in seqs.items()}
    x2 = seqs["a"].clone(); x2[0] /= 6.0     # it is in fact felt at the end (else a lost state would not show)
    assert rel(plain(x2.to(DT[dtype]).double(), stored, "", m, 1e-5)[-1:], want["a"][-1:]) > 1e-3
    dev = {k: x.to(DT[dtype]).to(DEV) for k, x in seqs.items()}
    outs = {}
    for name, sched in SCHEDULES.items():
        hs = Harness(dtype, [part.cache_spec()], slots=2)
        got, i = [], 0
        for q in cut(n, sched(n)):
            got.append(hs.run([("a", q)], lambda ctx, cache: part.forward(dev["a"][i: i + q], ctx, cache)))
            i += q
        outs[name] = torch.cat(got)
        assert outs[name].dtype == torch.float32 and close(outs[name], want["a"], dtype), name
        hs.engine.end(["a"])
        got_b = hs.run([("b", 31)], lambda ctx, cache: part.forward(dev["b"], ctx, cache))
        assert close(got_b, want["b"], dtype)
        hs.engine.end(["b"])
        # two requests in one step, unequal portions; c takes a slot that was used (two slots, four requests)
        both = hs.run([("c", 50), ("b2", 20)], lambda ctx, cache: part.forward(
            torch.cat([dev["c"][:50], dev["b"][:20]]), ctx, cache))
        assert close(both[:50], want["c"][:50], dtype) and close(both[50:], want["b"][:20], dtype)
        rest = hs.run([("b2", 11), ("c", 33)], lambda ctx, cache: part.forward(
            torch.cat([dev["b"][20:], dev["c"][50:]]), ctx, cache))
        assert close(rest[:11], want["b"][20:], dtype) and close(rest[11:], want["c"][50:], dtype)
        hs.cache.check()
    if dtype == "float32":
        assert all(rel(o, outs["whole"]) < 2e-6 for o in outs.values())


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("kind,m", [RECURRENT[0], RECURRENT[6]])
def test_recurrent_mixers_long_portions_then_single_tokens(dtype, kind, m):
    """Portions of several hundred tokens, two sequences of unequal length in one step, one of them with a state
    from an earlier step; then single tokens that continue from the state the long portions left."""
    W = 32
    w = (ssm_weights if kind == "ssm" else delta_weights)(W, m, seed=50)
    plain = P.state_space if kind == "ssm" else P.delta_rule
    part = make_recurrent(kind, W, m)
    bind(part, w, dtype, "x.")
    seqs = {"a": rnd(30 + 500 + 4, W, seed=60), "b": rnd(130 + 3, W, seed=61)}
    seqs["a"][31] *= 6.0
    stored = as_stored(strip(w), dtype)
    want = {k: plain(x.to(DT[dtype]).double(), stored, "", m, 1e-5, stored_as(dtype)) for k, x in seqs.items()}
    dev = {k: x.to(DT[dtype]).to(DEV) for k, x in seqs.items()}
    hs = Harness(dtype, [part.cache_spec()], slots=2)
    got = {"a": [], "b": []}
    got["a"].append(hs.run([("a", 30)], lambda ctx, cache: part.forward(dev["a"][:30], ctx, cache)))
    y = hs.run([("a", 500), ("b", 130)], lambda ctx, cache: part.forward(torch.cat([dev["a"][30:530], dev["b"][:130]]), ctx, cache))
    got["a"].append(y[:500]); got["b"].append(y[500:])
    for i in range(3):
        y = hs.run([("b", 1), ("a", 1)], lambda ctx, cache: part.forward(
            torch.cat([dev["b"][130 + i: 131 + i], dev["a"][530 + i: 531 + i]]), ctx, cache))
        got["b"].append(y[:1]); got["a"].append(y[1:])
    got["a"].append(hs.run([("a", 1)], lambda ctx, cache: part.forward(dev["a"][533:], ctx, cache)))
    assert close(torch.cat(got["a"]), want["a"], dtype) and close(torch.cat(got["b"]), want["b"], dtype)


# ------------------------------------------------------------------ whole models

def requests_for(name, lens=(9, 61, 23, 150, 37, 2)):
    vocab = B.TINY[name][0]["vocab"]
    return {f"r{i}": B.random_prompt(n, vocab, 100 * len(name) + ord(name[1]) + i) for i, n in enumerate(lens)}


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("bazulorn")
    return {n: B.make_model_dir(root, n) for n in B.TINY}


@pytest.fixture(scope="module")
def plain(dirs):
    out = {}
    for name, d in dirs.items():
        cfg, w = P.read_model_dir(d)
        out[name] = {}
        for rid, toks in requests_for(name).items():
            lg = P.forward(cfg, w, toks).numpy()
            out[name].update({(rid, i): lg[i] for i in range(len(toks))})
    return out


FAMILIES = {"whole": replay.whole, "decode": lambda r: replay.prefill_then_decode(r, tail=40), "portions": replay.portions,
            "mixed": lambda r: replay.mixed(r, max_live=3)}


def engine_for(dirs, name, dtype, steps, reqs, max_requests=3):
    from rllm_b200.engine import load_engine
    return load_engine(dirs[name], dtype=dtype, page_size=B.TINY[name][4],
                       max_tokens=replay.max_live_tokens(steps, reqs), max_requests=max_requests)


@pytest.mark.parametrize("name", list(B.TINY))
def test_residual_stream_after_every_layer(dirs, name):
    """In float32, layer by layer: the first layer that differs names the mechanism."""
    from rllm_b200.engine import Entry, load_engine
    cfg, w = P.read_model_dir(dirs[name])
    toks = B.random_prompt(45, cfg["vocab"], 9)
    _, kept = P.forward(cfg, w, toks, keep_layers=True)
    eng = load_engine(dirs[name], dtype="float32", page_size=B.TINY[name][4], max_tokens=64, max_requests=1)
    got = []
    for b in eng.model.blocks:          # a block adds to the stream it is given, in place

        def wrap(h, ctx, cache, f=b.forward):
            out = f(h, ctx, cache)
            got.append(h.detach().float().cpu().clone())
            return out
        b.forward = wrap
    eng.step([Entry("a", toks, [])])
    assert len(got) == len(kept)
    for i, (g, k) in enumerate(zip(got, kept)):
        assert rel(g, k) < 2e-5, f"{name}: the stream differs after layer {i} ({cfg['layers'][i]['type']})"


@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("name", list(B.TINY))
def test_family_matches_plain(dirs, plain, name, dtype, family):
    """The pool holds just what the live requests need and there are three state slots for six requests:
    pages and slots are used again."""
    reqs = requests_for(name)
    steps = FAMILIES[family](reqs)
    eng = engine_for(dirs, name, dtype, steps, reqs)
    got = replay.run_in_process(eng, steps)
    eng.check()
    if dtype == "float32":
        check(got, plain[name], 3e-5, f"{name} float32 {family}")
    else:
        check(got, plain[name], 6e-2, f"{name} bfloat16 {family}", allow=0.25)


@pytest.mark.parametrize("name", list(B.TINY))
def test_float32_is_the_same_however_it_is_cut(dirs, name):
    reqs = requests_for(name)
    ref = None
    for family, make in FAMILIES.items():
        steps = make(reqs)
        got = replay.run_in_process(engine_for(dirs, name, "float32", steps, reqs), steps)
        if ref is None:
            ref = got
        else:
            worst = max(float(np.abs(got[k] - ref[k]).max()) for k in ref)
            assert worst <= 2e-6, f"{name} {family}: differs from whole prompts by {worst}"


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 6e-2)])
def test_long_decoding_through_graphs(dirs, dtype, tol):
    """Two requests decoded side by side for 120 steps from prompts of 3 and 30 tokens: the window passes over
    decoded tokens, pages are given back on the way, the states and the last token of each request are carried
    through replayed graphs."""
    from rllm_b200.engine import Entry, load_engine
    name = "BA"
    cfg, w = P.read_model_dir(dirs[name])
    toks = {"x": B.random_prompt(123, cfg["vocab"], 5), "y": B.random_prompt(150, cfg["vocab"], 6)}
    want = {k: P.forward(cfg, w, t).numpy() for k, t in toks.items()}
    eng = load_engine(dirs[name], dtype=dtype, page_size=4, max_tokens=320, max_requests=2)
    eng.step([Entry("x", toks["x"][:3], []), Entry("y", toks["y"][:30], [])])
    got = {}
    for i in range(120):
        lg = eng.step([Entry("x", [toks["x"][3 + i]], [0]), Entry("y", [toks["y"][30 + i]], [0])]).float().cpu().numpy()
        got[("x", 3 + i)], got[("y", 30 + i)] = lg[0], lg[1]
        eng.cache.check()
    eng.check()
    assert eng.graphs is not None and eng.graph_steps == 120
    check(got, {(k, i): want[k][i] for (k, i) in got}, tol, f"long decoding {dtype}", allow=0.0 if dtype == "float32" else 0.25)


@pytest.mark.parametrize("name", ["BB", "BC", "BD"])
def test_greedy_generation_through_the_entry_point(dirs, name):
    """LLM.generate (scheduler, sampler, run-ahead decoding) against greedy decoding with the plain model."""
    from rllm_b200.api import LLM
    from rllm_b200.sampling import SamplingParams
    cfg, w = P.read_model_dir(dirs[name])
    prompts = [B.random_prompt(n, cfg["vocab"], 70 + n) for n in (4, 19, 33)]
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(12):
            lg = P.forward(cfg, w, toks)[-1]
            top2 = lg.topk(2).values
            toks.append(int(lg.argmax()))
            if float(top2[0] - top2[1]) < 1e-4:      # a close call: the rest of this prompt proves nothing
                break
        want.append(toks[len(p):])
    llm = LLM(dirs[name], dtype="float32", page_size=B.TINY[name][4], num_pages=40, max_active=2, max_chunk=16)
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for g, w_ in zip(got, want):
        assert g[: len(w_)] == w_
    llm.engine.cache.check()


def test_ten_requests_decode_in_a_padded_graph(dirs):
    """Ten requests decode side by side: their graph has more rows than requests; the stand-in rows have no state
    slot, pages or wanted logits, and must neither disturb the others nor touch a state or a kept token."""
    from rllm_b200.engine import Entry, load_engine
    name = "BA"
    cfg, w = P.read_model_dir(dirs[name])
    toks = {i: B.random_prompt(5 + 3 * i + 9, cfg["vocab"], 300 + i) for i in range(10)}
    want = {i: P.forward(cfg, w, t).numpy() for i, t in toks.items()}
    eng = load_engine(dirs[name], dtype="float32", page_size=4, max_tokens=10 * 64, max_requests=10)
    eng.step([Entry(i, t[:-9], []) for i, t in toks.items()])
    got = {}
    for k in range(9):
        lg = eng.step([Entry(i, [t[len(t) - 9 + k]], [0]) for i, t in toks.items()]).float().cpu().numpy()
        for row, (i, t) in enumerate(toks.items()):
            got[(i, len(t) - 9 + k)] = lg[row]
    eng.check()
    assert eng.graph_steps == 9
    check(got, {(i, p): want[i][p] for (i, p) in got}, 3e-5, "padded graph")


def test_command_line_runs_the_design(dirs):
    name = "BE"
    cfg, w = P.read_model_dir(dirs[name])
    prompt = B.random_prompt(11, cfg["vocab"], 3)
    toks = prompt + P.greedy(cfg, w, prompt, 5)
    r = subprocess.run([sys.executable, os.path.join(replay.ROOT, "bin", "rllm"), "run", "--model", dirs[name],
                        "--prompt-ids", " ".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0",
                        "--dtype", "float32", "--kv-pages", "32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [int(x) for x in r.stdout.split()] == toks[len(prompt):]


@pytest.mark.parametrize("name,dtype", [("BC", "float32"), ("BD", "bfloat16")])
def test_trace_program_runs_the_design(dirs, plain, tmp_path, name, dtype):
    """BD has no attention at all: the program then has no pages to size."""
    reqs = requests_for(name)
    steps = replay.mixed(reqs, max_live=4)
    got = replay.run_program(dirs[name], dtype, steps, str(tmp_path / "out"), replay.max_live_tokens(steps, reqs),
                             B.TINY[name][0]["vocab"], extra_args=["--page-size", "16"])
    if dtype == "float32":
        check(got, plain[name], 3e-5, "trace program")
    else:
        check(got, plain[name], 6e-2, "trace program bfloat16", allow=0.25)
