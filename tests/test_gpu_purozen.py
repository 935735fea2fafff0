"""Purozen on the GPU against the plain implementation (tests/plain_purozen.py): each mechanism alone, then whole
models through the step function, the scheduler and the trace program; prompts whole, in portions down to two
tokens, decoded token by token, and in mixed batches with pages and slots used again. Where random inputs would hide
a fault the inputs are made so that it shows: the input at one position is scaled up, or (where queries and keys
are normed) pointed the way of the queries that should find it, so that its key wins every score it takes part in
(a window's edge that is one off, a kept first token that is lost, a far key), update gates
are kept small so that the first token is still felt at the end, and stored norm weights are small enough to vanish
if they were added to one in 16 bits."""
import itertools
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_purozen as P
import purozen_tiny as Z
import replay
from test_gpu_zukotar import SCHEDULES, Harness, check, cut, rel, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def as_stored(weights, dtype, prefix="x."):
    """The weights as the run keeps them (rounded to its type), under names without `prefix`."""
    return {k[len(prefix):]: (v.to(DT[dtype]) if v.is_floating_point() else v).to(F64) for k, v in weights.items()}


def stored_as(dtype):
    """What a run of this type does to the activations it keeps between two kernels."""
    return P.exact if dtype == "float32" else (lambda x: x.to(torch.bfloat16).to(F64))


def bind(part, weights, dtype, prefix=""):
    """Give a part the named float tensors as the loader would (matrices in the run dtype; a scalar stays a scalar)."""
    from rllm_b200.weights.loader import storage_dtype
    part.prefix = prefix
    for c in part.children():
        c.prefix = prefix
    for p in part.params():
        pieces = [weights[prefix + s.name] for s in p.sources]
        t = pieces[0] if len(pieces) == 1 else torch.cat(pieces, 0)
        setattr(part, p.attr, t.to(storage_dtype(p.role, torch.bfloat16, DT[dtype])).to(DEV).contiguous())
    for p in part.walk():
        p.finalize(torch.device(DEV), DT[dtype])


class TwoLayers(Harness):
    """A harness for two parts with a cache layer each (two mixers side by side, or two layers that share something
    within a step): `fn` gets a tuple of two layer caches."""

    def run(self, entries, fn):
        from rllm_b200.engine import Entry
        entries = [Entry(r, [0] * n, []) for r, n in entries]
        rcs = self.engine.prepare(entries)
        ctx, _ = self.engine.build_context(entries, rcs)
        out = fn(ctx, (self.cache.layer_view(0, ctx, True), self.cache.layer_view(1, ctx, True)))
        for e, rc in zip(entries, rcs):
            self.cache.commit(rc, rc.num_tokens + len(e.tokens))
        return out


def over_schedules(dtype, n, run_step, new_harness, want, tol):
    """Run the n rows through every cutting of SCHEDULES, each on a harness of its own; in float32 the cuttings must
    agree to rounding. Returns the outputs by name."""
    outs = {}
    for name, sched in SCHEDULES.items():
        hs = new_harness()
        got, i = [], 0
        for q in cut(n, sched(n)):
            got.append(run_step(hs, [("a", q)], {"a": (i, i + q)}))
            i += q
            hs.cache.check()
        outs[name] = torch.cat(got)
        assert outs[name].dtype == torch.float32 and rel(outs[name], want) < tol, name
    if dtype == "float32":
        assert all(rel(o, outs["whole"]) < 2e-6 for o in outs.values())
    return outs


# ------------------------------------------------------------------ small kernels

@pytest.mark.parametrize("W", [40, 96, 100, 1024])
def test_gated_sum_into_the_stream(W):
    """h += sigmoid(g + b) * (c0 y0 + c1 y1): one or two summands, a gate that is a view of wider rows, no bias."""
    from rllm_b200.kernels import hybrid
    T = 11
    h, y0, y1, b = rnd(T, W, seed=1), rnd(T, W, seed=2, scale=2.0), rnd(T, W, seed=3), rnd(W, seed=4)
    wide = rnd(T, W + 8, seed=5, scale=2.0)
    gate = wide[:, 4: 4 + W]
    for terms, bias, g in (([(y0, 1.0)], b, gate.contiguous()), ([(y0, 0.7), (y1, -1.3)], b, gate.contiguous()),
                           ([(y0, 0.7), (y1, 2.0)], None, gate), ([(y1, 0.25)], b, gate)):
        want = h.double() + torch.sigmoid(g.double() + (0 if bias is None else bias.double())) * sum(c * y.double() for y, c in terms)
        hd = h.to(DEV)
        gd = wide.to(DEV)[:, 4: 4 + W] if not g.is_contiguous() else g.to(DEV)
        hybrid.gated_add(hd, gd, None if bias is None else bias.to(DEV), [(y.to(DEV), c) for y, c in terms])
        assert rel(hd, want) < 2e-6


@pytest.mark.parametrize("dtype", list(DT))
def test_gelu_rows(dtype):
    from rllm_b200.kernels import hybrid
    x = rnd(37, 50, seed=1, scale=2.5)
    got = hybrid.act_rows(x.to(DEV), DT[dtype], "gelu_tanh")
    assert got.dtype == DT[dtype] and rel(got, P.gelu_tanh(x.double())) < (2e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("nkv,vd", [(2, 24), (1, 12), (4, 64), (3, 40)])
def test_values_mixed_on_their_way_into_the_pages(dtype, nkv, vd):
    """The kernel that caches keys and values stores (1 - lam) v + lam v_first, formed in float and rounded once, and
    leaves the projected rows as they were; rows without a slot are not stored."""
    from rllm_b200.kernels import sink
    T, nh, kd, page = 21, 2 * nkv, 16, 4
    cols = (nh + nkv) * kd + nkv * vd
    proj = rnd(T, cols + 8, seed=1).to(DT[dtype])
    first = rnd(T, nkv * vd + 16, seed=2).to(DT[dtype])
    lam = torch.tensor([0.3125])
    slots = torch.randperm(32)[:T].int()
    slots[5] = -1
    kc = torch.zeros(8, nkv, page, kd, dtype=DT[dtype], device=DEV)
    vc = torch.zeros(8, nkv, page, vd, dtype=DT[dtype], device=DEV)
    pd = proj.to(DEV)
    sink.qk_norm_rope_store(pd[:, :cols], 0, nh * kd, (nh + nkv) * kd, nh, nkv, kd, vd, 0, None, None, 1e-6, None, slots.to(DEV), kc, vc,
                            first.to(DEV)[:, 8: 8 + nkv * vd], lam.to(DEV))
    assert torch.equal(pd.cpu(), proj)
    v = proj[:, (nh + nkv) * kd: cols].double().view(T, nkv, vd)
    want = (1 - 0.3125) * v + 0.3125 * first[:, 8: 8 + nkv * vd].double().view(T, nkv, vd)
    for t in range(T):
        s_ = int(slots[t])
        if s_ < 0:
            continue
        assert rel(vc[s_ // page, :, s_ % page], want[t]) < (2e-6 if dtype == "float32" else 5e-3)
        assert torch.equal(kc[s_ // page, :, s_ % page].cpu(), proj[t, nh * kd: (nh + nkv) * kd].view(nkv, kd))
    assert int((vc.abs().sum((1, 3)) > 0).sum()) == T - 1


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("T,K,N", [(3, 64, 96), (40, 128, 320), (300, 256, 512), (5, 72, 100)])
def test_gelu_behind_a_product_with_and_without_the_norm_in_front(dtype, T, K, N):
    """act(x W^T) as the feed-forward asks for it: in bfloat16 the activation runs on the float accumulator in the
    product's epilogue (few tokens: the norm in front of the same kernel), rounded once."""
    from rllm_b200.kernels.backend import Backend
    be = Backend(DT[dtype], DEV)
    h, g, w = rnd(T, K, seed=1, scale=2.0), rnd(K, seed=2, scale=0.2) + 1, rnd(N, K, seed=3, scale=0.2)
    ws = w.to(DT[dtype])
    n = P.unit_rms(h.double(), 1e-5) * g.double()
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    got = be.linear_act(be.normed(h.to(DEV), g.to(DEV), 1e-5), ws.to(DEV), "gelu_tanh")
    assert got.dtype == DT[dtype] and rel(got, P.gelu_tanh(stored_as(dtype)(n) @ ws.double().T)) < tol
    x = n.to(DT[dtype])
    got = be.linear_act(x.to(DEV), ws.to(DEV), "gelu_tanh")
    assert rel(got, P.gelu_tanh(x.double() @ ws.double().T)) < tol


@pytest.mark.parametrize("dtype", list(DT))
def test_norm_weight_stored_around_zero_is_added_in_float(dtype):
    """Stored weights of a few thousandths: 1 + w formed in 16 bits would lose them."""
    from rllm_b200.parts import RMSNorm
    W = 72
    w = {"x.n": rnd(W, seed=1, scale=3e-3)}
    norm = RMSNorm(W, 1e-5, "n", offset=1.0)
    bind(norm, w, dtype, "x.")
    h = rnd(9, W, seed=2, scale=4.0)
    from rllm_b200.kernels.backend import Backend
    got = norm.forward_f32(h.to(DEV), type("C", (), {"backend": Backend(DT[dtype], DEV)})())
    stored = as_stored(w, dtype)["n"]
    assert rel(got, P.norm_around_zero(h.double(), stored, 1e-5)) < 2e-6
    assert rel(got, P.unit_rms(h.double(), 1e-5)) > 1e-3          # the weight is felt


# ------------------------------------------------------------------ the gated recurrence, over steps and slots

def gru_weights(W, R, seed, slow=True):
    shapes = {"z": (R, W), "z.b": (R,), "x": (R, W), "x.b": (R,), "g": (R, W), "o": (W, R)}
    w = {"x." + k: rnd(*s, seed=seed + i, scale=0.3) for i, (k, s) in enumerate(shapes.items())}
    if slow:                      # small update gates on half the channels: the first token is felt at the end
        w["x.z.b"][::2] -= 7.0
        w["x.z"][::2] *= 0.1
    return w


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("W,R", [(40, 37), (48, 300), (64, 128), (24, 1)])
def test_gated_recurrence_over_steps_and_slots(dtype, W, R):
    from rllm_b200.parts import MinGRUMixer
    n = 97
    w = gru_weights(W, R, seed=R)
    h = rnd(n, W, seed=9)
    h[0] *= 5.0
    m = {"width": R}
    x = h.to(DT[dtype])
    want = P.min_gru(x.double(), as_stored(w, dtype), "", m, stored=stored_as(dtype))
    # the first token is still felt by the last one
    x0 = x.double().clone()
    x0[0] = 0
    assert rel(P.min_gru(x0, as_stored(w, dtype), "", m)[-1:], want[-1:]) > 1e-3
    part = MinGRUMixer(W, R)
    bind(part, w, dtype, "x.")
    hd = x.to(DEV)
    tol = 2e-5 if dtype == "float32" else 1.5e-2

    def step(hs, entries, spans):
        rows = torch.cat([hd[a:b] for a, b in spans.values()])
        return hs.run(entries, lambda ctx, cache: part.forward(rows, ctx, cache))
    over_schedules(dtype, n, step, lambda: Harness(dtype, [part.cache_spec()], slots=2), want, tol)
    # two requests in one step, unequal portions beside single tokens; then a third in a slot that was used
    hb = rnd(47, W, seed=10).to(DT[dtype])
    want_b = P.min_gru(hb.double(), as_stored(w, dtype), "", m, stored=stored_as(dtype))
    hbd = hb.to(DEV)
    hs = Harness(dtype, [part.cache_spec()], slots=2)
    got_a, got_b, ia, ib = [], [], 0, 0
    for qa, qb in ((30, 5), (1, 40), (66, 2)):
        y = hs.run([("a", qa), ("b", qb)], lambda ctx, cache: part.forward(torch.cat([hd[ia: ia + qa], hbd[ib: ib + qb]]), ctx, cache))
        got_a.append(y[:qa]); got_b.append(y[qa:])
        ia += qa; ib += qb
    assert rel(torch.cat(got_a), want) < tol and rel(torch.cat(got_b), want_b) < tol
    hs.engine.end(["a", "b"])
    again = hs.run([("c", 47)], lambda ctx, cache: part.forward(hbd, ctx, cache))       # starts from zero
    assert rel(again, want_b) < tol


@pytest.mark.parametrize("dtype", list(DT))
def test_gated_recurrence_long_portions_run_in_pieces_side_by_side(dtype):
    """Portions longer than two chunks are cut into pieces whose maps are folded in order: 333 tokens beside 70 and a
    single one, the state carried on into further portions and single tokens; against the walk token by token."""
    from rllm_b200.kernels import hybrid
    from rllm_b200.parts import MinGRUMixer
    W, R = 40, 150
    w = gru_weights(W, R, seed=3)
    m = {"width": R}
    lens = {"a": 333 + 100 + 3, "b": 70 + 1 + 3, "c": 1 + 200 + 3}
    hsrc = {k: rnd(n, W, seed=20 + i).to(DT[dtype]) for i, (k, n) in enumerate(lens.items())}
    want = {k: P.min_gru(x.double(), as_stored(w, dtype), "", m, stored=stored_as(dtype)) for k, x in hsrc.items()}
    part = MinGRUMixer(W, R)
    bind(part, w, dtype, "x.")
    hs = Harness(dtype, [part.cache_spec()], slots=3)
    at = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    plan = [{"a": 333, "b": 70, "c": 1}, {"a": 100, "b": 1, "c": 200}] + [{"a": 1, "b": 1, "c": 1}] * 3
    assert 333 > 2 * hybrid.MINGRU_CHUNK and 70 > 2 * hybrid.MINGRU_CHUNK
    for st in plan:
        rows = torch.cat([hsrc[k][at[k]: at[k] + q] for k, q in st.items()]).to(DEV)
        y = hs.run(list(st.items()), lambda ctx, cache: part.forward(rows, ctx, cache))
        o = 0
        for k, q in st.items():
            got[k].append(y[o: o + q]); o += q; at[k] += q
    for k in lens:
        assert rel(torch.cat(got[k]), want[k]) < (2e-5 if dtype == "float32" else 1.5e-2), k


# ------------------------------------------------------------------ attention with sigmoid weights, over steps

def sig_weights(W, m, seed):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    shapes = {"q": (H * D, W), "k": (G * D, W), "v": (G * V, W), "pb": (H,), "o": (W, H * V)}
    w = {"x." + k: rnd(*s, seed=seed + i, scale=0.25) for i, (k, s) in enumerate(shapes.items())}
    w["x.pb"] = w["x.pb"] * 6 - 1.0           # biases that move the weights visibly, of both signs
    return w


def make_sig(W, m):
    from rllm_b200.parts import SinkGQAttention
    return SinkGQAttention(W, m["heads"], m["kv_heads"], m["dim"], m["vdim"], scale=m["scale"], weights="sigmoid",
                           score_bias="pb")


SIGS = [
    (Z.sig(4, 2, 32, 16, 0.2), 4),        # heads that share keys, several pages
    (Z.sig(3, 3, 8, 40, 0.3), 16),        # as many key/value heads as heads
    (Z.sig(6, 1, 24, 40, 0.17), 8),       # one key/value head
    (Z.sig(2, 2, 48, 80, 0.125), 8),      # values wider than keys, in steps of 16
    (Z.sig(3, 1, 20, 12, 0.25), 16),      # nothing a multiple of 8
    (Z.sig(16, 4, 64, 32, 0.11), 16),     # many heads
    (Z.sig(2, 2, 128, 128, 0.09), 16),    # large heads, equal sizes
    (Z.sig(1, 1, 40, 24, 0.2), 4),        # one head
]


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("m,page", SIGS)
def test_sigmoid_attention_over_steps(dtype, m, page):
    """Inputs at the first positions, at page borders and far back are scaled up: their keys weigh close to one or
    close to zero for the queries that see them. Nothing is normalised, so a key that is lost or seen twice moves the
    row by its value."""
    W, n = 40, 97
    w = sig_weights(W, m, seed=m["heads"])
    h = rnd(n, W, seed=9)
    for p in {0, 1, page - 1, page, 2 * page + 1, 50}:
        h[p] *= 5.0
    x = h.to(DT[dtype])
    st = as_stored(w, dtype)
    want = P.sigmoid_attention(x.double(), st, "", m, stored=stored_as(dtype))
    assert rel(P.sigmoid_attention(x.double(), st, "", m, bias=False), want) > 1e-2      # the bias is felt
    part = make_sig(W, m)
    assert part.cache_spec().window is None and part.cache_spec().keep_first == 0
    bind(part, w, dtype, "x.")
    hd = x.to(DEV)
    tol = TOL[dtype]

    def step(hs, entries, spans):
        rows = torch.cat([hd[a:b] for a, b in spans.values()])
        return hs.run(entries, lambda ctx, cache: part.forward(rows, ctx, cache))
    over_schedules(dtype, n, step, lambda: Harness(dtype, [part.cache_spec()], page_size=page, pages=2 + (n + page - 1) // page),
                   want, tol)
    hb = rnd(47, W, seed=10)
    hb[3] *= 5.0
    xb = hb.to(DT[dtype])
    want_b = P.sigmoid_attention(xb.double(), st, "", m, stored=stored_as(dtype))
    hbd = xb.to(DEV)
    hs = Harness(dtype, [part.cache_spec()], page_size=page, pages=4 + (n + 47 + 2 * page - 1) // page)
    got_a, got_b, ia, ib = [], [], 0, 0
    for qa, qb in ((30, 5), (1, 40), (66, 2)):
        y = hs.run([("a", qa), ("b", qb)], lambda ctx, cache: part.forward(torch.cat([hd[ia: ia + qa], hbd[ib: ib + qb]]), ctx, cache))
        got_a.append(y[:qa]); got_b.append(y[qa:])
        ia += qa; ib += qb
        hs.cache.check()
    assert rel(torch.cat(got_a), want) < tol and rel(torch.cat(got_b), want_b) < tol
    hs.engine.end(["a", "b"])
    again = hs.run([("c", 47)], lambda ctx, cache: part.forward(hbd, ctx, cache))       # pages that were used
    assert rel(again, want_b) < tol


# ------------------------------------------------------------------ windowed attention with kept first tokens, over steps

def win_weights(W, m, seed, prefix):
    """Queries and keys are brought to root mean square 1, so a larger input changes nothing; what makes a key stand
    out for a query is its direction. Input channel 0 feeds one direction per key/value head into the keys and into the
    queries of the heads that read them: tokens with a large channel 0 find each other."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    shapes = {"q": (H * D, W), "k": (G * D, W), "v": (G * V, W), "o": (W, H * V)}
    w = {prefix + k: rnd(*s, seed=seed + i, scale=0.25) for i, (k, s) in enumerate(shapes.items())}
    a = rnd(G, D, seed=seed + 50, scale=0.5)
    w[prefix + "k"][:, 0] = a.reshape(-1)
    w[prefix + "q"][:, 0] = a.repeat_interleave(H // G, 0).reshape(-1)
    w[prefix + "vmix"] = torch.tensor(0.3 + 0.01 * seed)
    return w


def make_win(W, m, eps, role):
    from rllm_b200.config.llama import RopeScaling
    from rllm_b200.config.purozen import WindowAttentionConfig
    from rllm_b200.parts import RotaryEmbedding, SinkGQAttention
    c = WindowAttentionConfig.from_dict(m, "mixer")
    pos = None
    if c.rot_dims:
        pos = RotaryEmbedding(c.dim, c.rot_base, None if c.rot_factor is None else RopeScaling("linear", c.rot_factor),
                              rot_dim=c.rot_dims)
    return SinkGQAttention(W, c.heads, c.kv_heads, c.dim, c.vdim, position=pos, scale=c.scale, window=c.window, qk_norm=True,
                           qk_norm_weight=False, eps=eps, keep_first=c.keep_first, value_mix=(role, "t"))


def winm(heads, kv_heads, dim, vdim, scale, mask=None, rot=None):
    return Z.att(heads, kv_heads, dim, vdim, scale, None, mask, rot, True)["mixer"]


WINS = [    # scale * dim is about 8: what two aligned unit vectors score
    (winm(4, 2, 40, 24, 0.2, (21, 3), (5000.0, 16, 2.5)), 4),       # a window over several pages, kept tokens inside the first
    (winm(2, 2, 16, 32, 0.5, (16, 16), (100.0, 8, None)), 16),      # window = kept = page
    (winm(6, 1, 24, 40, 0.33, (3, 9), None), 8),                    # a window shorter than a page, more kept tokens than that
    (winm(2, 2, 48, 48, 0.17, None, (10000.0, 8, 8.0)), 8),         # every key seen
    (winm(3, 1, 20, 12, 0.4, (33, 1), (77.0, 6, 1.5)), 16),         # nothing a multiple of 8; one kept token
    (winm(8, 2, 32, 64, 0.25, (17, 33), (500.0, 16, None)), 16),    # kept tokens beyond two pages, heads in steps of 16
    (winm(2, 2, 128, 128, 0.06, (50, 5), (1e6, 64, 4.0)), 16),      # large heads
    (winm(8, 4, 16, 16, 0.5, (1, 2), None), 4),                     # a window of the query alone
    (winm(4, 2, 64, 64, 0.125, (40, 19), (20000.0, 32, 2.0)), 16),  # equal head sizes of 64
    (winm(2, 1, 32, 16, 0.25, (30, 0), (50.0, 32, 3.0)), 8),        # a window and nothing kept; the whole head turns
]


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("m,page", WINS)
def test_window_attention_with_kept_first_tokens_and_mixed_values_over_steps(dtype, m, page):
    """Two layers in one step: the first keeps its values, the second mixes them into its own before they are cached.
    The tokens at the first positions, at the last kept position and the one after it, at page borders, far back, just
    inside and just outside the windows of queries 96 and 70, and those two queries themselves carry a large channel 0:
    their keys win the scores of the marked queries that see them."""
    W, n, eps = 40, 97, 1e-5
    w = {**win_weights(W, m, 3 * m["heads"], "a."), **win_weights(W, m, 7 * m["heads"], "b.")}
    h1, h2 = rnd(n, W, seed=9), rnd(n, W, seed=19)
    mask = m.get("mask") or {"size": 30, "keep_first": 0}
    size, kept = mask["size"], mask["keep_first"]
    special = {0, 1, page - 1, page, 2 * page + 1, 50, max(kept - 1, 0), kept}
    for qpos in (96, 70):
        special |= {max(0, qpos - size), max(0, qpos - size + 1)}
    for p in special | {96, 70}:
        h1[p, 0] += 8.0
        h2[p, 0] += 8.0
    x1, x2 = h1.to(DT[dtype]), h2.to(DT[dtype])
    st, sa = as_stored(w, dtype, prefix=""), stored_as(dtype)
    want1, own = P.window_attention(x1.double(), st, "a.", m, eps, stored=sa)
    want2, _ = P.window_attention(x2.double(), st, "b.", m, eps, v_first=own, stored=sa)
    # the yardstick itself moves with what is tested: the mix, the window's size, the number of kept tokens
    assert rel(P.window_attention(x2.double(), st, "b.", m, eps)[0], want2) > 1e-2
    if m.get("mask"):
        off = dict(m, mask={"size": size + 1, "keep_first": kept})
        assert size + 1 > 96 or rel(P.window_attention(x1.double(), st, "a.", off, eps)[0], want1) > 1e-3
        off = dict(m, mask={"size": size, "keep_first": kept + 1})
        assert rel(P.window_attention(x1.double(), st, "a.", off, eps)[0], want1) > 1e-3
    first, second = make_win(W, m, eps, "first"), make_win(W, m, eps, "mix")
    bind(first, w, dtype, "a.")
    bind(second, w, dtype, "b.")
    spec = first.cache_spec()
    assert spec == second.cache_spec() and spec.window == m.get("mask", {}).get("size") and spec.keep_first == (kept if m.get("mask") else 0)
    d1, d2 = x1.to(DEV), x2.to(DEV)
    want = torch.cat([want1, want2], 1)
    tol = 2e-5 if dtype == "float32" else 2e-2       # a window or a kept token that is one off moves the rows by 4 % and more

    def both(rows1, rows2, ctx, caches):
        return torch.cat([first.forward(rows1, ctx, caches[0]), second.forward(rows2, ctx, caches[1])], 1)

    def step(hs, entries, spans):
        r1 = torch.cat([d1[a:b] for a, b in spans.values()])
        r2 = torch.cat([d2[a:b] for a, b in spans.values()])
        return hs.run(entries, lambda ctx, caches: both(r1, r2, ctx, caches))
    over_schedules(dtype, n, step, lambda: TwoLayers(dtype, [spec, spec], page_size=page, pages=2 + (n + page - 1) // page), want, tol)
    # two requests in one step, unequal portions beside single tokens; then a third on pages that were used
    hb1, hb2 = rnd(47, W, seed=10), rnd(47, W, seed=11)
    hb1[3, 0] += 8.0
    hb1[40, 0] += 8.0
    xb1, xb2 = hb1.to(DT[dtype]), hb2.to(DT[dtype])
    wb1, own_b = P.window_attention(xb1.double(), st, "a.", m, eps, stored=sa)
    wb2, _ = P.window_attention(xb2.double(), st, "b.", m, eps, v_first=own_b, stored=sa)
    want_b = torch.cat([wb1, wb2], 1)
    b1, b2 = xb1.to(DEV), xb2.to(DEV)
    hs = TwoLayers(dtype, [spec, spec], page_size=page, pages=4 + (n + 47 + 2 * page - 1) // page)
    got_a, got_b, ia, ib = [], [], 0, 0
    for qa, qb in ((30, 5), (1, 40), (66, 2)):
        y = hs.run([("a", qa), ("b", qb)], lambda ctx, caches: both(torch.cat([d1[ia: ia + qa], b1[ib: ib + qb]]),
                                                                    torch.cat([d2[ia: ia + qa], b2[ib: ib + qb]]), ctx, caches))
        got_a.append(y[:qa]); got_b.append(y[qa:])
        ia += qa; ib += qb
        hs.cache.check()
    assert rel(torch.cat(got_a), want) < tol and rel(torch.cat(got_b), want_b) < tol
    hs.engine.end(["a", "b"])
    again = hs.run([("c", 47)], lambda ctx, caches: both(b1, b2, ctx, caches))
    assert rel(again, want_b) < tol


@pytest.mark.parametrize("window,kept,sigmoid", [(None, 0, True), (77, 20, False), (300, 130, False), (77, 70, True), (64, 64, False)])
def test_far_kept_and_edge_keys_in_long_contexts_on_both_kernels(window, kept, sigmoid):
    """Contexts of up to 2,048 keys over scattered pages, single query tokens and a portion in one launch: a kept first
    key, the last kept key and the first that is not, one key just inside the window and one just outside are made to
    stand out. Against plain arithmetic on the same keys and values; the tensor-core kernel also with the keys of a
    row tile dealt out to several CTAs."""
    from rllm_b200.kernels import sink
    g = torch.Generator().manual_seed(5)
    nh, nkv, kd, vd, page, n_pages = 8, 2, 64, 48, 16, 130
    lens = [1500, 333, 2048, 1]
    S = len(lens)
    scale = 0.11
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        k = [(torch.randn(n, nkv, kd, generator=g) * 0.5).to(dtype) for n in lens]
        v = [torch.randn(n, nkv, vd, generator=g).to(dtype) for n in lens]
        qlens = [1, 1, 40, 1]
        q = [torch.randn(ql, nh, kd, generator=g).to(dtype) for ql in qlens]
        stand_out = [0, 99] if window is None else [0, max(kept - 1, 0), kept, 1499 - window + 1, 1499 - window]
        for far in stand_out:
            k[0][far] = q[0][0].view(nh, kd)[::4] * 3
        bias = torch.randn(nh, generator=g) * 2 - 3 if sigmoid else None
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
                j = torch.arange(i + 1)
                seen = torch.ones(i + 1, dtype=torch.bool) if window is None else ((i - j < window) | (j < kept))
                sc = torch.einsum("hd,jhd->hj", q[s][r].double(), k[s][: i + 1].double().repeat_interleave(nh // nkv, 1)) * scale
                if sigmoid:
                    p = torch.sigmoid(sc + bias.double()[:, None]) * seen
                else:
                    p = torch.softmax(sc.masked_fill(~seen, float("-inf")), 1)
                want.append(torch.einsum("hj,jhv->hv", p, v[s][: i + 1].double().repeat_interleave(nh // nkv, 1)).reshape(-1))
        want = torch.stack(want)
        pos = torch.cat([torch.arange(n - ql, n) for n, ql in zip(lens, qlens)]).int().to(DEV)
        seq = torch.cat([torch.full((ql,), i) for i, ql in enumerate(qlens)]).int().to(DEV)
        qd = torch.cat([x.reshape(-1, nh * kd) for x in q]).to(DEV)
        bd = None if bias is None else bias.to(DEV)
        got = sink.sink_attention_simt(qd, kc.to(DEV), vc.to(DEV), seq, pos, bt.to(DEV), nh, scale, window, None, bd, None, kept, sigmoid)
        assert rel(got, want) < tol, dtype
        if dtype == torch.bfloat16:
            assert sink.mma_supported(dtype, kd, vd, page)
            cu = torch.tensor([0] + list(itertools.accumulate(qlens)), dtype=torch.int32, device=DEV)
            for splits in (1, 3):
                got = sink.sink_attention_mma(qd, kc.to(DEV), vc.to(DEV), seq, pos, bt.to(DEV), cu, S, max(qlens), nh, scale, window,
                                              None, bd, None, splits, 2048, kept, sigmoid)
                assert rel(got, want) < tol, splits
            one = [0, 1, 42]                   # single tokens alone: the four warps of a CTA share a tile's keys
            cu1 = torch.arange(4, dtype=torch.int32, device=DEV)
            for splits in (1, 4):
                got1 = sink.sink_attention_mma(qd[one], kc.to(DEV), vc.to(DEV), seq[one], pos[one], bt[[0, 1, 3]].to(DEV), cu1, 3, 1, nh,
                                               scale, window, None, bd, None, splits, 2048, kept, sigmoid)
                assert rel(got1, want[one]) < tol, splits


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("window,kept,sigmoid", [(None, 0, True), (300, 70, False), (128, 128, False), (100, 3, False), (257, 200, True),
                                                  (64, 1, False)])
def test_long_portions_with_equal_head_sizes_on_tcgen05(hd, window, kept, sigmoid):
    """Equal key and value sizes of 64 or 128: long portions take the tcgen05 kernel, which walks the kept keys' tiles
    before the window's and has the sigmoid branch. Three portions beside each other (one with all its keys in the step,
    one behind 800 cached keys, one short), a kept key, the last kept key and the first that is not, and keys just
    inside and just outside the last query's window made to stand out; against the float kernel on the same cache."""
    from rllm_b200.kernels import sink, sm100
    g = torch.Generator().manual_seed(hd + (window or 0))
    nh, nkv, page, n_pages = 8, 2, 16, 100
    lens, qlens = [1500, 700, 1024], [700, 700, 130]
    S = len(lens)
    kc = (torch.randn(n_pages * S, nkv, page, hd, generator=g) * 0.5).bfloat16().to(DEV)
    vc = torch.randn(n_pages * S, nkv, page, hd, generator=g).bfloat16().to(DEV)
    bt = torch.randperm(n_pages * S, generator=g).int().view(S, n_pages).contiguous().to(DEV)
    bias = (torch.randn(nh, generator=g) * 2 - 3).to(DEV) if sigmoid else None
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    T = sum(qlens)
    q = torch.randn(T, nh * hd, generator=g).bfloat16().to(DEV)
    last = q[qlens[0] - 1].view(nh, hd)[::4]                   # the last query of the first portion, one head per kv head
    marks = [0, 99] if window is None else [0, max(kept - 1, 0), kept, 1499 - window + 1, 1499 - window]
    for far in marks:
        kc[bt[0, far // page].item(), :, far % page] = last * 2
    cu = torch.tensor([0, 700, 1400, 1530], dtype=torch.int32, device=DEV)
    pos = torch.cat([torch.arange(n - ql, n) for n, ql in zip(lens, qlens)]).int().to(DEV)
    seq = torch.cat([torch.full((ql,), i) for i, ql in enumerate(qlens)]).int().to(DEV)
    want = sink.sink_attention_simt(q, kc, vc, seq, pos, bt, nh, 0.11, window, None, bias, None, kept, sigmoid)
    got = sm100.attention_prefill_tc(q, kc, vc, cu, kv, bt, max(qlens), nh, 0.11, window, sinks=bias, keep_first=kept, sigmoid=sigmoid)
    sm100.check_error(DEV)
    assert rel(got, want) < 2e-2
    got = sink.sink_attention_mma(q, kc, vc, seq, pos, bt, cu, S, max(qlens), nh, 0.11, window, None, bias, None, 1, 1500, kept, sigmoid)
    assert rel(got, want) < 2e-2
    # the float kernel itself against plain arithmetic, for the marked query
    i, r = 1499, qlens[0] - 1
    j = torch.arange(i + 1)
    seen = torch.ones(i + 1, dtype=torch.bool) if window is None else ((i - j < window) | (j < kept))
    pages = bt[0].cpu()[j // page].long()
    K = kc.cpu()[pages, :, j % page].double().repeat_interleave(nh // nkv, 1)          # [keys, heads, hd]
    V = vc.cpu()[pages, :, j % page].double().repeat_interleave(nh // nkv, 1)
    sc = torch.einsum("hd,jhd->hj", q[r].cpu().double().view(nh, hd), K) * 0.11
    w_ = torch.sigmoid(sc + bias.cpu().double()[:, None]) * seen if sigmoid else torch.softmax(sc.masked_fill(~seen, float("-inf")), 1)
    assert rel(want[r].cpu().double().view(nh, hd), torch.einsum("hj,jhd->hd", w_, V)) < 2e-2


def test_the_engine_sends_long_portions_of_equal_head_sizes_to_tcgen05():
    """A windowed attention layer with kept first tokens and a sigmoid attention layer, heads of 64 / 64: a portion of
    600 tokens behind 200 cached ones runs on the tcgen05 kernel, single tokens on the `mma.sync` kernel; both agree
    with the plain implementation."""
    from rllm_b200.kernels import sink, sm100
    W, n, eps, dtype = 64, 860, 1e-5, "bfloat16"
    m = winm(4, 2, 64, 64, 0.125, (150, 70), (20000.0, 32, 2.0))
    w = {**win_weights(W, m, 5, "a."), **win_weights(W, m, 9, "b.")}
    h1, h2 = rnd(n, W, seed=9), rnd(n, W, seed=19)
    for p in (0, 69, 70, 799 - 150, 799 - 149, 799, 859 - 150, 859 - 149, 859):
        h1[p, 0] += 8.0
        h2[p, 0] += 8.0
    x1, x2 = h1.to(DT[dtype]), h2.to(DT[dtype])
    st, sa = as_stored(w, dtype, prefix=""), stored_as(dtype)
    want1, own = P.window_attention(x1.double(), st, "a.", m, eps, stored=sa)
    want2, _ = P.window_attention(x2.double(), st, "b.", m, eps, v_first=own, stored=sa)
    first, second = make_win(W, m, eps, "first"), make_win(W, m, eps, "mix")
    bind(first, w, dtype, "a.")
    bind(second, w, dtype, "b.")
    calls = {"tc": 0, "mma": 0}
    real_tc, real_mma = sm100.attention_prefill_tc, sink.sink_attention_mma
    sm100.attention_prefill_tc = lambda *a, **k: (calls.__setitem__("tc", calls["tc"] + 1), real_tc(*a, **k))[1]
    sink.sink_attention_mma = lambda *a, **k: (calls.__setitem__("mma", calls["mma"] + 1), real_mma(*a, **k))[1]
    try:
        hs = TwoLayers(dtype, [first.cache_spec()] * 2, page_size=16, pages=60)
        d1, d2 = x1.to(DEV), x2.to(DEV)
        got, i = [], 0
        for qn in [200, 600] + [1] * 60:
            got.append(hs.run([("a", qn)], lambda ctx, caches: torch.cat(
                [first.forward(d1[i: i + qn], ctx, caches[0]), second.forward(d2[i: i + qn], ctx, caches[1])], 1)))
            i += qn
        sm100.check_error(DEV)
    finally:
        sm100.attention_prefill_tc, sink.sink_attention_mma = real_tc, real_mma
    assert calls["tc"] == 2 and calls["mma"] == 2 * 61          # the portion of 200 has fewer keys than the tcgen05 kernel asks for
    assert rel(torch.cat(got), torch.cat([want1, want2], 1)) < 2e-2


# ------------------------------------------------------------------ attention over latents without positions, over steps

def lat_weights(W, m, seed):
    H, d, vd, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    shapes = {"q": (H * d, W), "dkv": (r, W), "dkv.norm": (r,), "uk": (H * d, r), "uv": (H * vd, r), "o": (W, H * vd)}
    w = {"x." + k: rnd(*s, seed=seed + i, scale=0.3) for i, (k, s) in enumerate(shapes.items())}
    w["x.dkv.norm"] = w["x.dkv.norm"] + 1
    return w


LATS = [(Z.lat(3, 16, 24, 40, 0.25, None)["mixer"], 4), (Z.lat(5, 8, 8, 24, 0.35, None)["mixer"], 8),
        (Z.lat(1, 12, 20, 16, 0.3, None)["mixer"], 16), (Z.lat(4, 32, 16, 128, 0.2, None)["mixer"], 16),
        (Z.lat(8, 16, 32, 64, 0.3, None)["mixer"], 16)]


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("m,page", LATS)
def test_latent_attention_without_positions_or_gate_over_steps(dtype, m, page):
    from rllm_b200.parts import LatentAttention
    W, n, eps = 40, 97, 1e-6
    w = lat_weights(W, m, seed=m["heads"])
    h = rnd(n, W, seed=9)
    for p in {0, 1, page - 1, page, 2 * page + 1, 50}:
        h[p] *= 5.0
    x = h.to(DT[dtype])
    want = P.plain_latent_attention(x.double(), as_stored(w, dtype), "", m, eps, stored=stored_as(dtype))
    part = LatentAttention(W, m["heads"], m["dim"], 0, m["vdim"], m["kv_rank"], m["scale"], None, eps=eps, gate=False)
    assert part.cache_spec().width == m["kv_rank"] and "x.g" not in {part.prefix + s.name for p_ in part.params() for s in p_.sources}
    bind(part, w, dtype, "x.")
    hd = x.to(DEV)
    tol = 2e-5 if dtype == "float32" else 5e-2

    def step(hs, entries, spans):
        rows = torch.cat([hd[a:b] for a, b in spans.values()])
        return hs.run(entries, lambda ctx, cache: part.forward(rows, ctx, cache))
    over_schedules(dtype, n, step, lambda: Harness(dtype, [part.cache_spec()], page_size=page, pages=2 + (n + page - 1) // page), want, tol)


# ------------------------------------------------------------------ whole models

def requests_for(name, lens=(9, 61, 23, 150, 37, 2)):
    vocab = Z.TINY[name][0]["vocab"]
    return {f"r{i}": Z.random_prompt(n, vocab, 100 * len(name) + ord(name[1]) + i) for i, n in enumerate(lens)}


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("purozen")
    return {n: Z.make_model_dir(root, n) for n in Z.TINY}


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
    return load_engine(dirs[name], dtype=dtype, page_size=Z.TINY[name][3],
                       max_tokens=replay.max_live_tokens(steps, reqs), max_requests=max_requests)


@pytest.mark.parametrize("name", list(Z.TINY))
def test_residual_stream_after_every_layer(dirs, name):
    """In float32, layer by layer: the first layer that differs names the mechanism."""
    from rllm_b200.engine import Entry, load_engine
    cfg, w = P.read_model_dir(dirs[name])
    toks = Z.random_prompt(45, cfg["vocab"], 9)
    _, kept = P.forward(cfg, w, toks, keep_layers=True)
    eng = load_engine(dirs[name], dtype="float32", page_size=Z.TINY[name][3], max_tokens=64, max_requests=1)
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
@pytest.mark.parametrize("name", list(Z.TINY))
def test_family_matches_plain(dirs, plain, name, dtype, family):
    """The pool holds just what the live requests need and there are three state slots for six requests: pages and
    slots are used again."""
    reqs = requests_for(name)
    steps = FAMILIES[family](reqs)
    eng = engine_for(dirs, name, dtype, steps, reqs)
    got = replay.run_in_process(eng, steps)
    eng.check()
    if dtype == "float32":
        check(got, plain[name], 3e-5, f"{name} float32 {family}")
    else:
        check(got, plain[name], 6e-2, f"{name} bfloat16 {family}", allow=0.02)


@pytest.mark.parametrize("name", list(Z.TINY))
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
            assert worst <= 4e-6, f"{name} {family}: differs from whole prompts by {worst}"


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 6e-2)])
def test_long_decoding_through_graphs(dirs, dtype, tol):
    """Two requests decoded side by side for 120 steps from prompts of 3 and 30 tokens: the windows pass over decoded
    tokens, pages are given back on the way while those of the kept first tokens stay, the recurrences' states are
    carried through replayed graphs."""
    from rllm_b200.engine import Entry, load_engine
    name = "PA"
    cfg, w = P.read_model_dir(dirs[name])
    toks = {"x": Z.random_prompt(123, cfg["vocab"], 5), "y": Z.random_prompt(150, cfg["vocab"], 6)}
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
    held = eng.cache.live["y"].pages
    windowed = [g for g, grp in enumerate(eng.cache.groups) if getattr(grp.spec, "window", None)]
    assert windowed and all(held[g][0] >= 0 and -1 in held[g] for g in windowed)     # the first page stays, later ones went back
    check(got, {(k, i): want[k][i] for (k, i) in got}, tol, f"long decoding {dtype}", allow=0.0 if dtype == "float32" else 0.02)


@pytest.mark.parametrize("name", ["PB", "PC", "PD"])
def test_greedy_generation_through_the_entry_point(dirs, name):
    """LLM.generate (scheduler, sampler, run-ahead decoding) against greedy decoding with the plain model."""
    from rllm_b200.api import LLM
    from rllm_b200.sampling import SamplingParams
    cfg, w = P.read_model_dir(dirs[name])
    prompts = [Z.random_prompt(n, cfg["vocab"], 70 + n) for n in (4, 19, 33)]
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
    llm = LLM(dirs[name], dtype="float32", page_size=Z.TINY[name][3], num_pages=40, max_active=2, max_chunk=16)
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for g, w_ in zip(got, want):
        assert g[: len(w_)] == w_
    llm.engine.cache.check()


def test_ten_requests_decode_in_a_padded_graph(dirs):
    """Ten requests decode side by side: their graph has more rows than requests; the stand-in rows have no state
    slot, pages or wanted logits, and must neither disturb the others nor touch a state."""
    from rllm_b200.engine import Entry, load_engine
    name = "PA"
    cfg, w = P.read_model_dir(dirs[name])
    toks = {i: Z.random_prompt(5 + 3 * i + 9, cfg["vocab"], 300 + i) for i in range(10)}
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
    name = "PF"
    cfg, w = P.read_model_dir(dirs[name])
    prompt = Z.random_prompt(11, cfg["vocab"], 3)
    toks = prompt + P.greedy(cfg, w, prompt, 5)
    r = subprocess.run([sys.executable, os.path.join(replay.ROOT, "bin", "rllm"), "run", "--model", dirs[name],
                        "--prompt-ids", " ".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0",
                        "--dtype", "float32", "--kv-pages", "32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [int(x) for x in r.stdout.split()] == toks[len(prompt):]


@pytest.mark.parametrize("name,dtype", [("PC", "float32"), ("PE", "bfloat16")])
def test_trace_program_runs_the_design(dirs, plain, tmp_path, name, dtype):
    reqs = requests_for(name)
    steps = replay.mixed(reqs, max_live=4)
    got = replay.run_program(dirs[name], dtype, steps, str(tmp_path / "out"), replay.max_live_tokens(steps, reqs),
                             Z.TINY[name][0]["vocab"], extra_args=["--page-size", "16"])
    if dtype == "float32":
        check(got, plain[name], 3e-5, "trace program")
    else:
        check(got, plain[name], 6e-2, "trace program bfloat16", allow=0.02)
