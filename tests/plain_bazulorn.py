"""A plain, slow Bazulorn on the CPU: the tests' yardstick for the package's Bazulorn parts.

One function per mechanism, written from the design's equations with float64 torch tensors on the CPU and
python loops over tokens where the design is recurrent. It shares no code with `rllm_b200`: its only inputs
are the raw `config.json` dictionary and the checkpoint's tensors by name.

Notation: n is a sublayer's input [T, width] (the layer's one norm applied to the stream); positions count
from 0; `eps` is `norm.eps`; a weight W is stored [out, in] and applied as n @ W.T.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

DT = torch.float64
SWISH_ALPHA = 1.702
UNIT_EPS = 1e-6


# ------------------------------------------------------------------ files

def read_safetensors(path):
    """name -> float64 tensor (integer tables stay integers)."""
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16, "F64": torch.float64}
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        lo, hi = ent["data_offsets"]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=kinds[ent["dtype"]]).reshape(ent["shape"])
        out[name] = t.to(DT) if t.is_floating_point() else t.clone()
    return out


def read_model_dir(d):
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(d, "model.safetensors"))


# ------------------------------------------------------------------ small pieces

def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension (w None: no weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 40, x, torch.log1p(torch.exp(torch.clamp(x, max=40))))


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def short_conv(x, w, b=None):
    """Causal convolution over time per channel: x [T, C], w [C, taps] whose last column meets the current
    token; inputs before the start are zero."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros(T, C, dtype=DT)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1 - j)
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y if b is None else y + b


def pair_rows(ids, bg):
    """Row of the pair table for each token of one sequence."""
    rows = [bg["buckets"]]
    for prev, cur in zip(ids[:-1], ids[1:]):
        rows.append((prev * bg["mul_prev"] + cur * bg["mul_cur"]) % bg["buckets"])
    return rows


def embed(cfg, w, ids):
    x = w["embed"][torch.tensor(ids)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + w["bigram"][torch.tensor(pair_rows(list(ids), bg))]
    return rms_norm(x, w["embed.norm"], cfg["norm"]["eps"])


# ------------------------------------------------------------------ mixers

def talk_attention(n, w, p, m, eps, sink=0.0):
    """Grouped-query attention without rotation: biased projections, values normed per head, a sliding
    window, a sink in the softmax's denominator, the heads' weights mixed by `talk`."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = n.shape[0]
    q = (n @ w[p + "q"].T + w[p + "q.b"]).view(T, H, D)
    k = (n @ w[p + "k"].T + w[p + "k.b"]).view(T, G, D)
    v = rms_norm((n @ w[p + "v"].T + w[p + "v.b"]).view(T, G, V), None, eps)
    size = (m.get("mask") or {}).get("size")
    probs = torch.zeros(H, T, T, dtype=DT)
    for h in range(H):
        c = h // (H // G)
        for i in range(T):
            lo = 0 if size is None else max(0, i - size + 1)
            s = (k[lo: i + 1, c] @ q[i, h]) * m["scale"]
            e = torch.exp(s)
            probs[h, i, lo: i + 1] = e / (math.exp(sink) + e.sum()) if sink is not None else e / e.sum()
    mixed = torch.einsum("hg,gij->hij", w[p + "talk"], probs)
    o = torch.stack([mixed[h] @ v[:, h // (H // G)] for h in range(H)], 1).reshape(T, H * V)
    return o @ w[p + "o"].T


def exact(x):
    return x


def state_space(n, w, p, m, eps, stored=exact):
    """State-space recurrence with a convolution over x, B and C, a gate before a norm in parts. `stored`: what
    a run that keeps its activations in fewer bits does to the input projection's output and to the input of the
    output projection (the tests of such a run pass a rounding; the design itself has none)."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    I, T = H * P, n.shape[0]
    u = stored(n @ w[p + "in"].T)
    z, xbc, dt = u[:, :I], u[:, I: 2 * I + 2 * G * N], u[:, 2 * I + 2 * G * N:]
    xbc = silu(short_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x, B, C = xbc[:, :I].view(T, H, P), xbc[:, I: I + G * N].view(T, G, N), xbc[:, I + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    a = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    S = torch.zeros(H, N, P, dtype=DT)
    y = torch.zeros(T, H, P, dtype=DT)
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = a[t, h] * S[h] + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g] + w[p + "D"][h] * x[t, h]
    y = y.reshape(T, I) * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.view(T, parts, I // parts), None, eps).reshape(T, I) * w[p + "norm"]
    return stored(y) @ w[p + "o"].T


def side_by_side(n, w, p, m, eps):
    l = talk_attention(n, w, p + "left.", m["left"], eps)
    r = state_space(n, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(l, w[p + "left.out"], eps) + rms_norm(r, w[p + "right.out"], eps))


def delta_rule(n, w, p, m, eps, stored=exact):
    """Gated delta rule with a decay per head and key channel. `stored` as in `state_space`: applied to the outputs
    of the projections from the layer's input that are not gates of the recurrence, and to W_o's input."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = n.shape[0]
    q = silu(short_conv(stored(n @ w[p + "q"].T), w[p + "q.conv"])).view(T, G, D)
    k = silu(short_conv(stored(n @ w[p + "k"].T), w[p + "k.conv"])).view(T, G, D)
    v = silu(short_conv(stored(n @ w[p + "v"].T), w[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + UNIT_EPS) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + UNIT_EPS)
    beta = torch.sigmoid(n @ w[p + "b"].T)
    step = softplus(stored(n @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, D)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * step)
    S = torch.zeros(H, D, V, dtype=DT)
    o = torch.zeros(T, H, V, dtype=DT)
    for t in range(T):
        for h in range(H):
            c = h // (H // G)
            S[h] = g[t, h][:, None] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, c])
            S[h] = S[h] + torch.outer(k[t, c], u)
            o[t, h] = S[h].T @ q[t, c]
    o = rms_norm(o, w[p + "norm"], eps)
    gate = torch.sigmoid(stored(n @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, V)
    return stored((o * gate).reshape(T, H * V)) @ w[p + "o"].T


# ------------------------------------------------------------------ feed-forwards

def clamped_expert(n, w, p, limit):
    g = torch.clamp(n @ w[p + "gate"].T, max=limit)
    u = torch.clamp(n @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(SWISH_ALPHA * g) * (u + 1)) @ w[p + "down"].T


def route(z, top):
    """(chosen experts [T, top], weights [T, top]): the largest logits, softmax over the chosen ones only."""
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def feed_forward(n, w, p, mlp):
    if mlp["kind"] == "dense":
        return (gelu_tanh(n @ w[p + "gate"].T) * (n @ w[p + "up"].T)) @ w[p + "down"].T
    idx, wt = route(n @ w[p + "router"].T + w[p + "router.b"], mlp["router"]["top"])
    out = torch.zeros_like(n)
    for t in range(n.shape[0]):
        for s in range(idx.shape[1]):
            out[t] += wt[t, s] * clamped_expert(n[t: t + 1], w, f"{p}e{int(idx[t, s])}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(n, w, p + "shared.", mlp["shared"]["limit"])
    return out


# ------------------------------------------------------------------ the model

MIXERS = {"parallel": side_by_side, "channel_delta": delta_rule}


def forward(cfg, w, ids, keep_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = embed(cfg, w, ids)
    kept = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = rms_norm(x, w[p + "norm1"], eps)
        y = MIXERS[L["type"]](n, w, p + "mix.", L["mixer"], eps)
        if L.get("mlp"):
            y = y + feed_forward(n, w, p + "mlp.", L["mlp"])
        x = x + y
        kept.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, kept) if keep_layers else logits


def greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
