"""A plain, slow Purozen on the CPU: the tests' yardstick for the package's Purozen parts.

One function per mechanism, written from the design's equations with float64 torch tensors on the CPU and
python loops over tokens where the design is recurrent. It shares no code with `rllm_b200`: its only inputs
are the raw `config.json` dictionary and the checkpoint's tensors by name.

Notation: n is a sublayer's input [T, width] (a layer's norm applied to the stream); positions count from 0;
`eps` is `norm.eps`; a weight W is stored [out, in] and applied as n @ W.T; `p` is a mixer's tensor prefix.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

DT = torch.float64


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

def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """The layers' norm: the stored weight is the factor minus one."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def exact(x):
    return x


def causal(T):
    i = torch.arange(T)
    return i[None, :] <= i[:, None]                 # [query, key]


def grouped(x, heads):
    """[T, kv_heads, d] -> [T, heads, d]: query head h reads key/value head h // (heads / kv_heads)."""
    return x.repeat_interleave(heads // x.shape[1], dim=1)


# ------------------------------------------------------------------ mixers

def sigmoid_attention(n, w, p, m, bias=True, stored=exact):
    """Causal grouped-query attention without positions and without a softmax: key j's weight for query i is
    sigmoid(scale q_i . k_j + b_h) for j <= i and 0 otherwise; the weights are not normalised."""
    T, H, G, d, vd = n.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = stored(n @ w[p + "q"].T).view(T, H, d)
    k = grouped(stored(n @ w[p + "k"].T).view(T, G, d), H)
    v = grouped(stored(n @ w[p + "v"].T).view(T, G, vd), H)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    if bias:
        s = s + w[p + "pb"][:, None, None]
    a = torch.sigmoid(s) * causal(T)
    o = torch.einsum("hij,jhv->ihv", a, v).reshape(T, H * vd)
    return stored(o) @ w[p + "o"].T


def min_gru(n, w, p, m, stored=exact, state=None):
    """z = sigmoid(W_z n + b_z); u = W_x n + b_x; c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0);
    S_t = (1 - z_t) S_(t-1) + z_t c_t from S = 0 (or `state`); out = W_o (S_t * silu(W_g n))."""
    T, R = n.shape[0], m["width"]
    z = torch.sigmoid(n @ w[p + "z"].T + w[p + "z.b"])
    u = n @ w[p + "x"].T + w[p + "x.b"]
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = n @ w[p + "g"].T
    S = torch.zeros(R, dtype=DT) if state is None else state.clone()
    rows = []
    for t in range(T):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        rows.append(S * (g[t] * torch.sigmoid(g[t])))
    return stored(torch.stack(rows)) @ w[p + "o"].T


def side_by_side(n, w, p, m, stored=exact):
    return m["left_scale"] * sigmoid_attention(n, w, p + "left.", m["left"], stored=stored) + \
        m["right_scale"] * min_gru(n, w, p + "right.", m["right"], stored=stored)


def rotate_half_layout(x, rot, positions):
    """The first rot.dims numbers of each head: number i pairs with number i + dims/2; the pair (a, b) at position t
    turns by the angle t * f_i, f_i = base^(-2i/dims) / factor. The rest of the head passes."""
    dims = rot["dims"]
    half = dims // 2
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(half)], dtype=DT)
    if rot.get("scaling") is not None:
        f = f / rot["scaling"]["factor"]
    ang = positions.to(DT)[:, None] * f[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def window_mask(T, mask):
    """[query, key]: causal; with a mask, key j is seen by query i when i - j < size or j < keep_first."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if mask is not None:
        ok = ok & ((i - j < mask["size"]) | (j < mask.get("keep_first", 0)))
    return ok


def window_attention(n, w, p, m, eps, v_first=None, stored=exact):
    """Grouped-query attention with a rotation of part of each head, queries and keys brought to root mean square 1
    after it, a sliding window that keeps the first tokens, a softmax over the visible keys, and the values
    optionally mixed with another layer's: v <- (1 - lam) v + lam v_first. Returns (output, this layer's unmixed
    values)."""
    T, H, G, d, vd = n.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = stored(n @ w[p + "q"].T).view(T, H, d)
    k = stored(n @ w[p + "k"].T).view(T, G, d)
    v = stored(n @ w[p + "v"].T).view(T, G, vd)
    own = v
    if m.get("rot") is not None and m["rot"]["dims"] > 0:
        pos = torch.arange(T)
        q, k = rotate_half_layout(q, m["rot"], pos), rotate_half_layout(k, m["rot"], pos)
    q, k = stored(unit_rms(q, eps)), stored(unit_rms(k, eps))
    if v_first is not None:
        lam = w[p + "vmix"]
        v = stored((1.0 - lam) * v + lam * v_first)
    s = torch.einsum("ihd,jhd->hij", q, grouped(k, H)) * m["scale"]
    s = s.masked_fill(~window_mask(T, m.get("mask")), float("-inf"))
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhv->ihv", a, grouped(v, H)).reshape(T, H * vd)
    return stored(o) @ w[p + "o"].T, own


def plain_latent_attention(n, w, p, m, eps, stored=exact):
    """c = rms_norm(W_dkv n) * g (the cached latent); per head k = W_uk c, v = W_uv c; causal softmax attention without
    positions."""
    T, H, d, vd = n.shape[0], m["heads"], m["dim"], m["vdim"]
    q = stored(n @ w[p + "q"].T).view(T, H, d)
    c = stored(unit_rms(stored(n @ w[p + "dkv"].T), eps) * w[p + "dkv.norm"])
    k = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, vd)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    s = s.masked_fill(~causal(T), float("-inf"))
    o = torch.einsum("hij,jhv->ihv", torch.softmax(s, dim=-1), v).reshape(T, H * vd)
    return stored(o) @ w[p + "o"].T


def feed_forward(n, w, p):
    return gelu_tanh(n @ w[p + "up"].T) @ w[p + "down"].T


def gate(n, w, name):
    return torch.sigmoid(n @ w[name].T + w[name + ".b"])


# ------------------------------------------------------------------ the model

def forward(cfg, w, ids, keep_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer with `keep_layers`)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(ids)]
    v_first, kept = None, []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = norm_around_zero(x, w[p + "norm1"], eps)
        if L["type"] == "parallel":
            y = side_by_side(n, w, p + "mix.", L["mixer"])
        elif L["type"] == "attention":
            mixes = bool(L["mixer"].get("v_mix"))
            y, own = window_attention(n, w, p + "mix.", L["mixer"], eps, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = own
        elif L["type"] == "latent_attention":
            y = plain_latent_attention(n, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + gate(n, w, p + "rg1") * y
        if L["mlp"] is not None:
            n = norm_around_zero(x, w[p + "norm2"], eps)
            x = x + gate(n, w, p + "rg2") * feed_forward(n, w, p + "mlp.")
        kept.append(x.clone())
    logits = norm_around_zero(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, kept) if keep_layers else logits


def greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
