"""The tests' own small Bazulorn configurations and model folders. They differ from each other in every size
and option: with and without the pair table, attention with a window (longer than a page, shorter than one, of
the query alone) and without, as many key/value heads as query heads and fewer, key and value sizes that differ,
state-space heads in one group and several, the norm after the gate in one part and several, convolutions of one
to five taps, delta-rule heads that share queries and keys and that do not, key channels beyond a warp's lanes,
dense, routed (with and without the expert every token uses, one expert a token) and absent feed-forwards, and
models without any attention (no pages) or without any delta rule."""
import os

import torch


def talk(heads, kv_heads, dim, vdim, scale, window):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def ssm(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def par(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank, mlp):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def bigram(buckets, mul_prev, mul_cur):
    return {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}


BA = {  # both mixers, a window over several pages, heads that share keys; dense, routed and shared feed-forwards
    "architecture": "Bazulorn", "vocab": 160, "width": 96, "embedding": bigram(211, 31, 5), "norm": {"eps": 1e-5},
    "layers": [
        par(talk(4, 2, 24, 16, 0.2, 21), ssm(4, 12, 20, 2, 2, 3), dense(72)),
        delta(4, 2, 20, 24, 4, 8, 12, moe(24, 1.25, 6, 2, (40, 0.75))),
        par(talk(4, 2, 24, 16, 0.2, 21), ssm(4, 12, 20, 2, 2, 3), moe(16, 2.5, 5, 3)),
    ],
}
BB = {  # no pair table; every key seen; one group, one norm part, two taps; one expert a token; a layer without feed-forward
    "architecture": "Bazulorn", "vocab": 200, "width": 64, "norm": {"eps": 3e-6},
    "layers": [
        delta(1, 1, 64, 72, 2, 16, 4, moe(32, 0.5, 4, 1)),
        par(talk(3, 3, 8, 40, 0.35, None), ssm(3, 24, 8, 1, 1, 2), None),
        delta(6, 3, 8, 8, 5, 4, 20, dense(40)),
    ],
}
BC = {  # windows shorter than a page and of the query alone; key channels beyond a warp's lanes; one tap
    "architecture": "Bazulorn", "vocab": 120, "width": 72, "embedding": bigram(64, 3, 1), "norm": {"eps": 1e-6},
    "layers": [
        par(talk(6, 1, 12, 20, 0.3, 7), ssm(2, 36, 44, 2, 4, 4), moe(20, 1.0, 9, 2, (12, 3.0))),
        par(talk(2, 2, 36, 12, 0.15, 1), ssm(6, 8, 12, 3, 1, 1), dense(48)),
        delta(2, 2, 130, 20, 1, 8, 8, None),
    ],
}
BD = {  # recurrent layers only: no pages at all
    "architecture": "Bazulorn", "vocab": 90, "width": 40, "embedding": bigram(17, 1, 2), "norm": {"eps": 1e-5},
    "layers": [
        delta(2, 1, 12, 20, 3, 4, 6, None),
        delta(5, 5, 8, 8, 2, 12, 4, moe(16, 2.0, 3, 3, (8, 1.0))),
    ],
}
BE = {  # nothing a multiple of 8; no delta rule; more buckets than tokens squared
    "architecture": "Bazulorn", "vocab": 77, "width": 100, "embedding": bigram(7919, 77, 1), "norm": {"eps": 1e-6},
    "layers": [
        par(talk(3, 1, 10, 14, 0.25, 19), ssm(5, 6, 14, 5, 5, 3), moe(12, 1.5, 7, 2)),
        par(talk(2, 2, 14, 10, 0.3, None), ssm(1, 30, 6, 1, 3, 2), moe(20, 0.8, 7, 3, (28, 1.2))),
    ],
}
# name -> (config, seed, weight std, norm std, page size)
TINY = {"BA": (BA, 21, 0.09, 0.2, 4), "BB": (BB, 22, 0.12, 0.1, 8), "BC": (BC, 23, 0.1, 0.3, 16),
        "BD": (BD, 24, 0.15, 0.2, 16), "BE": (BE, 25, 0.1, 0.2, 8)}


def make_model_dir(root, name, dtype=torch.bfloat16):
    from rllm_b200.weights import write_random_model
    cfg, seed, std, norm_std, _ = TINY[name]
    d = os.path.join(str(root), f"tiny_{name}_{str(dtype).split('.')[-1]}")
    if not os.path.isdir(d):
        write_random_model(cfg, seed, d, std=std, norm_std=norm_std, dtype=dtype)
    return d


def random_prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
