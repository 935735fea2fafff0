"""The tests' own small Purozen configurations and model folders. They differ from each other in every size and
option: heads that share keys and heads that do not, key and value sizes that differ (and that are equal), windows
over several pages, shorter than a page, of the query alone and absent; kept first tokens fewer than a page, more
than a page, more than the window and none; a rotation of a part of a head, of all of it and none, with and without
the factor on its frequencies; values mixed over two and three layers, and not at all; recurrences narrower than a
warp and wider than a block; scales of 1 and other numbers; layers without a feed-forward; models without any window
(no page is ever given back), without any attention of a kind, and of one layer."""
import os

import torch


def sig(heads, kv_heads, dim, vdim, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}


def par(left, width, left_scale, right_scale, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": width}, "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": dense(ff)}


def att(heads, kv_heads, dim, vdim, scale, ff, mask=None, rot=None, v_mix=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if rot[2] is not None:
            m["rot"]["scaling"] = {"factor": rot[2]}
    if v_mix is not None:
        m["v_mix"] = v_mix
    return {"type": "attention", "mixer": m, "mlp": dense(ff)}


def lat(heads, dim, vdim, kv_rank, scale, ff):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale},
            "mlp": dense(ff)}


def dense(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


PA = {  # every kind; a window over several pages with kept tokens inside the first page; values mixed over two layers
    "architecture": "Purozen", "vocab": 150, "width": 80, "norm": {"eps": 1e-5},
    "layers": [
        par(sig(4, 2, 24, 40, 0.2), 72, 0.7, 1.3, 96),
        att(4, 2, 40, 24, 0.15, 64, mask=(21, 3), rot=(5000.0, 16, 2.5), v_mix=True),
        lat(3, 16, 24, 40, 0.25, 48),
        att(6, 2, 24, 24, 0.2, None, mask=(9, 6), rot=(300.0, 24, None), v_mix=True),
        par(sig(2, 2, 16, 16, 0.3), 200, 1.0, 0.4, 56),
    ],
}
PB = {  # no window anywhere: nothing is given back; no rotation; as many key/value heads as heads; a layer without feed-forward
    "architecture": "Purozen", "vocab": 210, "width": 64, "norm": {"eps": 3e-6},
    "layers": [
        att(3, 3, 16, 32, 0.25, 40),
        lat(5, 8, 8, 24, 0.35, None),
        att(2, 1, 32, 8, 0.18, 72, rot=(10000.0, 8, 8.0), v_mix=False),
    ],
}
PC = {  # nothing a multiple of 8; a window of the query alone beside kept tokens; more kept tokens than the window; three layers mix
    "architecture": "Purozen", "vocab": 99, "width": 52, "norm": {"eps": 1e-6},
    "layers": [
        att(3, 1, 10, 14, 0.3, 30, mask=(1, 3), rot=(77.0, 6, 1.5), v_mix=True),
        par(sig(6, 3, 12, 6, 0.22), 37, 0.25, 2.0, 44),
        att(2, 1, 14, 14, 0.28, 20, mask=(5, 11), rot=(1000.0, 14, 3.0), v_mix=True),
        att(1, 1, 22, 14, 0.2, 36, mask=(30, 0), v_mix=True),
    ],
}
PD = {  # parallel layers only: pages that are never given back beside states; a recurrence wider than a block of threads
    "architecture": "Purozen", "vocab": 64, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        par(sig(1, 1, 48, 20, 0.12), 300, 1.0, 1.0, None),
        par(sig(8, 2, 8, 8, 0.4), 16, -0.5, 0.9, 64),
    ],
}
PE = {  # sizes the tensor-core kernels take: heads in steps of 16, equal and unequal, pages of 16; kept tokens beyond a page
    "architecture": "Purozen", "vocab": 256, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        att(4, 2, 64, 64, 0.12, 128, mask=(40, 19), rot=(20000.0, 32, 2.0), v_mix=True),
        par(sig(4, 1, 32, 64, 0.15), 128, 0.6, 0.8, 160),
        att(8, 2, 32, 64, 0.17, 96, mask=(17, 33), rot=(500.0, 32, None), v_mix=True),
        lat(4, 32, 16, 128, 0.2, 64),
    ],
}
PF = {  # one layer, one head
    "architecture": "Purozen", "vocab": 40, "width": 32, "norm": {"eps": 1e-5},
    "layers": [lat(1, 12, 20, 16, 0.3, 24)],
}
# name -> (config, seed, weight std, page size)
TINY = {"PA": (PA, 31, 0.11, 4), "PB": (PB, 32, 0.13, 8), "PC": (PC, 33, 0.14, 16), "PD": (PD, 34, 0.15, 4),
        "PE": (PE, 35, 0.09, 16), "PF": (PF, 36, 0.2, 8)}


def make_model_dir(root, name, dtype=torch.bfloat16):
    from rllm_b200.weights import write_random_model
    cfg, seed, std, _ = TINY[name]
    d = os.path.join(str(root), f"tiny_{name}_{str(dtype).split('.')[-1]}")
    if not os.path.isdir(d):
        write_random_model(cfg, seed, d, std=std, dtype=dtype)
    return d


def random_prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
