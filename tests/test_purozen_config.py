"""Purozen without a GPU: the configuration reader, the registry, the tensors the model expects, its cache layers,
the cache's rule for kept first positions, and the plain implementation's own mechanisms against closed forms."""
import json
import math

import pytest
import torch

import plain_purozen as P
import purozen_tiny as Z


def test_registry_finds_the_design_by_its_architecture_string():
    from rllm_b200.config import config_from_dict, registered_architectures
    assert "Purozen" in registered_architectures()
    arch, cfg = config_from_dict(Z.PA)
    assert arch.name == "Purozen" and cfg.width == 80 and cfg.vocab == 150 and cfg.norm_eps == 1e-5
    par, att, lat = cfg.layers[0], cfg.layers[1], cfg.layers[2]
    assert par.type == "parallel" and par.mixer.left.kv_heads == 2 and par.mixer.left.vdim == 40
    assert par.mixer.right_width == 72 and par.mixer.left_scale == 0.7 and par.mixer.right_scale == 1.3 and par.ff == 96
    assert att.mixer.window == 21 and att.mixer.keep_first == 3 and att.mixer.rot_dims == 16 and att.mixer.rot_base == 5000.0
    assert att.mixer.rot_factor == 2.5 and att.mixer.v_mix and att.mixer.scale == 0.15
    assert lat.mixer.kv_rank == 40 and lat.mixer.vdim == 24 and cfg.layers[3].ff is None
    assert cfg.layers[3].mixer.rot_factor is None
    assert type(cfg).from_dict(cfg.to_dict()) == cfg
    _, pb = config_from_dict(Z.PB)            # what a configuration leaves out does not exist
    m = pb.layers[0].mixer
    assert m.window is None and m.keep_first == 0 and m.rot_dims == 0 and not m.v_mix and pb.layers[1].ff is None
    assert type(pb).from_dict(pb.to_dict()) == pb


@pytest.mark.parametrize("spoil,what", [
    (lambda c: c["layers"][0].update(type="serial"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("width"), "width"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rotated"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=48), "rotated"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0.0), "factor"),
    (lambda c: c["layers"][1]["mixer"].update(v_mix="yes"), "v_mix"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "agree"),
    (lambda c: c["layers"][2]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_configuration_that_cannot_be_is_refused(spoil, what):
    from rllm_b200.config import ConfigError, config_from_dict
    raw = json.loads(json.dumps(Z.PA))
    spoil(raw)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert what in str(e.value)


def test_cache_layers_pages_states_and_kept_first_positions():
    from rllm_b200.config import config_from_dict
    from rllm_b200.parts import KVCacheSpec, LatentCacheSpec, StateSpec
    arch, cfg = config_from_dict(Z.PA)
    model = arch.build(cfg)
    specs = model.cache_specs()
    assert [type(s) for s in specs] == [KVCacheSpec, StateSpec, KVCacheSpec, LatentCacheSpec, KVCacheSpec, KVCacheSpec, StateSpec]
    assert specs[0] == KVCacheSpec(kv_heads=2, head_dim=24, window=None, chunk=None, v_dim=40, keep_first=0)
    assert specs[1].tensors == (("S", (72,), torch.float32),)
    assert specs[2] == KVCacheSpec(kv_heads=2, head_dim=40, window=21, chunk=None, v_dim=24, keep_first=3)
    assert specs[3] == LatentCacheSpec(width=40, window=None)
    assert specs[4].window == 9 and specs[4].keep_first == 6 and specs[4].v_dim is None
    assert [c.cache_layer for c in model.schedule] == [(0, 1), 2, 3, 4, (5, 6)] and model.embedding_cache_layer == -1
    arch, cfg = config_from_dict(Z.PB)        # without a window the kept tokens mean nothing to the cache
    assert all(getattr(s, "keep_first", 0) == 0 and s.window is None for s in arch.build(cfg).cache_specs())
    # the first layer that mixes values keeps them, the later ones mix them in; a layer that does not say so does neither
    arch, cfg = config_from_dict(Z.PC)
    roles = [b.mixer.value_mix for b in arch.build(cfg).blocks if hasattr(b.mixer, "value_mix")]
    assert roles == [("first", "v_mix"), ("mix", "v_mix"), ("mix", "v_mix")]
    arch, cfg = config_from_dict(Z.PB)
    assert [b.mixer.value_mix for b in arch.build(cfg).blocks if hasattr(b.mixer, "value_mix")] == [None, None]


def test_expected_tensors(tmp_path):
    from rllm_b200.config import config_from_dict
    from rllm_b200.weights import WeightError, expected_tensors, load_weights, write_random_model
    arch, cfg = config_from_dict(Z.PA)
    names = {n: tuple(s.shape) for n, s, *_ in expected_tensors(arch.build(cfg))}
    assert names["embed"] == (150, 80) and names["final.norm"] == (80,) and "lm_head.weight" not in names
    assert names["l0.norm1"] == (80,) and names["l0.norm2"] == (80,) and "l3.norm2" not in names
    assert names["l0.rg1"] == (80, 80) and names["l0.rg1.b"] == (80,) and names["l0.rg2.b"] == (80,) and "l3.rg2" not in names
    assert names["l0.mix.left.q"] == (96, 80) and names["l0.mix.left.k"] == (48, 80) and names["l0.mix.left.v"] == (80, 80)
    assert names["l0.mix.left.pb"] == (4,) and names["l0.mix.left.o"] == (80, 160)
    assert names["l0.mix.right.z"] == (72, 80) and names["l0.mix.right.z.b"] == (72,) and names["l0.mix.right.x.b"] == (72,)
    assert names["l0.mix.right.g"] == (72, 80) and names["l0.mix.right.o"] == (80, 72)
    assert names["l1.mix.q"] == (160, 80) and names["l1.mix.k"] == (80, 80) and names["l1.mix.v"] == (48, 80)
    assert names["l1.mix.vmix"] == () and names["l3.mix.vmix"] == () and names["l1.mix.o"] == (80, 96)
    assert names["l2.mix.q"] == (48, 80) and names["l2.mix.dkv"] == (40, 80) and names["l2.mix.dkv.norm"] == (40,)
    assert names["l2.mix.uk"] == (48, 40) and names["l2.mix.uv"] == (72, 40) and names["l2.mix.o"] == (80, 72)
    assert names["l2.mlp.up"] == (48, 80) and names["l2.mlp.down"] == (80, 48)
    assert not any(n.endswith((".g", ".sink", ".q.norm")) for n in names if ".mix." in n and ".right." not in n)
    arch, cfg = config_from_dict(Z.PB)
    assert not any(n.endswith("vmix") for n, *_ in expected_tensors(arch.build(cfg)))
    # a scalar tensor passes through a model folder as a scalar
    d = write_random_model(Z.PA, 2, str(tmp_path / "a"), std=0.3)
    _, wa = P.read_model_dir(d)
    assert wa["l1.mix.vmix"].shape == () and wa["l3.mix.vmix"].shape == () and float(wa["l3.mix.vmix"]) != 0.0
    # the tensors of the smallest model, by name
    d = write_random_model(Z.PF, 1, str(tmp_path / "m"))
    cfgf, w = P.read_model_dir(d)
    assert set(w) == {"embed", "final.norm", "l0.norm1", "l0.norm2", "l0.rg1", "l0.rg1.b", "l0.rg2", "l0.rg2.b", "l0.mix.q",
                      "l0.mix.dkv", "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.o", "l0.mlp.up", "l0.mlp.down"}


def test_the_cache_never_gives_back_the_pages_of_kept_first_positions():
    from rllm_b200.cache import CacheManager
    from rllm_b200.parts import KVCacheSpec
    ps = 4
    specs = [KVCacheSpec(2, 8, window=6, keep_first=5), KVCacheSpec(2, 8, window=6), KVCacheSpec(2, 8, window=6, keep_first=4),
             KVCacheSpec(2, 8)]
    cm = CacheManager(specs, ps, 32, 2, torch.float32, "cpu", allocate=False)
    assert len(cm.groups) == 4
    rc = cm.open("a")
    cm.reserve(rc, 41)
    cm.commit(rc, 41)
    pages = rc.pages
    # the next query is position 41: its window begins at 36, page 9. Kept: 5 positions = pages 0 and 1; 4 positions = page 0
    assert [p >= 0 for p in pages[0]] == [True, True] + [False] * 7 + [True, True]
    assert [p >= 0 for p in pages[1]] == [False] * 9 + [True, True]
    assert [p >= 0 for p in pages[2]] == [True] + [False] * 8 + [True, True]
    assert all(p >= 0 for p in pages[3])
    cm.check()
    free = cm.free_pages()
    assert free == [32 - 4, 32 - 2, 32 - 3, 32 - 11]
    cm.close("a")
    assert cm.free_pages() == [32] * 4
    rc = cm.open("b")                       # a short request: nothing to give back yet, then the window passes the kept pages' neighbours
    cm.reserve(rc, 3)
    cm.commit(rc, 3)
    assert all(p >= 0 for g in rc.pages for p in g)
    cm.reserve(rc, 17)
    cm.commit(rc, 17)
    assert [p >= 0 for p in rc.pages[0]] == [True, True, False, True, True]
    cm.check()


# ------------------------------------------------------------------ the plain implementation against closed forms

def test_plain_norm_and_activation():
    x = torch.tensor([[3.0, -4.0]], dtype=P.DT)
    assert torch.allclose(P.norm_around_zero(x, torch.tensor([0.5, -1.0], dtype=P.DT), 0.0),
                          torch.tensor([[1.5 * 3 / math.sqrt(12.5), 0.0]], dtype=P.DT))
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=P.DT))) - 0.8411919906082768) < 1e-12
    assert float(P.gelu_tanh(torch.tensor(0.0, dtype=P.DT))) == 0.0


def test_plain_sigmoid_attention_is_a_running_sum_when_scores_vanish():
    """With zero queries every visible key weighs sigmoid(b): position i's output is sigmoid(b) times the sum of the
    first i + 1 values, which grows with i (nothing is normalised)."""
    T, W = 6, 4
    m = {"heads": 2, "kv_heads": 1, "dim": 3, "vdim": 2, "scale": 0.5}
    w = {"q": torch.zeros(6, W, dtype=P.DT), "k": torch.randn(3, W, dtype=P.DT), "v": torch.randn(2, W, dtype=P.DT),
         "pb": torch.tensor([0.3, -1.2], dtype=P.DT), "o": torch.eye(4, dtype=P.DT)}
    n = torch.randn(T, W, dtype=P.DT)
    got = P.sigmoid_attention(n, w, "", m)
    v = n @ w["v"].T
    want = torch.cat([torch.sigmoid(w["pb"][h]) * torch.cumsum(v, 0) for h in range(2)], dim=1)
    assert torch.allclose(got, want)


def test_plain_gated_recurrence_against_its_closed_form():
    """Constant gates: S_t = (1 - z)^t S_0-free geometric sum; and both branches of the candidate."""
    R, W, T = 3, 2, 7
    w = {"z": torch.zeros(R, W, dtype=P.DT), "z.b": torch.tensor([0.0, 2.0, -2.0], dtype=P.DT),
         "x": torch.zeros(R, W, dtype=P.DT), "x.b": torch.tensor([1.5, -0.5, 0.0], dtype=P.DT),
         "g": torch.zeros(R, W, dtype=P.DT), "o": torch.eye(R, dtype=P.DT)}
    w["g"][:, 0] = 1.0
    n = torch.ones(T, W, dtype=P.DT)
    got = P.min_gru(n, w, "", {"width": R})
    z = torch.sigmoid(w["z.b"])
    c = torch.tensor([2.0, float(torch.sigmoid(torch.tensor(-0.5))), 0.5], dtype=P.DT)
    silu1 = 1.0 / (1.0 + math.exp(-1.0))
    for t in range(T):
        assert torch.allclose(got[t], c * (1 - (1 - z) ** (t + 1)) * silu1)


def test_plain_window_mask_keeps_the_first_positions():
    ok = P.window_mask(12, {"size": 3, "keep_first": 2})
    assert ok[11].tolist() == [True, True] + [False] * 7 + [True] * 3
    assert ok[3].tolist() == [True, True, True, True] + [False] * 8
    assert ok[1].tolist() == [True, True] + [False] * 10
    assert P.window_mask(5, None)[4].all() and not P.window_mask(5, {"size": 1})[4][:4].any()


def test_plain_rotation_turns_pairs_half_a_head_apart():
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0}}
    x = torch.tensor([[[1.0, 0.0, 0.0, 1.0, 7.0]]], dtype=P.DT).repeat(3, 1, 1)
    y = P.rotate_half_layout(x, rot, torch.arange(3))
    for t in range(3):
        a0, a1 = t * 1.0 / 2.0, t * 100.0 ** -0.5 / 2.0
        want = [math.cos(a0), -math.sin(a1), math.sin(a0), math.cos(a1), 7.0]
        assert torch.allclose(y[t, 0], torch.tensor(want, dtype=P.DT))
