"""Bazulorn without a GPU: the configuration reader, the registry, the tensors the model expects, its cache
layers, and the plain implementation's own mechanisms against closed forms."""
import json
import math

import pytest
import torch

import bazulorn_tiny as B
import plain_bazulorn as P


def test_registry_finds_the_design_by_its_architecture_string():
    from rllm_b200.config import config_from_dict, registered_architectures
    assert "Bazulorn" in registered_architectures()
    arch, cfg = config_from_dict(B.BA)
    assert arch.name == "Bazulorn" and cfg.width == 96 and cfg.vocab == 160 and cfg.norm_eps == 1e-5
    assert cfg.bigram.buckets == 211 and cfg.bigram.mul_prev == 31 and cfg.bigram.mul_cur == 5
    par, delta = cfg.layers[0], cfg.layers[1]
    assert par.type == "parallel" and par.mixer.left.window == 21 and par.mixer.left.scale == 0.2
    assert par.mixer.right.norm_groups == 2 and par.mixer.right.conv == 3 and par.mlp.kind == "dense"
    assert delta.type == "channel_delta" and delta.mixer.decay_rank == 8 and delta.mlp.shared_ff == 40
    assert delta.mlp.limit == 1.25 and delta.mlp.shared_limit == 0.75 and cfg.layers[2].mlp.shared_ff is None
    assert type(cfg).from_dict(cfg.to_dict()) == cfg
    _, bb = config_from_dict(B.BB)
    assert bb.bigram is None and bb.layers[1].mixer.left.window is None and bb.layers[1].mlp is None


@pytest.mark.parametrize("spoil,what", [
    (lambda c: c["layers"][0].update(type="serial"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(norm_groups=5), "parts"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_configuration_that_cannot_be_is_refused(spoil, what):
    from rllm_b200.config import ConfigError, config_from_dict
    raw = json.loads(json.dumps(B.BA))
    spoil(raw)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert what in str(e.value)


def test_cache_layers_pages_for_attention_states_for_the_rest():
    from rllm_b200.config import config_from_dict
    from rllm_b200.parts import KVCacheSpec, StateSpec
    arch, cfg = config_from_dict(B.BC)
    model = arch.build(cfg)
    specs = model.cache_specs()
    # two parallel layers (pages and a state each), a delta-rule layer, and the embedding's last token
    assert [type(s) for s in specs] == [KVCacheSpec, StateSpec, KVCacheSpec, StateSpec, StateSpec, StateSpec]
    assert specs[0] == KVCacheSpec(kv_heads=1, head_dim=12, window=7, chunk=None, v_dim=20)
    assert specs[2].window == 1 and specs[2].v_dim == 12
    shapes = [dict((n, s) for n, s, _ in sp.tensors) for sp in specs if isinstance(sp, StateSpec)]
    assert shapes[0]["S"] == (2, 44, 36) and shapes[0]["tail"] == (3, 2 * 36 + 2 * 2 * 44)
    assert shapes[1]["S"] == (6, 12, 8)                       # one tap: nothing of the convolution is kept
    assert shapes[2]["S"] == (2, 130, 20)
    assert [c.cache_layer for c in model.schedule] == [(0, 1), (2, 3), 4] and model.embedding_cache_layer == 5
    arch, cfg = config_from_dict(B.BD)                        # no attention: no cache layer has pages
    assert not any(isinstance(s, KVCacheSpec) for s in arch.build(cfg).cache_specs())
    arch, cfg = config_from_dict(B.BB)                        # no pair table: the embedding keeps nothing
    assert arch.build(cfg).embedding_cache_layer == -1


def test_expected_tensors_and_sizes_the_checkpoint_alone_knows(tmp_path):
    from rllm_b200.config import config_from_dict
    from rllm_b200.weights import WeightError, expected_tensors, load_weights, write_random_model
    arch, cfg = config_from_dict(B.BC)
    names = {n: tuple(s.shape) for n, s, *_ in expected_tensors(arch.build(cfg))}
    assert names["embed"] == (120, 72) and names["bigram"] == (65, 72) and names["embed.norm"] == (72,)
    assert names["final.norm"] == (72,) and "lm_head.weight" not in names and "l0.norm2" not in names
    assert names["l0.mix.left.q"] == (72, 72) and names["l0.mix.left.k"] == (12, 72) and names["l0.mix.left.v"] == (20, 72)
    assert names["l0.mix.left.q.b"] == (72,) and names["l0.mix.left.talk"] == (6, 6) and names["l0.mix.left.o"] == (72, 120)
    assert names["l0.mix.right.in"] == (2 * 72 + 2 * 2 * 44 + 2, 72) and names["l0.mix.right.conv"] == (72 + 176, 4)
    assert names["l0.mix.right.conv.b"] == (248,) and names["l0.mix.right.norm"] == (72,) and names["l0.mix.right.D"] == (2,)
    assert names["l0.mix.left.out"] == (72,) and names["l0.mix.right.out"] == (72,)
    assert names["l0.mlp.router"] == (9, 72) and names["l0.mlp.router.b"] == (9,) and names["l0.mlp.e8.down"] == (72, 20)
    assert names["l0.mlp.shared.gate"] == (12, 72) and names["l1.mlp.up"] == (48, 72)
    assert names["l2.mix.q"] == (260, 72) and names["l2.mix.v.conv"] == (40, 1) and names["l2.mix.a2"] == (260, 8)
    assert names["l2.mix.dt_bias"] == (260,) and names["l2.mix.A_log"] == (2,) and names["l2.mix.norm"] == (20,)
    assert names["l2.mix.b"] == (2, 72) and names["l2.mix.g1"] == (8, 72) and names["l2.mix.g2"] == (40, 8)
    assert not any(n.startswith("l2.mlp") for n in names)
    # a folder written with bottleneck widths loads into a model whose configuration names none
    d = write_random_model(B.BC, 3, str(tmp_path / "m"))
    raw = json.loads(json.dumps(B.BC))
    del raw["layers"][2]["mixer"]["decay_rank"], raw["layers"][2]["mixer"]["gate_rank"]
    arch, cfg = config_from_dict(raw)
    model = arch.build(cfg)
    load_weights(model, d, torch.float32, "cpu")
    # any other wrong size is still an error
    raw["layers"][0]["mixer"]["right"]["state"] = 40
    arch, cfg = config_from_dict(raw)
    with pytest.raises(WeightError) as e:
        load_weights(arch.build(cfg), d, torch.float32, "cpu")
    assert any(n == "l0.mix.right.in" for n, *_ in e.value.wrong_shape)


# ------------------------------------------------------------------ the plain implementation against closed forms

def test_plain_pair_rows_and_short_convolution():
    bg = {"buckets": 11, "mul_prev": 3, "mul_cur": 2}
    assert P.pair_rows([4, 5, 1, 1], bg) == [11, (12 + 10) % 11, (15 + 2) % 11, (3 + 2) % 11]
    x = torch.arange(1.0, 6.0, dtype=P.DT)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=P.DT)
    assert P.short_conv(x, w)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]


def test_plain_attention_window_sink_and_mix_in_closed_form():
    """Keys and queries of zero: every score is 0, the sink counts as one key more, and head h's output is the
    sum over heads g of talk[h, g] / (keys seen + 1) times the sum of the normed values it sees."""
    m = B.talk(2, 1, 4, 3, 0.5, 3)
    W, T = 5, 6
    g = torch.Generator().manual_seed(0)
    w = {"q": torch.zeros(8, W, dtype=P.DT), "k": torch.zeros(4, W, dtype=P.DT), "q.b": torch.zeros(8, dtype=P.DT),
         "k.b": torch.zeros(4, dtype=P.DT), "v": torch.randn(3, W, generator=g, dtype=P.DT), "v.b": torch.randn(3, generator=g, dtype=P.DT),
         "talk": torch.tensor([[1.0, 2.0], [0.0, -1.0]], dtype=P.DT), "o": torch.eye(6, dtype=P.DT)}
    n = torch.randn(T, W, generator=g, dtype=P.DT)
    v = n @ w["v"].T + w["v.b"]
    v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5)
    got = P.talk_attention(n, w, "", m, 1e-5)
    for i in range(T):
        seen = v[max(0, i - 2): i + 1]
        mean = seen.sum(0) / (len(seen) + 1)
        assert torch.allclose(got[i, :3], 3.0 * mean) and torch.allclose(got[i, 3:], -1.0 * mean)


def test_plain_recurrences_in_closed_form():
    # state space with one head, one state row, unit B and C: y_t = sum_s (prod_{r in (s, t]} a_r) dt_s x_s + D x_t
    m = B.ssm(1, 1, 1, 1, 1, 1)
    W, T = 3, 5
    g = torch.Generator().manual_seed(1)
    n = torch.randn(T, W, generator=g, dtype=P.DT)
    w = {"in": torch.randn(5, W, generator=g, dtype=P.DT), "conv": torch.ones(3, 1, dtype=P.DT), "conv.b": torch.zeros(3, dtype=P.DT),
         "dt_bias": torch.tensor([0.3], dtype=P.DT), "A_log": torch.tensor([-0.5], dtype=P.DT), "D": torch.tensor([0.7], dtype=P.DT),
         "norm": torch.ones(1, dtype=P.DT), "o": torch.ones(1, 1, dtype=P.DT)}
    u = n @ w["in"].T
    z, x, Bv, Cv = u[:, 0], P.silu(u[:, 1]), P.silu(u[:, 2]), P.silu(u[:, 3])
    dt = torch.log1p(torch.exp(u[:, 4] + 0.3))
    a = torch.exp(-math.exp(-0.5) * dt)
    y = []
    for t in range(T):
        s_t = sum(float(torch.prod(a[s + 1: t + 1])) * float(dt[s] * Bv[s] * x[s]) for s in range(t + 1))
        y.append(s_t * float(Cv[t]) + 0.7 * float(x[t]))
    y = torch.tensor(y, dtype=P.DT) * P.silu(z)
    want = y / torch.sqrt(y * y + 1e-5)
    assert torch.allclose(P.state_space(n, w, "", m, 1e-5)[:, 0], want)
    # delta rule with beta = 1 and no decay stores v under a unit key: reading with the same key returns it
    S = torch.zeros(4, 3, dtype=P.DT)
    k = torch.tensor([0.0, 1.0, 0.0, 0.0], dtype=P.DT)
    for v in (torch.tensor([1.0, 2.0, 3.0], dtype=P.DT), torch.tensor([-4.0, 0.5, 9.0], dtype=P.DT)):
        S = S + torch.outer(k, 1.0 * (v - S.T @ k))
        assert torch.allclose(S.T @ k, v)            # the second write replaces the first: the rule corrects, it does not add


def test_plain_experts_and_router():
    idx, wt = P.route(torch.tensor([[0.1, 2.0, -1.0, 1.5]], dtype=P.DT), 2)
    assert idx.tolist() == [[1, 3]] and torch.allclose(wt, torch.softmax(torch.tensor([[2.0, 1.5]], dtype=P.DT), -1))
    w = {"gate": torch.tensor([[1.0], [1.0]], dtype=P.DT), "up": torch.tensor([[1.0], [-1.0]], dtype=P.DT), "down": torch.eye(2, dtype=P.DT)}
    y = P.clamped_expert(torch.tensor([[5.0]], dtype=P.DT), w, "", 2.0)      # gate 5 -> 2; up 5 -> 2 and -5 -> -2
    s = 2.0 / (1 + math.exp(-1.702 * 2.0))
    assert torch.allclose(y, torch.tensor([[s * 3.0, s * -1.0]], dtype=P.DT))
    y = P.clamped_expert(torch.tensor([[-5.0]], dtype=P.DT), w, "", 2.0)     # the gate has no lower clamp
    s = -5.0 / (1 + math.exp(1.702 * 5.0))
    assert torch.allclose(y, torch.tensor([[s * -1.0, s * 3.0]], dtype=P.DT))
