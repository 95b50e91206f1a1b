"""CPU suite of the Fipadra language model's host side: configuration, layer records and their stacked projections, state
records, synthetic models, and the plain restatement's own consistency."""

import copy
import math

import pytest
import torch

from oracle import fipadra_oracle as O


def config(**over):
    moe = {"kind": "moe", "expert": {"ff": 6, "limit": 1.5},
           "router": {"experts": 4, "top": 2, "identity": 2, "scale": 1.25, "groups": {"count": 3, "keep": 2}},
           "shared": {"ff": 10, "limit": 0.75}}
    cfg = {"architecture": "Fipadra", "vocab": 40, "width": 16, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
           "layers": [{"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 4, "vdim": 6, "conv": 3}, "mlp": {"kind": "dense", "ff": 12}},
                      {"type": "latent_attention",
                       "mixer": {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 4, "q_rank": 5, "kv_rank": 7, "scale": 0.3,
                                 "rot": {"base": 100.0, "dims": 4}, "mask": {"size": 5}}, "mlp": moe},
                      {"type": "retention", "mixer": {"heads": 2, "dim": 6, "vdim": 4, "decay": [0.9, 0.99], "rot": {"base": 50.0, "dims": 4}},
                       "mlp": None}]}
    cfg.update(over)
    return cfg


def test_configuration_is_read_by_layer_type_and_checked():
    from dia_tts_prune_b200.lm_config import FipadraConfig, load_config
    c = load_config(config())
    assert isinstance(c, FipadraConfig) and [l.type for l in c.layers] == ["delta", "latent_attention", "retention"]
    assert c.layers[0].mixer.conv == 3 and c.layers[1].mixer.rot_dim == 4 and c.layers[1].mixer.mask.size == 5
    assert c.layers[1].mlp.router.identity == 2 and c.layers[1].mlp.router.groups.keep == 2 and c.layers[1].mlp.router.scale == 1.25
    assert c.layers[2].mixer.decay == [0.9, 0.99] and c.layers[2].mlp is None and c.logit_scale == 0.5
    c.check()
    for breakage in (lambda b: b["layers"][0]["mixer"].update(kv_heads=3),            # heads not a multiple of kv_heads
                     lambda b: b["layers"][1]["mixer"]["rot"].update(dims=6),         # more turning channels than the turned part has
                     lambda b: b["layers"][2]["mixer"]["rot"].update(dims=3),         # an odd number of turning channels
                     lambda b: b["layers"][2]["mixer"].update(decay=[0.9]),           # one decay per head
                     lambda b: b["layers"][1]["mlp"]["router"].update(top=5),         # more than the kept groups hold
                     lambda b: b["layers"][1]["mlp"]["router"]["groups"].update(count=4)):   # 6 outputs in 4 equal groups
        bad = config()
        breakage(bad)
        with pytest.raises(ValueError):
            load_config(bad).check()
    with pytest.raises(Exception):
        load_config(dict(config(), layers=[{"type": "window", "mixer": {}, "mlp": None}]))
    free = config()
    del free["layers"][1]["mixer"]["mask"], free["layers"][1]["mlp"]["router"]["groups"], free["logit_scale"]
    f = load_config(free)
    f.check()
    assert f.layers[1].mixer.mask is None and f.layers[1].mlp.router.groups is None and f.logit_scale == 1.0


def test_layer_records_stack_their_projections_and_describe_their_state():
    from dia_tts_prune_b200.lm_config import load_config
    from dia_tts_prune_b200.lm_layers import DenseRelu2, GatedDelta, LatentAttention, Retention, RoutedExperts
    from dia_tts_prune_b200.lm_model import build_fipadra_layers
    cfg = config()
    w = O.random_weights(cfg, 3)
    layers, final = build_fipadra_layers(load_config(cfg), w, "cpu")
    assert len(layers) == 3 and all(l.parallel and l.rms and l.hc1.streams == 1 for l in layers)
    assert layers[0].hc2 is layers[0].hc1 and layers[2].hc2 is None       # both sublayers read with the same weights
    delta, att, ret = layers
    # delta rule: q | k | v | beta | decay | gate rows
    assert isinstance(delta.mixer, GatedDelta) and delta.n_in == 8 + 8 + 24 + 4 + 4 + 24
    assert torch.equal(delta.w_in[40:44].float(), w["l0.mix.b"]) and torch.equal(delta.w_in[44:48].float(), w["l0.mix.a"])
    assert torch.equal(delta.w_in[48:72].float(), w["l0.mix.g"]) and delta.mixer.conv_w.shape == (40, 3)
    sp = delta.mixer.state_spec()
    assert sp.recurrent == (4, 6, 4) and sp.conv == (3, 40) and sp.latent is None
    assert isinstance(delta.ff, DenseRelu2) and delta.ff.ff == 12
    # latent attention: query latent | key/value latent with the turned key part behind it | no gate rows; padded to four
    assert isinstance(att.mixer, LatentAttention) and not att.mixer.gated and att.n_in == 16 and att.w_in.shape == (16, 16)
    assert torch.equal(att.w_in[:5].float(), w["l1.mix.dq"]) and torch.equal(att.w_in[5:16].float(), w["l1.mix.dkv"])
    assert att.mixer.kv_rank == 7 and att.mixer.rot_dim == 4 and att.mixer.window == 5 and att.mixer.sink is None
    assert att.mixer.state_spec().latent == 11                 # the cached row: the latent and the turned key part
    uk = w["l1.mix.uk"].reshape(3, 6, 7)
    assert all(torch.equal(att.mixer.w_uk_t[h].float(), uk[h].T) for h in range(3))
    assert att.mixer.rot.numel() == 2 and math.isclose(float(att.mixer.rot[1]), 100.0 ** (-2.0 / 4), rel_tol=1e-6)
    # the mixture: one router row per expert and identity expert, and the shared unit's gate row behind them
    f = att.ff
    assert isinstance(f, RoutedExperts) and f.softmax_all and f.experts == 4 and f.identity == 2 and f.groups == (3, 2)
    assert f.w_router.shape == (7, 16) and torch.equal(f.w_router[6:].float(), w["l1.mlp.shared.sg"]) and f.has_shared_gate
    assert f.route_scale == 1.25 and torch.equal(f.correction, w["l1.mlp.correction"])
    # retention: q | k | v | gate rows; a fixed decay per head
    assert isinstance(ret.mixer, Retention) and ret.n_in == 12 + 12 + 8 + 8 and ret.ff is None
    assert ret.mixer.state_spec().recurrent == (2, 4, 6) and ret.mixer.head_norm is None and ret.mixer.rot_half
    assert torch.allclose(ret.mixer.decay, torch.tensor([0.9, 0.99]))
    assert final.w.shape == (16,)


def test_registry_knows_the_design():
    from dia_tts_prune_b200 import registry
    assert "fipadra" in registry.architectures()
    assert registry.architecture_of({"architecture": "Fipadra"}) == "Fipadra"


def test_synthetic_model_matches_the_builder():
    from dia_tts_prune_b200.lm_config import load_config
    from dia_tts_prune_b200.lm_model import build_fipadra_layers
    from dia_tts_prune_b200.synthetic import fipadra_config, fipadra_weights
    cfg = fipadra_config(64, ["delta", "latent_attention", "retention", "latent_attention"], heads=4, dim=16, vdim=8, vocab=100, kv_heads=2,
                         q_rank=24, kv_rank=32, rot_dim=8, window=9, ff=96, experts=6, top=2, identity=2, groups=(4, 2), expert_ff=32,
                         shared_ff=48, logit_scale=0.5)
    c = load_config(cfg)
    c.check()
    w = fipadra_weights(cfg, 5)
    layers, _ = build_fipadra_layers(c, w, "cpu")
    assert [type(l.mixer).__name__ for l in layers] == ["GatedDelta", "LatentAttention", "Retention", "LatentAttention"]
    assert layers[1].ff.identity == 2 and layers[3].ff.w_router.shape[0] == 9 and layers[0].ff.ff == 96
    ref = O.forward(cfg, {k: v.float() for k, v in w.items()}, [1, 2, 3, 4, 5])
    assert ref.shape == (5, 100) and torch.isfinite(ref).all()


# ---- the plain restatement against closed forms -------------------------------------------------------------------------
def test_rotation_pairs_and_angles():
    x = torch.arange(1.0, 9.0, dtype=torch.float64).repeat(3, 1)        # [3 positions, 8 channels]
    pos = torch.tensor([0, 1, 5])
    f = O.rotary_frequencies(100.0, 4)
    assert torch.allclose(f, torch.tensor([1.0, 0.1], dtype=torch.float64))
    inter = O.rotate(x, pos, 100.0, 4, "interleaved")
    half = O.rotate(x, pos, 100.0, 4, "half")
    assert torch.equal(inter[0], x[0]) and torch.equal(half[0], x[0])   # position 0 turns nothing
    assert torch.equal(inter[:, 4:], x[:, 4:]) and torch.equal(half[:, 4:], x[:, 4:])      # channels beyond dims pass
    a = 5 * 1.0
    assert math.isclose(float(inter[2, 0]), 1 * math.cos(a) - 2 * math.sin(a)) and math.isclose(float(inter[2, 1]), 2 * math.cos(a) + 1 * math.sin(a))
    assert math.isclose(float(half[2, 0]), 1 * math.cos(a) - 3 * math.sin(a)) and math.isclose(float(half[2, 2]), 3 * math.cos(a) + 1 * math.sin(a))
    b = 5 * 0.1
    assert math.isclose(float(half[2, 1]), 2 * math.cos(b) - 4 * math.sin(b)) and math.isclose(float(inter[2, 3]), 4 * math.cos(b) + 3 * math.sin(b))


def test_routing_rules_on_a_hand_made_row():
    f = {"router": {"experts": 4, "top": 2, "identity": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}}
    D = 3
    router = torch.zeros(6, D, dtype=torch.float64)
    router[:, 0] = torch.tensor([1.0, 0.0, 2.0, -1.0, 1.5, 1.4])
    p = {"router": router, "correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 0.5, 0.0], dtype=torch.float64)}
    h = torch.tensor([[1.0, 0.0, 0.0]], dtype=torch.float64)
    s = torch.softmax(router[:, 0], dim=0)
    picks, weights = O.route(h, p, f)
    # the correction lifts output 4 over output 2: its group (the identity experts 4, 5) is the one kept
    assert picks == [[4, 5]]
    assert torch.allclose(weights[0], s[[4, 5]] / s[[4, 5]].sum() * 2.0)         # weights without the correction
    picks, _ = O.route(h, p, f, correction=False)
    assert picks == [[2, 3]]                                                     # group 1 holds the largest score, then its neighbour
    picks, _ = O.route(h, p, f, groups=False)
    assert picks == [[4, 2]]
    y = O.moe_ff(h, dict(p), f)
    assert torch.allclose(y, h * 2.0)                                            # two identity experts return the input; weights sum to scale


def test_window_of_one_returns_the_own_value_and_the_recurrences_match_their_sums():
    cfg = config()
    w = {k: v.double() for k, v in O.random_weights(cfg, 7).items()}
    h = torch.randn(9, 16, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    m = copy.deepcopy(cfg["layers"][1]["mixer"])
    p = O.sub(w, "l1.mix.")
    m["mask"] = {"size": 1}
    c = O.rms_unit((h @ p["dkv"].T)[:, :7], 1e-5) * p["dkv.norm"]
    assert torch.allclose(O.latent_attention(h, p, m, 1e-5), (c @ p["uv"].T) @ p["o"].T)
    # retention as a plain double sum: o_t = sum_(s<=t) decay^(t-s) (q_t . k_s) v_s
    m2, p2 = cfg["layers"][2]["mixer"], O.sub(w, "l2.mix.")
    pos = torch.arange(9)
    q = O.rotate((h @ p2["q"].T).reshape(9, 2, 6), pos, 50.0, 4, "half")
    k = O.rotate((h @ p2["k"].T).reshape(9, 2, 6), pos, 50.0, 4, "half") * 6 ** -0.5
    v = (h @ p2["v"].T).reshape(9, 2, 4)
    o = torch.zeros(9, 2, 4, dtype=torch.float64)
    for hh in range(2):
        for t in range(9):
            for s in range(t + 1):
                o[t, hh] += m2["decay"][hh] ** (t - s) * (q[t, hh] @ k[s, hh]) * v[s, hh]
    want = (O.rms_unit(o, 1e-5).reshape(9, 8) * O.silu(h @ p2["g"].T)) @ p2["o"].T
    assert torch.allclose(O.retention(h, p2, m2, 1e-5), want)
    # the delta rule with beta = 1 and no decay stores v exactly: reading with the same unit key returns it
    S = torch.zeros(4, 6, dtype=torch.float64)
    kk = torch.tensor([0.6, 0.8, 0.0, 0.0], dtype=torch.float64)
    vv = torch.arange(6, dtype=torch.float64)
    S = S + torch.outer(kk, 1.0 * (vv - S.T @ kk))
    assert torch.allclose(S.T @ kk, vv)


def test_causal_convolution_takes_its_last_tap_for_the_current_token():
    u = torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64)
    wconv = torch.tensor([[3.0, 2.0, 1.0]], dtype=torch.float64)
    assert O.causal_conv(u, wconv).reshape(-1).tolist() == [1.0, 12.0, 123.0]
