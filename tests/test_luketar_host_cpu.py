"""CPU suite of the Luketar language model's host side: configuration, shared-weight layers, stacked projections and the
latent-space key matrices, state records, and the plain restatement's own consistency."""

import copy
import math

import pytest
import torch

from oracle import luketar_oracle as O


def config(**over):
    moe = {"kind": "moe", "expert": {"ff": 6, "limit": 1.5}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 10, "limit": 0.75}}
    cfg = {"architecture": "Luketar", "vocab": 40, "width": 16, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5}, "streams": 2,
           "layers": [{"type": "mlstm", "mixer": {"heads": 2, "dim": 4, "vdim": 6, "gate_cap": 10.0}, "mlp": None},
                      {"type": "latent_attention", "mixer": {"heads": 3, "dim": 6, "vdim": 4, "q_rank": 5, "kv_rank": 7, "scale": 0.3},
                       "mlp": moe},
                      {"type": "latent_attention", "mixer": {"heads": 3, "dim": 6, "vdim": 4, "q_rank": 5, "kv_rank": 7, "scale": 0.3},
                       "mlp": copy.deepcopy(moe), "weights_of": 1},
                      {"type": "mlstm", "mixer": {"heads": 1, "dim": 4, "vdim": 4, "gate_cap": 3.0},
                       "mlp": {"kind": "dense", "ff": 12, "limit": 2.0}}]}
    cfg.update(over)
    return cfg


def test_configuration_is_read_by_layer_type_and_checked():
    from dia_tts_prune_b200.lm_config import LuketarConfig, load_config
    c = load_config(config())
    assert isinstance(c, LuketarConfig) and [l.type for l in c.layers] == ["mlstm", "latent_attention", "latent_attention", "mlstm"]
    assert c.layers[1].mixer.kv_rank == 7 and c.layers[0].mixer.gate_cap == 10.0 and c.layers[3].mlp.kind == "dense"
    assert c.layers[1].mlp.shared.limit == 0.75 and c.streams == 2 and c.embedding.scale == 0.5
    assert [c.weight_layer(i) for i in range(4)] == [0, 1, 1, 3]
    c.check()
    plain = config()
    del plain["streams"], plain["embedding"]
    p = load_config(plain)
    assert p.streams is None and p.embedding.scale == 1.0
    bad = config()
    bad["layers"][2]["type"], bad["layers"][2]["mixer"] = "mlstm", bad["layers"][0]["mixer"]     # another kind than the layer whose weights it uses
    with pytest.raises(ValueError):
        load_config(bad).check()
    bad = config()
    bad["layers"][2]["weights_of"] = 2
    with pytest.raises(ValueError):
        load_config(bad).check()
    chain = config()
    chain["layers"].append(dict(copy.deepcopy(chain["layers"][2]), weights_of=2))     # names a layer that names layer 1
    c = load_config(chain)
    c.check()
    assert c.weight_layer(4) == 1
    bad = config()
    bad["layers"][1]["mlp"]["router"]["top"] = 6
    with pytest.raises(ValueError):
        load_config(bad).check()
    with pytest.raises(Exception):
        load_config(dict(config(), layers=[{"type": "window", "mixer": {}, "mlp": None}]))
    with pytest.raises(Exception):
        load_config(config(streams=0))


def test_layer_records_share_weights_and_stack_their_projections():
    from dia_tts_prune_b200.lm_config import load_config
    from dia_tts_prune_b200.lm_layers import GatedUnit, HyperConnection, RoutedExperts
    from dia_tts_prune_b200.lm_model import build_luketar_layers
    cfg = config()
    w = O.random_weights(cfg, 3)
    runs, final = build_luketar_layers(load_config(cfg), w, "cpu")
    assert len(runs) == 4 and runs[2] is runs[1] and runs[0] is not runs[3] and final.b is None
    att, mem = runs[1], runs[0]
    # latent attention: query latent | key/value latent | gate rows, padded to a multiple of four
    assert att.n_in == 24 and att.w_in.shape == (24, 16) and att.in_bias is None
    assert torch.equal(att.w_in[:5].float(), w["l1.mix.dq"]) and torch.equal(att.w_in[5:12].float(), w["l1.mix.dkv"])
    assert torch.equal(att.w_in[12:24].float(), w["l1.mix.g"])
    # the key up-projection per head, transposed: scores are taken in the latent space
    uk = w["l1.mix.uk"].reshape(3, 6, 7)
    assert att.mixer.w_uk_t.shape == (3, 7, 6) and all(torch.equal(att.mixer.w_uk_t[h].float(), uk[h].T) for h in range(3))
    assert att.mixer.state_spec().latent == 7 and att.mixer.state_spec().kv is None
    # matrix memory: q | k | v | input gate | forget gate | output gate rows, the gate biases in their columns
    assert mem.n_in == 8 + 8 + 12 + 2 + 2 + 12 and torch.equal(mem.in_bias[28:30], w["l0.mix.i.b"])
    assert torch.equal(mem.in_bias[30:32], w["l0.mix.f.b"]) and float(mem.in_bias.abs().sum()) == float(
        w["l0.mix.i.b"].abs().sum() + w["l0.mix.f.b"].abs().sum())
    assert mem.mixer.state_spec().recurrent == (2, 7, 4) and mem.mixer.state_spec().aux == 2
    assert isinstance(att.ff, RoutedExperts) and att.ff.softmax_top and att.ff.limit == 1.5 and att.ff.shared_limit == 0.75
    assert isinstance(runs[3].ff, GatedUnit) and runs[3].ff.w_gate_up.shape == (24, 16) and mem.ff is None and mem.hc2 is None
    assert att.hc1.streams == 2 and torch.equal(att.hc2.w_mix, w["l1.hc2.mix"])
    one = HyperConnection.residual("cpu")
    assert one.streams == 1 and float(one.w_in) == float(one.w_out) == float(one.w_mix) == 1.0
    plain = config()
    del plain["streams"]
    runs, _ = build_luketar_layers(load_config(plain), {k: v for k, v in w.items() if ".hc" not in k}, "cpu")
    assert runs[0].hc1.streams == 1


def test_state_records_hold_latent_pages_and_running_maxima():
    from dia_tts_prune_b200.lm_state import PagedState, StateSpec
    specs = [StateSpec(recurrent=(2, 7, 4), aux=2), StateSpec(latent=7), StateSpec(latent=9)]
    st = PagedState(specs, width=16, taps=0, max_tokens=40, device=torch.device("cpu"), page_size=4, max_sequences=3)
    assert st.latent_pages[0] is None and st.latent_pages[1].shape == (13, 4, 7) and st.latent_pages[2].shape == (13, 4, 9)
    assert st.k_pages[1] is None and st.rec_aux[0].shape == (3, 2) and st.rec_aux[1] is None
    r = st.record_state(0)
    assert r.rec_state.shape == (3, 2, 7, 4) and r.rec_aux is st.rec_aux[0] and st.record_state(1).latent_pages is st.latent_pages[1]


def test_synthetic_models_carry_the_tensors_the_builder_reads():
    from dia_tts_prune_b200 import synthetic
    from dia_tts_prune_b200.lm_config import load_config
    from dia_tts_prune_b200.lm_model import build_luketar_layers
    cfg = synthetic.luketar_config(32, ["latent_attention", "mlstm", "latent_attention"], 2, 8, 4, 50, q_rank=12, kv_rank=20, ff=24,
                                   experts=4, top=2, expert_ff=8, shared_ff=16, streams=3, repeat_last=True)
    c = load_config(cfg)
    c.check()
    runs, _ = build_luketar_layers(c, synthetic.luketar_weights(cfg, 1), "cpu")
    assert len(runs) == 4 and runs[3] is runs[2] and runs[0].ff.ff == 24 and runs[1].ff.experts == 4
    assert O.forward(cfg, {k: v.float() for k, v in synthetic.luketar_weights(cfg, 1).items()}, [1, 2, 3]).shape == (3, 50)


def test_the_plain_restatement_agrees_with_closed_forms():
    g = torch.Generator().manual_seed(0)
    f64 = lambda *s: torch.randn(*s, generator=g).double()      # noqa: E731
    # the clamped unit: flat in the gate above the limit, flat in the up branch beyond it on both sides, zero at g = 0
    lim = 1.5
    y = O.clamped_glu(torch.tensor([0.0, 1.5, 9.0, 1.0, 1.0, 1.0]).double(), torch.tensor([3.0, 0.2, 0.2, 1.5, 7.0, -7.0]).double(), lim)
    assert y[0] == 0 and y[1] == y[2] and y[3] == y[4] and math.isclose(float(y[5]), 1.0 / (1 + math.exp(-1.702)) * (1 - lim))
    # hyper-connections with one stream and unit weights are the residual sum
    X, yv = f64(5, 1, 8), f64(5, 8)
    one = torch.ones(1, dtype=torch.float64)
    assert torch.equal(O.hyper_read(X, one), X[:, 0]) and torch.equal(O.hyper_write(X, yv, one[None], one)[:, 0], X[:, 0] + yv)
    # the write takes every stream from the OLD ones: swapping the two streams with out = 0 is its own inverse
    X2 = f64(4, 2, 3)
    swap = torch.tensor([[0.0, 1.0], [1.0, 0.0]]).double()
    zero = torch.zeros(2).double()
    assert torch.equal(O.hyper_write(O.hyper_write(X2, f64(4, 3), swap, zero), f64(4, 3), swap, zero), X2)
    # routing: the largest logits, the lower index on a tie, weights that sum to one and follow the logits
    z = torch.tensor([[0.1, 2.0, 2.0, -1.0, 0.5]]).double()
    e, wt = O.route(z, 3)
    assert e.tolist() == [[1, 2, 4]] and math.isclose(float(wt.sum()), 1.0) and math.isclose(float(wt[0, 0]), float(wt[0, 1]))
    assert math.isclose(float(wt[0, 2] / wt[0, 0]), math.exp(0.5 - 2.0))
    # latent attention at the first position: the one key against the sink
    m = {"heads": 2, "dim": 3, "vdim": 2, "q_rank": 4, "kv_rank": 5, "scale": 0.7}
    D = 6
    p = {"dq": f64(4, D), "dq.norm": f64(4), "uq": f64(6, 4), "dkv": f64(5, D), "dkv.norm": f64(5), "uk": f64(6, 5), "uv": f64(4, 5),
         "sink": f64(2), "g": f64(4, D), "o": torch.eye(4).double()}
    h = f64(3, D)
    out = O.latent_attention(h, p, m, 1e-5)
    c = O.rms_unit(p["dkv"] @ h[0], 1e-5) * p["dkv.norm"]
    q = p["uq"] @ (O.rms_unit(p["dq"] @ h[0], 1e-5) * p["dq.norm"])
    k, v = p["uk"] @ c, p["uv"] @ c
    for hh in range(2):
        s = 0.7 * (q[3 * hh:3 * hh + 3] @ k[3 * hh:3 * hh + 3])
        share = torch.exp(s) / (torch.exp(s) + torch.exp(p["sink"][hh]))
        want = share * v[2 * hh:2 * hh + 2] * torch.sigmoid(p["g"] @ h[0])[2 * hh:2 * hh + 2]
        assert torch.allclose(out[0, 2 * hh:2 * hh + 2], want)
    # scores taken in the latent space equal scores against up-projected keys
    uk0 = p["uk"][:3]
    assert torch.allclose(q[:3] @ (uk0 @ c), (uk0.T @ q[:3]) @ c)
    # the matrix memory against the same recurrence without the running maximum (small gates: nothing overflows)
    mm = {"heads": 1, "dim": 3, "vdim": 2, "gate_cap": 5.0}
    pm = {"q": f64(3, D), "k": f64(3, D), "v": f64(2, D), "i": f64(1, D) * 0.3, "f": f64(1, D) * 0.3, "i.b": f64(1), "f.b": f64(1),
          "g": f64(2, D), "norm": torch.ones(2).double(), "o": torch.eye(2).double()}
    hs = f64(7, D)
    got = O.mlstm(hs, pm, mm, 0.0)
    S, n, raw = torch.zeros(3, 2).double(), torch.zeros(3).double(), []
    ig = 5.0 * torch.tanh((hs @ pm["i"].T + pm["i.b"]) / 5.0)
    fg = torch.nn.functional.logsigmoid(5.0 * torch.tanh((hs @ pm["f"].T + pm["f.b"]) / 5.0))
    mx = 0.0
    for t in range(7):
        kk, vv, qq = pm["k"] @ hs[t], pm["v"] @ hs[t], (pm["q"] @ hs[t]) * 3 ** -0.5
        S = torch.exp(fg[t, 0]) * S + torch.exp(ig[t, 0]) * torch.outer(kk, vv)
        n = torch.exp(fg[t, 0]) * n + torch.exp(ig[t, 0]) * kk
        mx = max(float(fg[t, 0]) + mx, float(ig[t, 0]))
        # unstabilised state = exp(m) x stabilised state: the floor exp(-m) and the 1e-6 scale with it
        raw.append((S.T @ qq) / (torch.maximum(torch.abs(n @ qq), torch.tensor(1.0).double()) + 1e-6 * math.exp(mx)))
    raw = torch.stack(raw)
    want = raw / raw.pow(2).mean(-1, keepdim=True).sqrt() * torch.sigmoid(hs @ pm["g"].T)
    assert torch.allclose(got, want)


def test_whole_model_restatement_runs_and_is_causal():
    cfg = config()
    w = O.random_weights(cfg, 3)
    toks = [1, 5, 7, 2, 9, 11, 3]
    logits, streams = O.forward(cfg, w, toks, keep_layers=True)
    assert logits.shape == (7, 40) and streams.shape == (4, 7, 16)
    other = O.forward(cfg, w, toks[:4] + [0, 0, 0])
    assert torch.allclose(other[:4], logits[:4]) and not torch.allclose(other[4:], logits[4:])
    # the embedding's scale reaches the logits only through the norms' eps and nonlinear layers: it is not a logit scale
    assert not torch.allclose(O.forward(dict(cfg, embedding={"scale": 1.0}), w, toks), logits)
    assert O.greedy(cfg, w, toks[:3], 4) == O.greedy(cfg, w, toks[:3], 4)
