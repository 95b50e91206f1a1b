"""GPU parity of the Luketar language model against the plain restatement in ``oracle/luketar_oracle.py``.

Small made-up configurations and random weights; the product runs through ``CausalLM`` / ``LMEngine`` (state records,
scheduler, CUDA kernels), the oracle recomputes whole sequences in float64 on the CPU without cache or carried state.
"""

import copy
import json
import math

import pytest
import torch

from oracle import luketar_oracle as O

pytestmark = pytest.mark.gpu

LAT = {"heads": 3, "dim": 24, "vdim": 16, "q_rank": 40, "kv_rank": 56, "scale": 0.2}
MEM = {"heads": 3, "dim": 16, "vdim": 24, "gate_cap": 12.0}
DENSE = {"kind": "dense", "ff": 72, "limit": 1.25}
MOE = {"kind": "moe", "expert": {"ff": 24, "limit": 1.0}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 40, "limit": 2.5}}


def layer(kind, mixer, mlp=DENSE, **more):
    return dict({"type": kind, "mixer": copy.deepcopy(mixer), "mlp": copy.deepcopy(mlp)}, **more)


def small_config(**over):
    cfg = {"architecture": "Luketar", "vocab": 130, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.75}, "streams": 2,
           "layers": [layer("latent_attention", LAT), layer("mlstm", MEM, MOE), layer("latent_attention", LAT, MOE),
                      layer("mlstm", MEM, MOE, weights_of=1)]}
    cfg.update(over)
    return cfg


def odd_config():
    """Sizes that share nothing and are multiples of nothing: one head and several, head sizes off every vector width,
    query and key/value latents of different size both ways, one chosen expert and all of them, a mixture without shared
    unit, layers without feed-forward, a recurrent first layer, an attention layer that runs twice, four streams."""
    return {"architecture": "Luketar", "vocab": 77, "width": 72, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5}, "streams": 4,
            "layers": [layer("mlstm", {"heads": 1, "dim": 37, "vdim": 9, "gate_cap": 4.0}, None),
                       layer("latent_attention", {"heads": 5, "dim": 10, "vdim": 7, "q_rank": 13, "kv_rank": 34, "scale": 0.4},
                             {"kind": "moe", "expert": {"ff": 9, "limit": 0.75}, "router": {"experts": 5, "top": 1}, "shared": None}),
                       layer("latent_attention", {"heads": 1, "dim": 33, "vdim": 70, "q_rank": 50, "kv_rank": 11, "scale": 0.15},
                             {"kind": "dense", "ff": 31, "limit": 3.0}),
                       layer("mlstm", {"heads": 6, "dim": 10, "vdim": 7, "gate_cap": 30.0},
                             {"kind": "moe", "expert": {"ff": 18, "limit": 2.0}, "router": {"experts": 3, "top": 3},
                              "shared": {"ff": 5, "limit": 0.5}}),
                       layer("latent_attention", {"heads": 5, "dim": 10, "vdim": 7, "q_rank": 13, "kv_rank": 34, "scale": 0.4},
                             {"kind": "moe", "expert": {"ff": 9, "limit": 0.75}, "router": {"experts": 5, "top": 1}, "shared": None},
                             weights_of=1),
                       layer("mlstm", {"heads": 2, "dim": 8, "vdim": 8, "gate_cap": 15.0}, None)]}


def plain_config():
    """One plain residual stream (no hyper-connection tensors), no embedding entry; a width and a vocabulary that admit no
    vector load and no tensor-core shape."""
    cfg = small_config(width=54, vocab=61)
    del cfg["streams"], cfg["embedding"]
    return cfg


def build(cfg, seed=1, dtype="float32", weights=None, **kw):
    from dia_tts_prune_b200.lm_config import LuketarConfig
    from dia_tts_prune_b200.lm_model import CausalLM
    w = O.random_weights(cfg, seed) if weights is None else weights
    kw.setdefault("max_tokens", 640)
    kw.setdefault("page_size", 8)
    return CausalLM(LuketarConfig.model_validate(cfg), w, dtype=dtype, device="cuda:0", **kw), w


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def close(got, ref, tol=2e-4, slack=0.0):
    got, ref = got.detach().cpu().double(), ref.double()
    err = (got - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()) + 2.0 * slack, err


def mixer_ref(kind, h, p, m, eps):
    """The float64 reference of a mixer and how far the same plain code lands from it in float32 arithmetic: where a
    configuration is ill-conditioned (a one-key normaliser next to its floor), that much is rounding, not a fault."""
    ref = O.MIXERS[kind](h.double(), p, m, eps)
    ref32 = O.MIXERS[kind](h.float(), {k: v.float() for k, v in p.items()}, m, eps)
    return ref, (ref32.double() - ref).abs().max().item()


def whole(model, name, toks, want=None, **kw):
    want = list(range(len(toks))) if want is None else want
    return model.run_step([{"id": name, "tokens": toks, "want": want}], [name], **kw)


def part(w, prefix):
    return {k[len(prefix):]: v.double() for k, v in w.items() if k.startswith(prefix)}


def run_mixer(model, record, h, cuts):
    """The mixer of one layer record alone on given inputs, fed in portions ``cuts`` to a fresh sequence."""
    T = h.shape[0]
    assert sum(cuts) == T
    seq = model.state.open("t")
    model.state.reserve(seq, T)
    out, at = [], 0
    for n in cuts:
        out.append(model.engine.op_mixer(record, h[at:at + n].cuda(), [(seq, n, at)]))
        at += n
    model.state.close("t")
    return torch.cat(out)


# ---- each mechanism alone -----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("make", [small_config, odd_config])
@pytest.mark.parametrize("cuts", [[75], [40] + [1] * 35, [17, 15, 1, 2, 16, 3, 21]])
def test_every_mixer_alone_whole_in_portions_and_decoded(make, cuts):
    cfg = make()
    model, w = build(cfg, 4)
    h = torch.randn(75, cfg["width"], generator=torch.Generator().manual_seed(6))
    for i, lc in enumerate(cfg["layers"]):
        src = lc.get("weights_of", i)
        ref, slack = mixer_ref(lc["type"], h, part(w, f"l{src}.mix."), lc["mixer"], cfg["norm"]["eps"])
        close(run_mixer(model, i, h, cuts), ref, 2e-5, slack)


@pytest.mark.parametrize("rows", [1, 3, 8, 40])
def test_feed_forwards_alone_on_every_branch_of_the_clamps(rows):
    cfg = small_config()
    model, w = build(cfg, 5)
    h = torch.randn(rows, cfg["width"], generator=torch.Generator().manual_seed(rows)) * 2
    p = part(w, "l0.mlp.")
    g, u = h.double() @ p["gate"].T, h.double() @ p["up"].T
    lim = DENSE["limit"]
    assert (g > lim).any() and (g < -lim).any() and (u > lim).any() and (u < -lim).any() and (u.abs() < lim).any()
    close(model.engine.op_ff(0, h.cuda()), O.dense_ff(h.double(), p, cfg["layers"][0]["mlp"]), 2e-5)
    close(model.engine.op_ff(1, h.cuda()), O.expert_ff(h.double(), part(w, "l1.mlp."), cfg["layers"][1]["mlp"]), 2e-5)


@pytest.mark.parametrize("experts,top,shared", [(1, 1, False), (7, 7, True), (70, 3, True), (12, 5, False)])
def test_router_takes_the_largest_biased_logits_and_weighs_outputs_by_their_softmax(experts, top, shared):
    mlp = {"kind": "moe", "expert": {"ff": 16, "limit": 1.5}, "router": {"experts": experts, "top": top},
           "shared": {"ff": 8, "limit": 1.0} if shared else None}
    cfg = small_config(layers=[layer("mlstm", MEM, mlp)])
    w = O.random_weights(cfg, 8)
    w["l0.mlp.router.b"] = torch.linspace(-3, 3, experts).to(torch.bfloat16).float()      # the bias decides many choices
    model, _ = build(cfg, weights=w)
    h = torch.randn(50, cfg["width"], generator=torch.Generator().manual_seed(experts))
    p = part(w, "l0.mlp.")
    ref = O.expert_ff(h.double(), p, mlp)
    if experts > top:
        unbiased = O.expert_ff(h.double(), dict(p, **{"router.b": torch.zeros(experts, dtype=torch.float64)}), mlp)
        assert (unbiased - ref).abs().max() > 1e-3
    close(model.engine.op_ff(0, h.cuda()), ref, 2e-5)
    close(torch.cat([model.engine.op_ff(0, h[i:i + 5].cuda()) for i in range(0, 50, 5)]), ref, 2e-5)


@pytest.mark.parametrize("heads,dim,vdim,q_rank,kv_rank", [(12, 128, 32, 64, 128), (16, 16, 128, 24, 64), (3, 136, 200, 9, 256),
                                                           (2, 8, 8, 200, 4), (32, 40, 8, 16, 48), (2, 16, 24, 32, 300), (3, 8, 8, 8, 1000),
                                                           (130, 8, 4, 16, 20), (40, 12, 8, 16, 250)])
def test_latent_attention_with_other_shapes(heads, dim, vdim, q_rank, kv_rank):
    """Tile heights from 16 rows down, latents up to 256 wide on the tiled kernel; wider latents and more heads than a tile
    holds on the kernel that takes every (row, head) on its own."""
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": dim ** -0.5}
    cfg = small_config(layers=[layer("latent_attention", mixer, None)])
    model, w = build(cfg, 48)
    h = torch.randn(90, cfg["width"], generator=torch.Generator().manual_seed(dim))
    ref = O.latent_attention(h.double(), part(w, "l0.mix."), mixer, cfg["norm"]["eps"])
    close(run_mixer(model, 0, h, [70] + [1] * 20), ref, 2e-5)


@pytest.mark.parametrize("heads,dim,vdim", [(4, 128, 128), (2, 200, 20), (5, 72, 130), (1, 3, 15), (9, 32, 16)])
def test_matrix_memory_with_other_state_shapes(heads, dim, vdim):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": 10.0}
    cfg = small_config(layers=[layer("mlstm", mixer, None)])
    model, w = build(cfg, 49)
    h = torch.randn(50, cfg["width"], generator=torch.Generator().manual_seed(vdim))
    ref, slack = mixer_ref("mlstm", h, part(w, "l0.mix."), mixer, cfg["norm"]["eps"])
    close(run_mixer(model, 0, h, [33, 1, 1, 15]), ref, 2e-5, slack)


# ---- the whole model ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("make", [small_config, odd_config, plain_config])
def test_whole_prompt_logits_and_layer_streams(make):
    cfg = make()
    model, w = build(cfg, 11)
    toks = tokens(cfg, 61, 2)
    ref, streams = O.forward(cfg, w, toks, keep_layers=True)
    got, got_streams = whole(model, "a", toks, keep_layers=True)
    assert got_streams.shape[0] == len(cfg["layers"])
    # (how far the plain code itself lands in float32 arithmetic: small, ill-conditioned layers amplify rounding)
    slack = (O.forward(cfg, w, toks, dtype=torch.float32, keep_layers=True)[1].double() - streams).abs().max().item()
    close(got_streams, streams, 2e-5, slack)
    close(got, ref)
    for n in (1, 2, 3):                                         # the first tokens of a sequence
        close(whole(model, "b", toks[:n]), ref[:n])


@pytest.mark.parametrize("streams", [None, 1, 3, 8])
def test_streams_are_read_mixed_and_written_with_their_own_weights(streams):
    cfg = small_config(streams=streams)
    if streams is None:
        del cfg["streams"]
    model, w = build(cfg, 10)
    toks = tokens(cfg, 33, 5)
    ref = O.forward(cfg, w, toks)
    if streams and streams > 1:                                 # [from, to], not [to, from]; all streams from the OLD ones
        wt = dict(w)
        for k in w:
            if k.endswith(".mix") and ".hc" in k:
                wt[k] = w[k].T.contiguous()
        assert (O.forward(cfg, wt, toks) - ref).abs().max() > 1e-2
    close(whole(model, "a", toks), ref)
    got = [model.run_step([{"id": "d", "tokens": toks[:20], "want": list(range(20))}])]
    got += [model.run_step([{"id": "d", "tokens": [t], "want": [0]}]) for t in toks[20:]]
    model.run_step([], ["d"])
    close(torch.cat(got), ref)


@pytest.mark.parametrize("make", [small_config, odd_config, plain_config])
def test_prefill_then_long_token_by_token_decoding(make):
    cfg = make()
    model, w = build(cfg, 12)
    toks = tokens(cfg, 150, 3)
    ref = O.forward(cfg, w, toks)
    got = [model.run_step([{"id": "d", "tokens": toks[:9], "want": list(range(9))}])]
    for t in range(9, 150):
        got.append(model.run_step([{"id": "d", "tokens": [toks[t]], "want": [0]}], ["d"] if t == 149 else []))
    close(torch.cat(got), ref)


@pytest.mark.parametrize("make", [small_config, odd_config])
@pytest.mark.parametrize("cuts", [[2] * 40, [1, 2, 3, 5, 8, 13, 21, 27], [19, 1, 20, 21, 2, 17], [79, 1], [3, 77]])
def test_portions_of_any_size_give_the_same_logits(make, cuts):
    cfg = make()
    model, w = build(cfg, 13, max_rows=32)                      # long portions are also split by the engine itself
    toks = tokens(cfg, 80, 4)
    ref = O.forward(cfg, w, toks)
    assert sum(cuts) == 80
    got, at = [], 0
    for n in cuts:
        got.append(model.run_step([{"id": "p", "tokens": toks[at:at + n], "want": list(range(n))}]))
        at += n
    model.run_step([], ["p"])
    close(torch.cat(got), ref)
    close(torch.cat(got), whole(model, "q", toks).cpu(), 2e-5)   # how the rows were cut changes rounding at most


@pytest.mark.parametrize("make", [small_config, odd_config])
def test_mixed_batch_of_unequal_requests_equals_each_alone(make):
    cfg = make()
    model, w = build(cfg, 15, max_sequences=4)
    A, B, C = tokens(cfg, 50, 6), tokens(cfg, 31, 7), tokens(cfg, 12, 8)
    alone = {n: whole(model, n, t) for n, t in (("A", A), ("B", B), ("C", C))}
    out = {"A": [], "B": [], "C": []}

    def run(parts, end=()):
        lg = model.run_step([{"id": n, "tokens": t, "want": list(range(len(t)))} for n, t in parts], list(end))
        at = 0
        for n, t in parts:
            out[n].append(lg[at:at + len(t)])
            at += len(t)

    run([("A", A[:23]), ("C", C)], end=["C"])                   # a portion beside a whole prompt
    run([("A", A[23:40]), ("B", B[:25])])
    for k in range(6):                                          # two requests decode side by side
        run([("B", [B[25 + k]]), ("A", [A[40 + k]])])
    run([("A", A[46:])], end=["A", "B"])
    for n in "ABC":
        got = torch.cat(out[n])
        close(got, alone[n][:got.shape[0]].cpu(), 2e-5)
    close(alone["A"], O.forward(cfg, w, A))
    # two prompts in one step against each alone, all on the kernels of long steps: the very same bits
    both = model.run_step([{"id": "A", "tokens": A, "want": list(range(50))},
                           {"id": "B", "tokens": B, "want": list(range(31))}], ["A", "B"])
    assert torch.equal(both[:50], alone["A"]) and torch.equal(both[50:], alone["B"])


def test_freed_pages_slots_and_states_are_used_again():
    cfg = small_config()
    model, w = build(cfg, 16, max_tokens=96, max_sequences=2, page_size=8)
    st = model.state
    X, Y, Z = tokens(cfg, 70, 9), tokens(cfg, 26, 10), tokens(cfg, 64, 11)
    ref = {n: O.forward(cfg, w, t) for n, t in (("X", X), ("Y", Y), ("Z", Z))}
    gx = model.run_step([{"id": "X", "tokens": X, "want": list(range(70))}])
    gy = model.run_step([{"id": "Y", "tokens": Y, "want": list(range(26))}])
    pages_x, slot_x = list(st.sequences["X"].pages), st.sequences["X"].slot
    assert st.free_slots == 0
    model.run_step([], ["X"])
    # Z takes X's slot and pages - dirty with X's latents, matrix states, normalisers and running maxima - and starts
    # with two tokens, while Y's state stays as it is
    gz = model.run_step([{"id": "Z", "tokens": Z[:2], "want": [0, 1]}])
    assert st.sequences["Z"].slot == slot_x and set(st.sequences["Z"].pages) <= set(pages_x)
    gz1 = model.run_step([{"id": "Z", "tokens": Z[2:40], "want": list(range(38))}])
    gz2 = model.run_step([{"id": "Z", "tokens": Z[40:], "want": list(range(24))}], ["Z", "Y"])
    close(gx, ref["X"]); close(gy, ref["Y"]); close(torch.cat([gz, gz1, gz2]), ref["Z"])
    assert st.free_pages == st.n_pages and st.free_slots == 2
    from dia_tts_prune_b200.lm_state import OutOfPages
    with pytest.raises(OutOfPages):
        model.run_step([{"id": "big", "tokens": tokens(cfg, 200, 1), "want": []}])


def test_a_layer_that_runs_twice_has_one_set_of_weights_and_two_states():
    cfg = small_config()
    model, w = build(cfg, 25)
    assert model.layers[3] is model.layers[1] and not any(k.startswith("l3.") for k in w)
    states = [t.data_ptr() for t in model.state.rec_states if t is not None]
    assert len(states) == 2 and len(set(states)) == 2
    toks = tokens(cfg, 40, 12)
    ref = O.forward(cfg, w, toks)
    once = dict(cfg, layers=cfg["layers"][:3])
    assert (O.forward(once, w, toks) - ref).abs().max() > 1e-2
    got = [model.run_step([{"id": "d", "tokens": toks[:25], "want": list(range(25))}])]
    got += [model.run_step([{"id": "d", "tokens": [t], "want": [0]}]) for t in toks[25:]]
    model.run_step([], ["d"])
    close(torch.cat(got), ref)


# ---- inputs and weights made so that one thing stands out -----------------------------------------------------------------
def standout_attention(page_size):
    """One latent attention layer whose query path equals its key path (same down-projection, same norm, same
    up-projection), so that a position whose input points the way the query's input does gets a score far above all
    others."""
    mixer = {"heads": 2, "dim": 32, "vdim": 32, "q_rank": 48, "kv_rank": 48, "scale": 0.5}
    cfg = small_config(layers=[layer("latent_attention", mixer, None)])
    w = O.random_weights(cfg, 21)
    w["l0.mix.dq"], w["l0.mix.dq.norm"], w["l0.mix.uq"] = w["l0.mix.dkv"], w["l0.mix.dkv.norm"], w["l0.mix.uk"]
    w["l0.mix.sink"] = torch.tensor([0.5, -1.0])
    model, _ = build(cfg, weights=w, max_tokens=512, page_size=page_size)
    return cfg, w, model


@pytest.mark.parametrize("decode", [False, True])
def test_standout_key_far_away_at_page_and_tile_borders(decode):
    P = 16
    cfg, w, model = standout_attention(P)
    T = 300
    g = torch.Generator().manual_seed(2)
    base = torch.randn(T, 96, generator=g) * 0.3
    mark, near = torch.randn(96, generator=g) * 3, torch.randn(96, generator=g) * 2
    p, m = part(w, "l0.mix."), cfg["layers"][0]["mixer"]
    i = T - 1
    blank = base.clone()
    blank[i] = mark
    ref_blank = O.latent_attention(blank.double(), p, m, 1e-5)
    # the first token, far back among hundreds, both sides of page borders and of the 64-key tile border, the neighbour
    for j in (0, 3, 63, 64, 127, 128, (i // P) * P, (i // P) * P - 1, i - 1):
        h = base.clone()
        h[j] = 2 * mark + near                                  # nearly the query's direction, a value of its own
        h[i] = mark
        ref = O.latent_attention(h.double(), p, m, 1e-5)
        assert (ref[i] - ref_blank[i]).abs().max() > 1e-2, j    # the marked key carries the row
        n0 = T - 60 if decode else T
        close(run_mixer(model, 0, h, [n0] + [1] * (T - n0)), ref, 2e-5)


def test_sink_counts_once_has_no_value_and_is_not_scaled():
    mixer = dict(LAT, scale=0.05)
    cfg = small_config(layers=[layer("latent_attention", mixer, None)])
    w = O.random_weights(cfg, 22)
    w["l0.mix.sink"] = torch.tensor([3.0, 2.0, 4.0])
    model, _ = build(cfg, weights=w, max_tokens=64)
    h = torch.randn(12, 96, generator=torch.Generator().manual_seed(3))
    p = part(w, "l0.mix.")
    ref = O.latent_attention(h.double(), p, mixer, 1e-5)
    for other in (dict(p, sink=torch.full((3,), -1e9, dtype=torch.float64)),          # no sink
                  dict(p, sink=p["sink"] + math.log(2.0)),                             # the sink counted twice
                  dict(p, sink=p["sink"] * mixer["scale"])):                           # the sink scaled like a score
        assert (O.latent_attention(h.double(), other, mixer, 1e-5) - ref).abs().max() > 1e-3
    close(run_mixer(model, 0, h, [12]), ref, 2e-5)
    close(run_mixer(model, 0, h, [5] + [1] * 7), ref, 2e-5)


def long_memory_model():
    """A matrix memory that forgets almost nothing (forget gates at the cap), so that the first tokens still carry the
    read-out hundreds of tokens on."""
    mixer = {"heads": 2, "dim": 16, "vdim": 16, "gate_cap": 8.0}
    cfg = small_config(layers=[layer("mlstm", mixer, None)])
    w = O.random_weights(cfg, 23)
    w["l0.mix.f.b"] = torch.full((2,), 40.0)
    model, _ = build(cfg, weights=w, max_tokens=512, page_size=16)
    return cfg, w, model


@pytest.mark.parametrize("cuts", [[400], [340] + [1] * 60, [2, 14, 16, 1, 31, 64, 272]])
def test_matrix_memory_keeps_the_first_tokens_over_hundreds_of_steps(cuts):
    cfg, w, model = long_memory_model()
    h = torch.randn(400, 96, generator=torch.Generator().manual_seed(5)) * 0.5
    p, m = part(w, "l0.mix."), cfg["layers"][0]["mixer"]
    ref = O.mlstm(h.double(), p, m, 1e-5)
    h2 = h.clone()
    h2[1] = h2[1] * -3.0                                        # what the second token wrote is still read at the end
    assert (O.mlstm(h2.double(), p, m, 1e-5)[-1] - ref[-1]).abs().max() > 1e-3
    close(run_mixer(model, 0, h, cuts), ref, 5e-5)


@pytest.mark.parametrize("cuts", [[30], [1] * 30, [2, 5, 23]])
def test_normaliser_floor_and_gate_cap_with_low_input_gates(cuts):
    """Input gates far below zero: the running maximum stays where it started and the normaliser n . q under its floor
    exp(-m); pre-activations beyond the cap show the cap."""
    mixer = {"heads": 2, "dim": 16, "vdim": 16, "gate_cap": 6.0}
    cfg = small_config(layers=[layer("mlstm", mixer, None)])
    w = O.random_weights(cfg, 26)
    w["l0.mix.i.b"], w["l0.mix.f.b"] = torch.tensor([-9.0, -2.5]), torch.tensor([9.0, 1.0])
    model, _ = build(cfg, weights=w)
    h = torch.randn(30, 96, generator=torch.Generator().manual_seed(9))
    p = part(w, "l0.mix.")
    ref = O.mlstm(h.double(), p, mixer, 1e-5)
    assert (O.mlstm(h.double(), p, mixer, 1e-5, floor=False) - ref).abs().max() > 1e-3
    assert (O.mlstm(h.double(), p, dict(mixer, gate_cap=60.0), 1e-5) - ref).abs().max() > 1e-3
    close(run_mixer(model, 0, h, cuts), ref, 2e-5)


# ---- precisions, replayed steps, drawn sizes ------------------------------------------------------------------------------
def wide_config():
    """Sizes the tensor-core kernel takes: every product of a 64-row step runs with bfloat16 operands."""
    lat = {"heads": 4, "dim": 32, "vdim": 32, "q_rank": 64, "kv_rank": 48, "scale": 0.18}
    moe = {"kind": "moe", "expert": {"ff": 32, "limit": 1.5}, "router": {"experts": 8, "top": 2}, "shared": {"ff": 64, "limit": 1.5}}
    return small_config(width=128, vocab=256, streams=3,
                        layers=[layer("latent_attention", lat, {"kind": "dense", "ff": 128, "limit": 2.0}),
                                layer("mlstm", {"heads": 4, "dim": 32, "vdim": 32, "gate_cap": 15.0}, moe),
                                layer("latent_attention", lat, moe)])


@pytest.mark.parametrize("make", [wide_config, small_config, plain_config])
def test_bfloat16_products_stay_within_bfloat16_rounding_of_the_oracle(make):
    cfg = make()
    lo, w = build(cfg, 31, dtype="bfloat16")
    toks = tokens(cfg, 70, 13)
    ref = O.forward(cfg, w, toks)
    got = whole(lo, "a", toks).cpu().double()
    err = (got - ref).abs().amax(dim=-1) / ref.abs().max()
    assert err.max() < 6e-2 and err.median() < 2e-2, (err.max(), err.median())
    dec = torch.cat([lo.run_step([{"id": "d", "tokens": toks[:40], "want": list(range(40))}])] +
                    [lo.run_step([{"id": "d", "tokens": [t], "want": [0]}]) for t in toks[40:]]).cpu().double()
    lo.run_step([], ["d"])
    err = (dec - ref).abs().amax(dim=-1) / ref.abs().max()
    assert err.max() < 6e-2 and err.median() < 2e-2, (err.max(), err.median())


def test_replayed_step_graphs_give_the_same_bits_as_plain_launches():
    cfg = small_config()
    a, w = build(cfg, 32, step_graphs=True)
    b, _ = build(cfg, 32, step_graphs=False)
    toks = tokens(cfg, 30, 14)
    for m in (a, b):
        m.run_step([{"id": "s", "tokens": toks[:20], "want": []}])
    for t in toks[20:]:
        ga = a.run_step([{"id": "s", "tokens": [t], "want": [0]}])
        gb = b.run_step([{"id": "s", "tokens": [t], "want": [0]}])
        assert torch.equal(ga, gb)


def drawn_config(seed):
    g = torch.Generator().manual_seed(2000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))          # noqa: E731
    layers = []
    for _ in range(r(2, 5)):
        m = {"heads": r(1, 6), "dim": r(3, 40), "vdim": r(3, 40)}
        if r(0, 1):
            kind = "latent_attention"
            m.update(q_rank=r(3, 60), kv_rank=r(3, 60), scale=0.05 + 0.05 * r(0, 6))
        else:
            kind = "mlstm"
            m.update(gate_cap=float(r(2, 30)))
        pick = r(0, 2)
        if pick == 0:
            mlp = None
        elif pick == 1:
            mlp = {"kind": "dense", "ff": r(5, 70), "limit": 0.5 * r(1, 14)}
        else:
            E = r(1, 9)
            mlp = {"kind": "moe", "expert": {"ff": r(3, 30), "limit": 0.5 * r(1, 14)}, "router": {"experts": E, "top": r(1, E)},
                   "shared": {"ff": r(3, 40), "limit": 0.5 * r(1, 14)} if r(0, 1) else None}
        layers.append(layer(kind, m, mlp))
    if r(0, 1):
        j = r(0, len(layers) - 1)
        layers.insert(r(j + 1, len(layers)), dict(copy.deepcopy(layers[j]), weights_of=j))
    cfg = {"architecture": "Luketar", "vocab": r(20, 200), "width": 2 * r(8, 60), "norm": {"eps": 10.0 ** -r(4, 7)},
           "embedding": {"scale": 0.25 * r(1, 8)}, "layers": layers}
    if r(0, 3):
        cfg["streams"] = r(1, 5)
    return cfg


@pytest.mark.parametrize("seed", range(8))
def test_drawn_configurations_whole_portioned_and_decoded(seed):
    cfg = drawn_config(seed)
    model, w = build(cfg, 40 + seed, page_size=(4, 8, 16)[seed % 3])
    toks = tokens(cfg, 55, seed)
    ref = O.forward(cfg, w, toks)
    close(whole(model, "a", toks), ref)
    got, at = [], 0
    for n in (7, 2, 19, 1, 1, 12):
        got.append(model.run_step([{"id": "p", "tokens": toks[at:at + n], "want": list(range(n))}]))
        at += n
    got += [model.run_step([{"id": "p", "tokens": [t], "want": [0]}]) for t in toks[at:]]
    model.run_step([], ["p"])
    close(torch.cat(got), ref)


# ---- generation through the scheduler, the registry and the command line ---------------------------------------------------
def test_greedy_generation_through_the_scheduler():
    cfg = small_config()
    model, w = build(cfg, 17, max_tokens=400, max_sequences=3, max_rows=24)
    prompts = [tokens(cfg, 37, 20), tokens(cfg, 5, 21), tokens(cfg, 1, 22), tokens(cfg, 50, 23), tokens(cfg, 18, 24)]
    outs = model.generate(prompts, max_new_tokens=10, max_step_tokens=24)      # 5 requests over 3 slots, portioned prompts
    assert model.state.free_slots == 3 and model.state.free_pages == model.state.n_pages
    for p, o in zip(prompts, outs):
        assert len(o) == 10
        ref = O.forward(cfg, w, p + o[:-1])[len(p) - 1:]
        top2 = torch.topk(ref, 2, dim=-1)
        for t, tok in enumerate(o):
            if tok != int(top2.indices[t, 0]):                 # only an exact near-tie may go the other way
                assert tok == int(top2.indices[t, 1]) and float(top2.values[t, 0] - top2.values[t, 1]) < 1e-4
    assert model.generate(prompts[:2], max_new_tokens=10) == outs[:2]


def test_registry_loads_a_model_folder_and_the_trace_command_replays_steps(tmp_path):
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    from dia_tts_prune_b200.checkpoint import save_safetensors
    from dia_tts_prune_b200.registry import load_model
    cfg = odd_config()
    w = O.random_weights(cfg, 30)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    model = load_model(tmp_path, dtype="float32", max_tokens=128)
    toks = tokens(cfg, 40, 31)
    ref = O.forward(cfg, w, toks)
    close(whole(model, "r", toks), ref)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:33], "want": [0, 32]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[33:35], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[35:], "want": [4, 1]}], "end": ["x"]}]
    root = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out",
                        str(tmp_path / "out"), "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (tmp_path / "out" / "1.f32").exists()
    got0 = torch.from_numpy(np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(2, -1))
    got2 = torch.from_numpy(np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(2, -1))
    close(got0, ref[[0, 32]])
    close(got2, ref[[39, 36]])
