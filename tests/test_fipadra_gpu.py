"""GPU parity of the Fipadra language model against the plain restatement in ``oracle/fipadra_oracle.py``.

Small made-up configurations and random weights; the product runs through ``CausalLM`` / ``LMEngine`` (state records,
scheduler, CUDA kernels), the oracle recomputes whole sequences in float64 on the CPU without cache or carried state.
"""

import copy
import json

import pytest
import torch

from oracle import fipadra_oracle as O

pytestmark = pytest.mark.gpu

DELTA = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 4}
LAT = {"heads": 3, "dim": 24, "rot_dim": 8, "vdim": 16, "q_rank": 40, "kv_rank": 56, "scale": 0.2,
       "rot": {"base": 1000.0, "dims": 8}, "mask": {"size": 21}}
RET = {"heads": 3, "dim": 16, "vdim": 24, "decay": [0.9, 0.97, 0.995], "rot": {"base": 500.0, "dims": 16}}
DENSE = {"kind": "dense", "ff": 72}
MOE = {"kind": "moe", "expert": {"ff": 24, "limit": 1.0},
       "router": {"experts": 6, "top": 2, "identity": 2, "scale": 1.5, "groups": {"count": 4, "keep": 2}},
       "shared": {"ff": 40, "limit": 2.5}}


def layer(kind, mixer, mlp=DENSE):
    return {"type": kind, "mixer": copy.deepcopy(mixer), "mlp": copy.deepcopy(mlp)}


def small_config(**over):
    cfg = {"architecture": "Fipadra", "vocab": 130, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.75,
           "layers": [layer("delta", DELTA), layer("latent_attention", LAT, MOE), layer("retention", RET, MOE),
                      layer("delta", DELTA, MOE), layer("retention", RET)]}
    cfg.update(over)
    return cfg


def odd_config():
    """Sizes that share nothing and are multiples of nothing: one head and several, as many key heads as heads and fewer,
    head sizes off every vector width, 1 and 5 taps, a turned part smaller and larger than the plain part, rotation of a
    part of the channels and of none, windows of 1 and beyond the prompt, no window, one group and groups that all stay,
    no identity experts and mostly identity experts, a mixture without shared unit, layers without feed-forward."""
    moe_a = {"kind": "moe", "expert": {"ff": 9, "limit": 0.75}, "router": {"experts": 5, "top": 1, "identity": 0, "scale": 1.0},
             "shared": None}
    moe_b = {"kind": "moe", "expert": {"ff": 18, "limit": 2.0},
             "router": {"experts": 2, "top": 3, "identity": 4, "scale": 2.5, "groups": {"count": 3, "keep": 3}},
             "shared": {"ff": 5, "limit": 0.5}}
    moe_c = {"kind": "moe", "expert": {"ff": 7, "limit": 1.5},
             "router": {"experts": 7, "top": 2, "identity": 1, "scale": 0.5, "groups": {"count": 4, "keep": 1}},
             "shared": {"ff": 11, "limit": 1.0}}
    return {"architecture": "Fipadra", "vocab": 77, "width": 72, "norm": {"eps": 1e-6},
            "layers": [layer("retention", {"heads": 1, "dim": 38, "vdim": 9, "decay": [0.98], "rot": {"base": 10000.0, "dims": 10}}, None),
                       layer("latent_attention", {"heads": 5, "dim": 10, "rot_dim": 6, "vdim": 7, "q_rank": 13, "kv_rank": 34, "scale": 0.4,
                                                  "rot": {"base": 77.0, "dims": 6}, "mask": {"size": 1}}, moe_a),
                       layer("delta", {"heads": 3, "kv_heads": 3, "dim": 37, "vdim": 9, "conv": 1}, moe_b),
                       layer("latent_attention", {"heads": 1, "dim": 6, "rot_dim": 34, "vdim": 70, "q_rank": 50, "kv_rank": 11, "scale": 0.15,
                                                  "rot": {"base": 10000.0, "dims": 34}, "mask": {"size": 500}}, DENSE),
                       layer("delta", {"heads": 6, "kv_heads": 1, "dim": 10, "vdim": 7, "conv": 5}, moe_c),
                       layer("latent_attention", {"heads": 2, "dim": 12, "rot_dim": 0, "vdim": 12, "q_rank": 8, "kv_rank": 20, "scale": 0.3},
                             None),
                       layer("retention", {"heads": 6, "dim": 10, "vdim": 7, "decay": [0.5, 0.9, 0.99, 0.999, 1.0, 0.0]}, DENSE)]}


def build(cfg, seed=1, dtype="float32", weights=None, **kw):
    from dia_tts_prune_b200.lm_config import FipadraConfig
    from dia_tts_prune_b200.lm_model import CausalLM
    w = O.random_weights(cfg, seed) if weights is None else weights
    kw.setdefault("max_tokens", 640)
    kw.setdefault("page_size", 8)
    return CausalLM(FipadraConfig.model_validate(cfg), w, dtype=dtype, device="cuda:0", **kw), w


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def close(got, ref, tol=2e-4, slack=0.0):
    got, ref = got.detach().cpu().double(), ref.double()
    err = (got - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()) + 2.0 * slack, err


def mixer_ref(kind, h, p, m, eps):
    """The float64 reference of a mixer and how far the same plain code lands from it in float32 arithmetic."""
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
@pytest.mark.parametrize("cuts", [[75], [40] + [1] * 35, [17, 15, 1, 2, 16, 3, 21], [2] * 37 + [1]])
def test_every_mixer_alone_whole_in_portions_and_decoded(make, cuts):
    cfg = make()
    model, w = build(cfg, 4)
    h = torch.randn(75, cfg["width"], generator=torch.Generator().manual_seed(6))
    for i, lc in enumerate(cfg["layers"]):
        ref, slack = mixer_ref(lc["type"], h, part(w, f"l{i}.mix."), lc["mixer"], cfg["norm"]["eps"])
        close(run_mixer(model, i, h, cuts), ref, 2e-5, slack)


@pytest.mark.parametrize("rows", [1, 3, 8, 9, 40])
def test_feed_forwards_alone_on_every_branch(rows):
    cfg = small_config()
    model, w = build(cfg, 5)
    h = torch.randn(rows, cfg["width"], generator=torch.Generator().manual_seed(rows)) * 2
    p = part(w, "l0.mlp.")
    z = h.double() @ p["up"].T
    assert (z > 0).any() and (z < 0).any()
    close(model.engine.op_ff(0, h.cuda()), O.dense_ff(h.double(), p), 2e-5)
    for i in (1, 2):
        p, f = part(w, f"l{i}.mlp."), cfg["layers"][i]["mlp"]
        g, u = h.double() @ p["e0.gate"].T, h.double() @ p["e0.up"].T
        lim = f["expert"]["limit"]
        assert (g > lim).any() and (u > lim).any() and (u < -lim).any() and (u.abs() < lim).any()
        close(model.engine.op_ff(i, h.cuda()), O.moe_ff(h.double(), p, f), 2e-5)


ROUTERS = [
    # experts, identity, top, groups, shared
    (1, 0, 1, None, False), (7, 0, 7, None, True), (60, 10, 3, (7, 2), True), (9, 3, 5, (4, 2), False), (2, 6, 4, (2, 1), True),
    (6, 2, 2, (4, 1), True), (6, 2, 4, (8, 5), True), (12, 4, 2, (2, 1), True), (5, 1, 6, (1, 1), False),
]


@pytest.mark.parametrize("experts,identity,top,groups,shared", ROUTERS)
def test_router_scores_groups_correction_identity_and_shared_gate(experts, identity, top, groups, shared):
    r = {"experts": experts, "top": top, "identity": identity, "scale": 1.75}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": 16, "limit": 1.5}, "router": r, "shared": {"ff": 8, "limit": 1.0} if shared else None}
    cfg = small_config(layers=[layer("retention", RET, mlp)])
    w = O.random_weights(cfg, 8)
    n = experts + identity
    # a correction that decides many choices, also with negative choice scores; it must not reach the weights
    w["l0.mlp.correction"] = (torch.linspace(-0.6, 0.4, n) * min(1.0, 2.0 / n)).to(torch.bfloat16).float()
    model, _ = build(cfg, weights=w)
    h = torch.randn(50, cfg["width"], generator=torch.Generator().manual_seed(experts))
    p = part(w, "l0.mlp.")
    ref = O.moe_ff(h.double(), p, mlp)
    if n > top:
        assert (O.moe_ff(h.double(), p, mlp, correction=False) - ref).abs().max() > 1e-3
        picks, wts = O.route(h.double(), p, mlp)                # the correction does not reach the weights: they sum to scale
        assert all(abs(float(x.sum()) - r["scale"]) < 1e-9 for x in wts)
    if groups and groups[1] < groups[0] and top < n and (n // groups[0] > 1 or top > groups[1]):
        assert (O.moe_ff(h.double(), p, mlp, groups=False) - ref).abs().max() > 1e-3
    if identity:
        picks, _ = O.route(h.double(), p, mlp)
        assert any(e >= experts for row in picks for e in row)     # identity experts are chosen
    close(model.engine.op_ff(0, h.cuda()), ref, 2e-5)                                      # grouped by expert
    close(torch.cat([model.engine.op_ff(0, h[i:i + 5].cuda()) for i in range(0, 50, 5)]), ref, 2e-5)   # row kernels
    if shared:                                                  # the gate number scales the shared unit alone
        ungated = dict(p, **{"shared.sg": torch.zeros_like(p["shared.sg"])})
        assert (O.moe_ff(h.double(), ungated, mlp) - ref).abs().max() > 1e-3


def test_groups_shut_out_larger_scores_elsewhere():
    """One group holds the largest choice score, another the second and third: with one group kept, the second choice
    comes from the first group although larger scores stand outside."""
    mlp = {"kind": "moe", "expert": {"ff": 8, "limit": 1.0},
           "router": {"experts": 6, "top": 2, "identity": 0, "scale": 1.0, "groups": {"count": 3, "keep": 1}}, "shared": None}
    cfg = small_config(layers=[layer("retention", RET, mlp)])
    w = O.random_weights(cfg, 9)
    D = cfg["width"]
    router = torch.zeros(6, D)
    for e, v in enumerate([4.0, -4.0, 3.0, 3.5, 0.0, -1.0]):
        router[e, 0] = v
    w["l0.mlp.router"], w["l0.mlp.correction"] = router, torch.zeros(6)
    model, _ = build(cfg, weights=w)
    h = torch.zeros(12, D)
    h[:, 0] = 1.0
    h[:, 1:] = torch.randn(12, D - 1, generator=torch.Generator().manual_seed(1)) * 0.3
    p = part(w, "l0.mlp.")
    picks, _ = O.route(h.double(), p, mlp)
    assert all(row == [0, 1] for row in picks)
    assert (O.moe_ff(h.double(), p, mlp, groups=False) - O.moe_ff(h.double(), p, mlp)).abs().max() > 1e-3
    close(model.engine.op_ff(0, h.cuda()), O.moe_ff(h.double(), p, mlp), 2e-5)
    close(model.engine.op_ff(0, h[:3].cuda()), O.moe_ff(h[:3].double(), p, mlp), 2e-5)


LATENTS = [(12, 96, 32, 32, 64, 128, 50), (16, 16, 8, 128, 24, 64, 7), (3, 100, 36, 200, 9, 220, 64), (2, 8, 2, 8, 200, 4, 65),
           (32, 40, 8, 8, 16, 48, 33), (2, 16, 64, 24, 32, 300, 40), (3, 8, 24, 8, 8, 1000, 90), (130, 8, 4, 4, 16, 20, 3),
           (4, 64, 32, 48, 80, 96, 57)]


@pytest.mark.parametrize("heads,dim,rot_dim,vdim,q_rank,kv_rank,window", LATENTS)
def test_latent_attention_with_other_shapes(heads, dim, rot_dim, vdim, q_rank, kv_rank, window):
    """Tile heights from 16 rows down, cached rows up to 256 wide on the tiled kernel; wider rows and more heads than a
    tile holds on the kernel that takes every (row, head) on its own."""
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": (dim + rot_dim) ** -0.5, "rot": {"base": 300.0, "dims": rot_dim}, "mask": {"size": window}}
    cfg = small_config(layers=[layer("latent_attention", mixer, None)])
    model, w = build(cfg, 48)
    h = torch.randn(100, cfg["width"], generator=torch.Generator().manual_seed(dim))
    ref = O.latent_attention(h.double(), part(w, "l0.mix."), mixer, cfg["norm"]["eps"])
    close(run_mixer(model, 0, h, [70] + [1] * 30), ref, 2e-5)


@pytest.mark.parametrize("kind,heads,kv_heads,dim,vdim", [("delta", 4, 2, 128, 128), ("delta", 2, 1, 200, 20), ("delta", 5, 5, 72, 130),
                                                          ("delta", 1, 1, 3, 15), ("delta", 9, 3, 32, 16), ("retention", 4, 4, 128, 128),
                                                          ("retention", 2, 2, 200, 20), ("retention", 5, 5, 72, 130),
                                                          ("retention", 1, 1, 4, 15), ("retention", 9, 9, 32, 16)])
def test_recurrences_with_other_state_shapes(kind, heads, kv_heads, dim, vdim):
    if kind == "delta":
        mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": 3}
    else:
        mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": [1.0 - 0.5 ** (h + 2) for h in range(heads)],
                 "rot": {"base": 100.0, "dims": dim - dim % 2}}
    cfg = small_config(layers=[layer(kind, mixer, None)])
    model, w = build(cfg, 49)
    h = torch.randn(50, cfg["width"], generator=torch.Generator().manual_seed(vdim))
    ref, slack = mixer_ref(kind, h, part(w, "l0.mix."), mixer, cfg["norm"]["eps"])
    close(run_mixer(model, 0, h, [33, 1, 1, 15]), ref, 2e-5, slack)


def test_rotary_layouts_are_not_interchangeable():
    """Retention pairs channel i with i + dims / 2, the attention's turned part pairs 2i with 2i + 1: the oracle with the
    other pairing differs, the product follows the right one (positions far from zero, where the angles matter)."""
    cfg = small_config(layers=[layer("retention", RET, None), layer("latent_attention", LAT, None)])
    model, w = build(cfg, 50)
    h = torch.randn(60, cfg["width"], generator=torch.Generator().manual_seed(3))
    real = O.rotate
    for i, kind in enumerate(("retention", "latent_attention")):
        p, m = part(w, f"l{i}.mix."), cfg["layers"][i]["mixer"]
        ref = O.MIXERS[kind](h.double(), p, m, 1e-5)
        try:
            O.rotate = lambda x, pos, base, dims, layout: real(x, pos, base, dims, "half" if layout == "interleaved" else "interleaved")
            assert (O.MIXERS[kind](h.double(), p, m, 1e-5) - ref).abs().max() > 1e-3
        finally:
            O.rotate = real
        close(run_mixer(model, i, h, [45] + [1] * 15), ref, 2e-5)


# ---- the whole model ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("make", [small_config, odd_config])
def test_whole_prompt_logits_and_residual_after_every_layer(make):
    cfg = make()
    model, w = build(cfg, 11)
    toks = tokens(cfg, 61, 2)
    ref, streams = O.forward(cfg, w, toks, keep_layers=True)
    got, got_streams = whole(model, "a", toks, keep_layers=True)
    assert got_streams.shape[0] == len(cfg["layers"])
    slack = (O.forward(cfg, w, toks, keep_layers=True, dtype=torch.float32)[1].double() - streams).abs().max().item()
    close(got_streams, streams, 2e-5, slack)
    close(got, ref, 2e-4, slack)
    for n in (1, 2, 3):                                         # the first tokens of a sequence
        close(whole(model, "b", toks[:n]), ref[:n], 2e-4, slack)


def test_both_sublayers_read_the_same_residual():
    """Against a sequential reading (the feed-forward sees the mixer's output) the oracle differs; the product follows the
    parallel one."""
    cfg = small_config()
    model, w = build(cfg, 10)
    toks = tokens(cfg, 33, 5)
    ref = O.forward(cfg, w, toks)
    eps = cfg["norm"]["eps"]
    x = O.rms_unit(w["embed"].double()[toks], eps) * w["embed.norm"].double()
    for i, lc in enumerate(cfg["layers"]):                      # the sequential reading, for contrast
        x = x + O.MIXERS[lc["type"]](O.rms_unit(x, eps) * w[f"l{i}.norm1"].double(), part(w, f"l{i}.mix."), lc["mixer"], eps)
        h2 = O.rms_unit(x, eps) * w[f"l{i}.norm2"].double()
        f = lc["mlp"]
        x = x + (O.dense_ff(h2, part(w, f"l{i}.mlp.")) if f["kind"] == "dense" else O.moe_ff(h2, part(w, f"l{i}.mlp."), f))
    seq = (O.rms_unit(x, eps) * w["final.norm"].double()) @ w["embed"].double().T * cfg["logit_scale"]
    assert (seq - ref).abs().max() > 1e-2
    close(whole(model, "a", toks), ref)


@pytest.mark.parametrize("make", [small_config, odd_config])
def test_prefill_then_long_token_by_token_decoding(make):
    cfg = make()
    model, w = build(cfg, 12)
    toks = tokens(cfg, 150, 3)
    ref = O.forward(cfg, w, toks)
    got = [model.run_step([{"id": "d", "tokens": toks[:9], "want": list(range(9))}])]
    for t in range(9, 150):                                     # the windows pass over decoded tokens
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
    both = model.run_step([{"id": "A", "tokens": A, "want": list(range(50))},
                           {"id": "B", "tokens": B, "want": list(range(31))}], ["A", "B"])
    assert torch.equal(both[:50], alone["A"]) and torch.equal(both[50:], alone["B"])


def test_freed_pages_slots_states_and_tails_are_used_again():
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
    # Z takes X's slot and pages - dirty with X's cached rows, matrix states and convolution tails - and starts with two
    # tokens (fewer than the convolution has taps), while Y's state stays as it is
    gz = model.run_step([{"id": "Z", "tokens": Z[:2], "want": [0, 1]}])
    assert st.sequences["Z"].slot == slot_x and set(st.sequences["Z"].pages) <= set(pages_x)
    gz1 = model.run_step([{"id": "Z", "tokens": Z[2:40], "want": list(range(38))}])
    gz2 = model.run_step([{"id": "Z", "tokens": Z[40:], "want": list(range(24))}], ["Z", "Y"])
    close(gx, ref["X"]); close(gy, ref["Y"]); close(torch.cat([gz, gz1, gz2]), ref["Z"])
    assert st.free_pages == st.n_pages and st.free_slots == 2
    from dia_tts_prune_b200.lm_state import OutOfPages
    with pytest.raises(OutOfPages):
        model.run_step([{"id": "big", "tokens": tokens(cfg, 200, 1), "want": []}])


# ---- inputs and weights made so that one thing stands out -----------------------------------------------------------------
def standout_attention(page_size, window, rot_dim=0):
    """One latent attention layer whose query path equals its key path (same down-projection, same norm, same
    up-projection; no turned part unless asked for), so that a position whose input points the way the query's input does
    gets a score far above all others."""
    mixer = {"heads": 2, "dim": 32, "rot_dim": rot_dim, "vdim": 32, "q_rank": 48, "kv_rank": 48, "scale": 0.5, "mask": {"size": window}}
    if rot_dim:
        mixer["rot"] = {"base": 10000.0, "dims": rot_dim}
    cfg = small_config(layers=[layer("latent_attention", mixer, None)])
    w = O.random_weights(cfg, 21)
    w["l0.mix.dq"], w["l0.mix.dq.norm"] = w["l0.mix.dkv"][:48], w["l0.mix.dkv.norm"]
    uq = w["l0.mix.uq"].reshape(2, 32 + rot_dim, 48).clone()
    uq[:, :32] = w["l0.mix.uk"].reshape(2, 32, 48)
    w["l0.mix.uq"] = uq.reshape(-1, 48)
    model, _ = build(cfg, weights=w, max_tokens=512, page_size=page_size)
    return cfg, w, model


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window", [1000, 130, 75])
def test_standout_key_far_away_at_page_tile_and_window_borders(decode, window):
    P = 16
    cfg, w, model = standout_attention(P, window)
    T = 300
    g = torch.Generator().manual_seed(2)
    base = torch.randn(T, 96, generator=g) * 0.3
    mark, near = torch.randn(96, generator=g) * 3, torch.randn(96, generator=g) * 2
    p, m = part(w, "l0.mix."), cfg["layers"][0]["mixer"]
    i = T - 1
    blank = base.clone()
    blank[i] = mark
    ref_blank = O.latent_attention(blank.double(), p, m, 1e-5)
    # the first token, far back among hundreds, both sides of page borders and of the 64-key tile border, the neighbour,
    # and the last key inside and the first outside the window
    for j in (0, 3, 63, 64, 127, 128, (i // P) * P, (i // P) * P - 1, i - 1, i - window + 1, i - window, i - window + 2):
        if j < 0:
            continue
        h = base.clone()
        h[j] = 2 * mark + near                                  # nearly the query's direction, a value of its own
        h[i] = mark
        ref = O.latent_attention(h.double(), p, m, 1e-5)
        carried = (ref[i] - ref_blank[i]).abs().max() > 1e-2
        assert carried == (i - j < window), j                   # the marked key carries the row exactly when it is seen
        n0 = T - 60 if decode else T
        close(run_mixer(model, 0, h, [n0] + [1] * (T - n0)), ref, 2e-5)


@pytest.mark.parametrize("cuts", [[200], [150] + [1] * 50, [3, 61, 2, 64, 70]])
def test_window_edge_moves_with_every_row_of_a_portion(cuts):
    """Every row of a portion has its own first visible key: a key made to stand out is seen by exactly the rows that are
    less than `window` tokens on."""
    window = 40
    cfg, w, model = standout_attention(8, window, rot_dim=8)
    T = 200
    g = torch.Generator().manual_seed(4)
    h = torch.randn(T, 96, generator=g) * 0.3
    mark = torch.randn(96, generator=g) * 3
    plain = h.clone()
    h[100] = 2 * mark
    h[101:] += mark * 0.5                                        # every later query leans towards the marked key
    plain[101:] += mark * 0.5
    p, m = part(w, "l0.mix."), cfg["layers"][0]["mixer"]
    ref = O.latent_attention(h.double(), p, m, 1e-5)
    gap = (O.latent_attention(plain.double(), p, m, 1e-5) - ref).abs().amax(dim=-1)
    assert gap[100 + window - 1] > 1e-2 and gap[100 + window:].max() == 0    # seen up to row 139, gone from row 140 on
    close(run_mixer(model, 0, h, cuts), ref, 2e-5)


def long_memory(kind):
    """A recurrence that forgets almost nothing, so that the first tokens still carry the read-out hundreds of tokens on."""
    if kind == "retention":
        mixer = {"heads": 2, "dim": 16, "vdim": 16, "decay": [0.9995, 1.0], "rot": {"base": 10000.0, "dims": 16}}
    else:
        mixer = {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "conv": 4}
    cfg = small_config(layers=[layer(kind, mixer, None)])
    w = O.random_weights(cfg, 23)
    if kind == "delta":
        w["l0.mix.dt_bias"] = torch.full((2,), -12.0)           # softplus ~ 0: decay ~ 1
        w["l0.mix.b"] = w["l0.mix.b"] * 0 - 0.0                 # beta = 1/2 everywhere
    model, _ = build(cfg, weights=w, max_tokens=512, page_size=16)
    return cfg, w, model


@pytest.mark.parametrize("kind", ["retention", "delta"])
@pytest.mark.parametrize("cuts", [[400], [340] + [1] * 60, [2, 14, 16, 1, 31, 64, 272]])
def test_recurrent_state_keeps_the_first_tokens_over_hundreds_of_steps(kind, cuts):
    cfg, w, model = long_memory(kind)
    h = torch.randn(400, 96, generator=torch.Generator().manual_seed(5)) * 0.5
    p, m = part(w, "l0.mix."), cfg["layers"][0]["mixer"]
    ref, slack = mixer_ref(kind, h, p, m, 1e-5)
    h2 = h.clone()
    h2[1] = h2[1] * -3.0                                        # what the second token wrote is still read at the end
    assert (O.MIXERS[kind](h2.double(), p, m, 1e-5)[-1] - ref[-1]).abs().max() > 1e-3
    close(run_mixer(model, 0, h, cuts), ref, 5e-5, slack)


def test_convolution_portions_shorter_than_equal_to_and_beyond_its_taps():
    mixer = dict(DELTA)
    cfg = small_config(layers=[layer("delta", mixer, None)])
    model, w = build(cfg, 27)
    h = torch.randn(40, 96, generator=torch.Generator().manual_seed(8))
    p = part(w, "l0.mix.")
    ref = O.gated_delta(h.double(), p, mixer, 1e-5)
    no_taps = dict(p, **{f"{n}.conv": torch.cat([torch.zeros_like(p[f"{n}.conv"][:, :-1]), p[f"{n}.conv"][:, -1:]], dim=1)
                         for n in "qkv"})
    assert (O.gated_delta(h.double(), no_taps, mixer, 1e-5) - ref).abs().max() > 1e-3    # the earlier tokens' taps matter
    for cuts in ([25] + [1] * 15, [1, 1, 1, 37], [2, 2, 36], [3, 37], [4, 36], [5, 35]):
        close(run_mixer(model, 0, h, cuts), ref, 2e-5)


# ---- precisions, replayed steps, drawn sizes ------------------------------------------------------------------------------
def wide_config():
    """Sizes the tensor-core kernel takes: every product of a 64-row step runs with bfloat16 operands."""
    lat = {"heads": 4, "dim": 32, "rot_dim": 16, "vdim": 32, "q_rank": 64, "kv_rank": 48, "scale": 0.18,
           "rot": {"base": 10000.0, "dims": 16}, "mask": {"size": 30}}
    moe = {"kind": "moe", "expert": {"ff": 32, "limit": 1.5},
           "router": {"experts": 6, "top": 2, "identity": 2, "scale": 1.5, "groups": {"count": 2, "keep": 1}},
           "shared": {"ff": 64, "limit": 1.5}}
    return small_config(width=128, vocab=256,
                        layers=[layer("delta", {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "conv": 4}, {"kind": "dense", "ff": 128}),
                                layer("latent_attention", lat, moe),
                                layer("retention", {"heads": 4, "dim": 32, "vdim": 32, "decay": [0.9, 0.95, 0.99, 0.999],
                                                    "rot": {"base": 10000.0, "dims": 32}}, moe)])


@pytest.mark.parametrize("make", [wide_config, small_config])
def test_bfloat16_products_stay_within_bfloat16_rounding_of_the_oracle(make):
    cfg = make()
    lo, w = build(cfg, 31, dtype="bfloat16")
    toks = tokens(cfg, 70, 13)
    ref = O.forward(cfg, w, toks)
    got = whole(lo, "a", toks).cpu().double()
    err = (got - ref).abs().amax(dim=-1) / ref.abs().max()
    # row by row: rounding may turn a near-tie of the router the other way in a row or two, no more
    assert (err > 6e-2).sum() <= 2 and err.median() < 2e-2, (err.max(), err.median())
    dec = torch.cat([lo.run_step([{"id": "d", "tokens": toks[:40], "want": list(range(40))}])] +
                    [lo.run_step([{"id": "d", "tokens": [t], "want": [0]}]) for t in toks[40:]]).cpu().double()
    lo.run_step([], ["d"])
    err = (dec - ref).abs().amax(dim=-1) / ref.abs().max()
    assert (err > 6e-2).sum() <= 2 and err.median() < 2e-2, (err.max(), err.median())


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
    g = torch.Generator().manual_seed(3000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))          # noqa: E731
    layers = []
    for _ in range(r(2, 5)):
        m = {"heads": r(1, 6), "dim": r(3, 40), "vdim": r(3, 40)}
        pick = r(0, 2)
        if pick == 0:
            kind = "latent_attention"
            rot_dim = 2 * r(0, 12)
            m.update(rot_dim=rot_dim, q_rank=r(3, 60), kv_rank=r(3, 60), scale=0.05 + 0.05 * r(0, 6))
            if rot_dim:
                m["rot"] = {"base": float(10 ** r(1, 6)), "dims": rot_dim}
            if r(0, 3):
                m["mask"] = {"size": r(1, 70)}
        elif pick == 1:
            kind = "delta"
            groups = [k for k in range(1, m["heads"] + 1) if m["heads"] % k == 0]
            m.update(kv_heads=groups[r(0, len(groups) - 1)], conv=r(1, 6))
        else:
            kind = "retention"
            m.update(decay=[1.0 - 2.0 ** -r(1, 10) for _ in range(m["heads"])])
            if r(0, 2):
                m["rot"] = {"base": float(10 ** r(1, 6)), "dims": 2 * r(0, m["dim"] // 2)}
        pick = r(0, 2)
        if pick == 0:
            mlp = None
        elif pick == 1:
            mlp = {"kind": "dense", "ff": r(5, 70)}
        else:
            count = r(1, 4)
            per = r(1, 4)
            n = count * per
            identity = r(0, n - 1)
            keep = r(1, count)
            router = {"experts": n - identity, "identity": identity, "top": r(1, keep * per), "scale": 0.5 * r(1, 5)}
            if r(0, 3):
                router["groups"] = {"count": count, "keep": keep}
            else:
                router["top"] = r(1, n)
            mlp = {"kind": "moe", "expert": {"ff": r(3, 30), "limit": 0.5 * r(1, 14)}, "router": router,
                   "shared": {"ff": r(3, 40), "limit": 0.5 * r(1, 14)} if r(0, 1) else None}
        layers.append(layer(kind, m, mlp))
    return {"architecture": "Fipadra", "vocab": r(20, 200), "width": 2 * r(8, 60), "norm": {"eps": 10.0 ** -r(4, 7)},
            "logit_scale": 0.25 * r(1, 8), "layers": layers}


@pytest.mark.parametrize("seed", range(10))
def test_drawn_configurations_whole_portioned_and_decoded(seed):
    cfg = drawn_config(seed)
    model, w = build(cfg, 40 + seed, page_size=(4, 8, 16)[seed % 3])
    toks = tokens(cfg, 75, seed)
    ref = O.forward(cfg, w, toks)
    slack = (O.forward(cfg, w, toks, dtype=torch.float32).double() - ref).abs().max().item()
    close(whole(model, "a", toks), ref, 2e-4, slack)
    got, at = [], 0
    for n in (7, 2, 19, 1, 1, 12):
        got.append(model.run_step([{"id": "p", "tokens": toks[at:at + n], "want": list(range(n))}]))
        at += n
    got += [model.run_step([{"id": "p", "tokens": [t], "want": [0]}]) for t in toks[at:]]
    model.run_step([], ["p"])
    close(torch.cat(got), ref, 2e-4, slack)


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
