"""Seeded synthetic weights and transcripts (there is no network for checkpoints).

The weight recipe is fixed here and shared by the oracle runs
that produced tests/golden/ and by every GPU test / bench run: iterate the
parameters in ``named_parameters()`` order with ONE seeded CPU generator,
RMSNorm weights = 1, embeddings ~ N(0,1), dense kernels ~ N(0, fan_in^-1/2),
then round every non-norm tensor to a bf16-representable fp32 value - so the
bf16 weight stream the kernels read holds exactly the oracle's numbers.
"""

from __future__ import annotations

import hashlib

import torch


def is_dense_kernel(name: str) -> bool:
    """True for DenseGeneral kernels (the tensors that may be stored bf16); norms and embeddings stay fp32."""
    return name.endswith(("_proj.weight", "mlp.wi_fused.weight", "mlp.wo.weight", "logits_dense.weight"))


def cast_dense_kernels_(model, dtype) -> None:
    """Store every DenseGeneral kernel of ``model`` in ``dtype`` (what Dia(config, "bfloat16") does)."""
    for n, p in model.named_parameters():
        if is_dense_kernel(n):
            p.data = p.data.to(dtype)


def fan_in_of(name: str, shape) -> int:
    # o_proj kernels contract (heads, head_dim); every other kernel contracts axis 0
    return int(shape[0]) * int(shape[1]) if "o_proj" in name else int(shape[0])


@torch.no_grad()
def init_synthetic_(named_params, seed: int = 1234) -> None:
    """In-place init of an iterable of (name, fp32 CPU tensor) in the given order."""
    g = torch.Generator().manual_seed(seed)
    for name, p in named_params:
        if "norm" in name:
            p.fill_(1.0)
            continue
        if "embedding" in name:
            p.normal_(0.0, 1.0, generator=g)
        else:
            p.normal_(0.0, fan_in_of(name, p.shape) ** -0.5, generator=g)
        p.copy_(p.to(torch.bfloat16).to(torch.float32))


def synthetic_state_dict(shapes: dict, seed: int = 1234) -> dict:
    """``shapes``: ordered name -> shape mapping (named_parameters order)."""
    sd = {n: torch.empty(s, dtype=torch.float32) for n, s in shapes.items()}
    init_synthetic_(sd.items(), seed)
    return sd


def weights_fingerprint(sd: dict, names=None) -> str:
    """sha256 over the bf16 bit patterns of a few tensors - lets a GPU box
    verify it regenerated the very weights the golden fixtures were made with."""
    h = hashlib.sha256()
    for n in (names or sorted(sd)):
        t = sd[n].detach().to("cpu", torch.float32).contiguous()
        h.update(n.encode())
        h.update(t.to(torch.bfloat16).view(torch.int16).numpy().tobytes())
    return h.hexdigest()


def synthetic_transcript(i: int, min_bytes: int = 60, max_bytes: int = 200) -> str:
    """Deterministic alternating [S1]/[S2] dialogue of 60-200 bytes (config 5)."""
    words = ("dia is an open weights text to dialogue model you get full control over scripts and voices "
             "the quick brown fox jumps over the lazy dog while rain keeps falling on the quiet harbor town "
             "please remember to bring the blue notebook when we meet at the station tomorrow morning").split()
    state = (i * 2654435761 + 12345) & 0xFFFFFFFF

    def nxt():
        nonlocal state
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        return state >> 8

    target = min_bytes + nxt() % (max_bytes - 12 - min_bytes + 1)      # a word adds at most 11 bytes
    out, spk, left = "[S1]", 1, 4 + nxt() % 6
    while len(out.encode()) < target:
        if left == 0:
            spk = 3 - spk
            out += f". [S{spk}]"
            left = 4 + nxt() % 6
        out += " " + words[nxt() % len(words)]
        left -= 1
    return out + "."


DEFAULT_TRANSCRIPT = ("[S1] Dia is an open weights text to dialogue model. "
                      "[S2] You get full control over scripts and voices. [S1]")


# ---- decoder-only language models: made-up configurations and random weights (benchmarks, smoke runs) ----------------
def pubopel_config(width: int, layers: int, heads: int, kv_heads: int, dim: int, experts: int, top: int, expert_ff: int,
                   shared_ff: int | None, vocab: int, window: int | None = None, keep_first: int = 0, taps: int = 4,
                   softcap: float | None = 30.0) -> dict:
    """A Pubopel ``config.json`` as a dictionary: ``layers`` equal layers of the given sizes."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": softcap,
             "mask": {"size": window, "keep_first": keep_first} if window else None}
    mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top},
           "shared": {"ff": shared_ff} if shared_ff else None}
    return {"architecture": "Pubopel", "vocab": vocab, "width": width, "canon": {"taps": taps}, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": dict(mixer), "mlp": dict(mlp)} for _ in range(layers)]}


def pubopel_weights(cfg: dict, seed: int = 1234, device="cpu") -> dict:
    """Random bfloat16 tensors under the checkpoint's names: matrices ~ N(0, 1 / fan_in), norms near the identity."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(n, k):
        return (torch.randn((n, k), generator=g, device=device) * k ** -0.5).to(torch.bfloat16)

    def vec(n, mean, spread):
        return (mean + spread * torch.randn((n,), generator=g, device=device)).to(torch.bfloat16)

    w = {"embed": (torch.randn((V, D), generator=g, device=device)).to(torch.bfloat16), "head": mat(V, D)}

    def norm(name):
        w[name], w[name + ".b"] = vec(D, 1.0, 0.05), vec(D, 0.0, 0.02)
        w[name + ".alpha"] = torch.tensor(0.7, dtype=torch.bfloat16, device=device)

    norm("final.norm")
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        nq, nk = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
        norm(p + "norm1"); norm(p + "norm1b")
        w[p + "canon1"] = (0.2 * torch.randn((D, cfg["canon"]["taps"]), generator=g, device=device)).to(torch.bfloat16)
        w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.o"] = mat(nq, D), mat(nk, D), mat(D, nq)
        w[p + "mix.q.norm"], w[p + "mix.k.norm"] = vec(nq, 1.0, 0.05), vec(nk, 1.0, 0.05)
        w[p + "mix.temp"], w[p + "mix.sink"] = vec(m["heads"], 1.0, 0.1), vec(m["heads"], 0.0, 0.5)
        if lc.get("mlp"):
            f = lc["mlp"]
            norm(p + "norm2"); norm(p + "norm2b")
            w[p + "canon2"] = (0.2 * torch.randn((D, cfg["canon"]["taps"]), generator=g, device=device)).to(torch.bfloat16)
            w[p + "mlp.router"] = mat(f["router"]["experts"], D)
            for e in range(f["router"]["experts"]):
                w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"] = mat(f["expert"]["ff"], D), mat(f["expert"]["ff"], D)
                w[p + f"mlp.e{e}.down"] = mat(D, f["expert"]["ff"])
            if f.get("shared"):
                sf = f["shared"]["ff"]
                w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"], w[p + "mlp.shared.down"] = mat(sf, D), mat(sf, D), mat(D, sf)
    return w


def kupelix_config(width: int, kinds: list[str], heads: int, kv_heads: int, dim: int, vdim: int, ff: int, vocab: int, taps: int = 4,
                   loop: dict | None = None) -> dict:
    """A Kupelix ``config.json`` as a dictionary: one layer per entry of ``kinds`` (``attention`` / ``hgrn2`` /
    ``channel_delta``), all with the given head sizes and a dense feed-forward of ``ff`` hidden units."""
    layers = []
    for kind in kinds:
        m = {"heads": heads, "dim": dim, "vdim": vdim}
        if kind == "attention":
            m.update(kv_heads=kv_heads, scale=dim ** -0.5,
                     rot={"base": 500000.0, "dims": dim // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}})
        elif kind == "channel_delta":
            m.update(kv_heads=heads, conv=taps)
        layers.append({"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff}})
    cfg = {"architecture": "Kupelix", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "logit_scale": 1.0, "layers": layers}
    if loop:
        cfg["loop"] = dict(loop)
    return cfg


def kupelix_weights(cfg: dict, seed: int = 1234, device="cpu", rank: int = 64) -> dict:
    """Random bfloat16 tensors under the checkpoint's names: matrices ~ N(0, 1 / fan_in), norms near the identity, gates
    and decays in their working range."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(n, k, s=1.0):
        return (torch.randn((n, k), generator=g, device=device) * (s * k ** -0.5)).to(torch.bfloat16)

    def vec(n, mean, spread):
        return (mean + spread * torch.randn((n,), generator=g, device=device)).to(torch.bfloat16)

    w = {"embed": torch.randn((V, D), generator=g, device=device).to(torch.bfloat16), "head": mat(V, D),
         "final.norm": vec(D, 1.0, 0.05), "final.norm.b": vec(D, 0.0, 0.02)}
    if cfg.get("loop"):
        w["loop.in"] = mat(D, 2 * D, 1.4)
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        G = m.get("kv_heads") or H
        w[p + "norm1"], w[p + "norm1.b"] = vec(D, 1.0, 0.05), vec(D, 0.0, 0.02)
        if lc["type"] == "attention":
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"] = mat(H * d, D), mat(G * d, D), mat(G * dv, D), mat(H, D)
            w[p + "mix.q.b"], w[p + "mix.k.b"], w[p + "mix.v.b"] = vec(H * d, 0.0, 0.1), vec(G * d, 0.0, 0.1), vec(G * dv, 0.0, 0.1)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = vec(d, 1.0, 0.05), vec(d, 1.0, 0.05)
            w[p + "mix.talk"] = (torch.eye(H, device=device) + 0.3 * H ** -0.5 * torch.randn((H, H), generator=g, device=device)).to(torch.bfloat16)
            w[p + "mix.sink"] = vec(H, 0.0, 0.5)
        elif lc["type"] == "hgrn2":
            w[p + "mix.q"], w[p + "mix.f"], w[p + "mix.v"] = mat(H * d, D), mat(H * d, D), mat(H * dv, D)
            w[p + "mix.f.b"] = vec(H * d, 1.0, 0.5)
            w[p + "mix.lower"] = (0.9 * torch.rand((H * d,), generator=g, device=device)).to(torch.bfloat16)
            w[p + "mix.norm"] = vec(dv, 1.0, 0.05)
        else:
            taps = m["conv"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.b"] = mat(G * d, D), mat(G * d, D), mat(H * dv, D), mat(H, D)
            for n, c in (("q", G * d), ("k", G * d), ("v", H * dv)):
                w[p + f"mix.{n}.conv"] = (0.5 * torch.randn((c, taps), generator=g, device=device)).to(torch.bfloat16)
            w[p + "mix.A_log"] = torch.log(0.3 + 3.0 * torch.rand((H,), generator=g, device=device)).to(torch.bfloat16)
            w[p + "mix.a1"], w[p + "mix.a2"], w[p + "mix.dt_bias"] = mat(rank, D), mat(H * d, rank), vec(H * d, -1.0, 0.5)
            w[p + "mix.g1"], w[p + "mix.g2"] = mat(rank, D), mat(H * dv, rank)
            w[p + "mix.norm"] = vec(dv, 1.0, 0.05)
        w[p + "mix.o"] = mat(D, H * dv)
        if lc.get("mlp"):
            F = lc["mlp"]["ff"]
            w[p + "mlp.up"], w[p + "mlp.down"], w[p + "mlp.act"] = mat(F, D), mat(D, F), vec(2, 0.3, 0.3)
    return w


def luketar_config(width: int, kinds: list[str], heads: int, dim: int, vdim: int, vocab: int, q_rank: int = 0, kv_rank: int = 0,
                   ff: int = 0, experts: int = 0, top: int = 0, expert_ff: int = 0, shared_ff: int = 0, streams: int | None = None,
                   repeat_last: bool = False) -> dict:
    """A Luketar ``config.json`` as a dictionary: one layer per entry of ``kinds`` (``latent_attention`` / ``mlstm``), the
    first with a dense gated unit of ``ff`` hidden units, the others with ``experts`` routed units (a dense one when
    ``experts`` is 0); ``repeat_last`` appends a layer that runs with the last layer's weights."""
    layers = []
    for n, kind in enumerate(kinds):
        m = {"heads": heads, "dim": dim, "vdim": vdim}
        if kind == "latent_attention":
            m.update(q_rank=q_rank, kv_rank=kv_rank, scale=dim ** -0.5)
        else:
            m.update(gate_cap=15.0)
        if experts and n > 0:
            mlp = {"kind": "moe", "expert": {"ff": expert_ff, "limit": 7.0}, "router": {"experts": experts, "top": top},
                   "shared": {"ff": shared_ff, "limit": 7.0} if shared_ff else None}
        else:
            mlp = {"kind": "dense", "ff": ff, "limit": 7.0} if ff else None
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    if repeat_last:
        layers.append(dict(layers[-1], weights_of=len(layers) - 1))
    cfg = {"architecture": "Luketar", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
           "layers": layers}
    if streams:
        cfg["streams"] = streams
    return cfg


def luketar_weights(cfg: dict, seed: int = 1234, device="cpu") -> dict:
    """Random bfloat16 tensors under the checkpoint's names: matrices ~ N(0, 1 / fan_in), norms and stream weights near
    the identity, forget gates mostly open."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    D, V, s = cfg["width"], cfg["vocab"], cfg.get("streams")

    def mat(n, k, gain=1.0):
        return (torch.randn((n, k), generator=g, device=device) * (gain * k ** -0.5)).to(torch.bfloat16)

    def vec(n, mean, spread):
        return (mean + spread * torch.randn((n,), generator=g, device=device)).to(torch.bfloat16)

    def unit(prefix, ff):
        w[prefix + "gate"], w[prefix + "up"], w[prefix + "down"] = mat(ff, D), mat(ff, D), mat(D, ff)

    w = {"embed": torch.randn((V, D), generator=g, device=device).to(torch.bfloat16), "final.norm": vec(D, 1.0, 0.05)}
    for i, lc in enumerate(cfg["layers"]):
        if lc.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", lc["mixer"]
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        w[p + "norm1"] = vec(D, 1.0, 0.05)
        if lc["type"] == "latent_attention":
            rq, rk = m["q_rank"], m["kv_rank"]
            w[p + "mix.dq"], w[p + "mix.dq.norm"], w[p + "mix.uq"] = mat(rq, D), vec(rq, 1.0, 0.05), mat(H * d, rq)
            w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(rk, D), vec(rk, 1.0, 0.05)
            w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.sink"] = mat(H * d, rk), mat(H * dv, rk), vec(H, 0.0, 0.5)
        else:
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * d, D), mat(H * d, D), mat(H * dv, D)
            w[p + "mix.i"], w[p + "mix.f"] = mat(H, D), mat(H, D)
            w[p + "mix.i.b"], w[p + "mix.f.b"], w[p + "mix.norm"] = vec(H, 0.0, 0.5), vec(H, 3.0, 1.0), vec(H * dv, 1.0, 0.05)
        w[p + "mix.g"], w[p + "mix.o"] = mat(H * dv, D), mat(D, H * dv)
        f = lc.get("mlp")
        if f:
            w[p + "norm2"] = vec(D, 1.0, 0.05)
            if f["kind"] == "dense":
                unit(p + "mlp.", f["ff"])
            else:
                for e in range(f["router"]["experts"]):
                    unit(p + f"mlp.e{e}.", f["expert"]["ff"])
                w[p + "mlp.router"], w[p + "mlp.router.b"] = mat(f["router"]["experts"], D), vec(f["router"]["experts"], 0.0, 0.2)
                if f.get("shared"):
                    unit(p + "mlp.shared.", f["shared"]["ff"])
        if s:
            for q in (1, 2) if f else (1,):
                w[p + f"hc{q}.in"], w[p + f"hc{q}.out"] = vec(s, 1.0 / s, 0.05), vec(s, 1.0, 0.1)
                w[p + f"hc{q}.mix"] = (torch.eye(s, device=device) + 0.1 * torch.randn((s, s), generator=g, device=device)).to(torch.bfloat16)
    return w


def fipadra_config(width: int, kinds: list[str], heads: int, dim: int, vdim: int, vocab: int, kv_heads: int = 0, q_rank: int = 0,
                   kv_rank: int = 0, rot_dim: int = 0, window: int = 0, taps: int = 4, ff: int = 0, experts: int = 0, top: int = 0,
                   identity: int = 0, groups: tuple[int, int] | None = None, expert_ff: int = 0, shared_ff: int = 0,
                   logit_scale: float = 1.0) -> dict:
    """A Fipadra ``config.json`` as a dictionary: one layer per entry of ``kinds`` (``delta`` / ``latent_attention`` /
    ``retention``); even layers get a dense unit of ``ff`` hidden units, odd ones ``experts`` routed units with ``identity``
    identity experts (a dense unit when ``experts`` is 0)."""
    layers = []
    for n, kind in enumerate(kinds):
        m = {"heads": heads, "dim": dim, "vdim": vdim}
        if kind == "delta":
            m.update(kv_heads=kv_heads or heads, conv=taps)
        elif kind == "latent_attention":
            m.update(q_rank=q_rank, kv_rank=kv_rank, rot_dim=rot_dim, scale=(dim + rot_dim) ** -0.5,
                     rot={"base": 10000.0, "dims": rot_dim})
            if window:
                m["mask"] = {"size": window}
        else:
            m.update(decay=[1.0 - 2.0 ** (-5.0 - 6.0 * h / max(heads - 1, 1)) for h in range(heads)],
                     rot={"base": 10000.0, "dims": dim})
        if experts and n % 2 == 1:
            router = {"experts": experts, "top": top, "identity": identity, "scale": 1.5}
            if groups:
                router["groups"] = {"count": groups[0], "keep": groups[1]}
            mlp = {"kind": "moe", "expert": {"ff": expert_ff, "limit": 7.0}, "router": router,
                   "shared": {"ff": shared_ff, "limit": 7.0} if shared_ff else None}
        else:
            mlp = {"kind": "dense", "ff": ff} if ff else None
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Fipadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": logit_scale,
            "layers": layers}


def fipadra_weights(cfg: dict, seed: int = 1234, device="cpu") -> dict:
    """Random bfloat16 tensors under the checkpoint's names: matrices ~ N(0, 1 / fan_in), norm weights near one, decays of
    the delta rule mostly close to one."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(n, k, gain=1.0):
        return (torch.randn((n, k), generator=g, device=device) * (gain * k ** -0.5)).to(torch.bfloat16)

    def vec(n, mean, spread):
        return (mean + spread * torch.randn((n,), generator=g, device=device)).to(torch.bfloat16)

    def unit(prefix, ff):
        w[prefix + "gate"], w[prefix + "up"], w[prefix + "down"] = mat(ff, D), mat(ff, D), mat(D, ff)

    w = {"embed": torch.randn((V, D), generator=g, device=device).to(torch.bfloat16), "embed.norm": vec(D, 1.0, 0.05),
         "final.norm": vec(D, 1.0, 0.05)}
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        w[p + "norm1"] = vec(D, 1.0, 0.05)
        if lc["type"] == "delta":
            G, taps = m.get("kv_heads") or H, m["conv"]
            for name, n in (("q", G * d), ("k", G * d), ("v", H * dv)):
                w[p + "mix." + name] = mat(n, D)
                w[p + f"mix.{name}.conv"] = (torch.randn((n, taps), generator=g, device=device) * taps ** -0.5).to(torch.bfloat16)
            w[p + "mix.b"], w[p + "mix.a"] = mat(H, D), mat(H, D)
            w[p + "mix.A_log"], w[p + "mix.dt_bias"] = vec(H, -1.0, 0.5), vec(H, -2.0, 1.0)
            w[p + "mix.norm"], w[p + "mix.g"] = vec(dv, 1.0, 0.05), mat(H * dv, D)
        elif lc["type"] == "latent_attention":
            rq, rk, dr = m["q_rank"], m["kv_rank"], m.get("rot_dim", 0)
            w[p + "mix.dq"], w[p + "mix.dq.norm"], w[p + "mix.uq"] = mat(rq, D), vec(rq, 1.0, 0.05), mat(H * (d + dr), rq)
            w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(rk + dr, D), vec(rk, 1.0, 0.05)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * d, rk), mat(H * dv, rk)
        else:
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * d, D), mat(H * d, D), mat(H * dv, D)
            w[p + "mix.g"] = mat(H * dv, D)
        w[p + "mix.o"] = mat(D, H * dv)
        f = lc.get("mlp")
        if f:
            w[p + "norm2"] = vec(D, 1.0, 0.05)
            if f["kind"] == "dense":
                w[p + "mlp.up"], w[p + "mlp.down"] = mat(f["ff"], D), mat(D, f["ff"])
            else:
                r = f["router"]
                n = r["experts"] + r.get("identity", 0)
                for e in range(r["experts"]):
                    unit(p + f"mlp.e{e}.", f["expert"]["ff"])
                w[p + "mlp.router"], w[p + "mlp.correction"] = mat(n, D), vec(n, 0.0, 0.05)
                if f.get("shared"):
                    unit(p + "mlp.shared.", f["shared"]["ff"])
                    w[p + "mlp.shared.sg"] = mat(1, D)
    return w
