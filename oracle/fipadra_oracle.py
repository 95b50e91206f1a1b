"""Plain, slow restatement of the Fipadra decoder-only language model (test infrastructure only).

Torch on the CPU, one function per mechanism, whole sequences at once, no cache and no carried state: every position
is recomputed from the start of its sequence, and every recurrence is an explicit loop over time.  Nothing here is
imported by the product path and nothing of the product path is imported here.  The arithmetic type is the type of the
tensors handed in (float64 gives a reference whose own rounding is negligible).

Notation: matrices are ``[out, in]`` and applied as ``W @ x``; ``p`` maps the short tensor names of one mixer or
feed-forward (``q.conv``, ``dkv.norm``, ``e3.gate``, ``shared.sg`` ...) to tensors, ``m`` / ``f`` is the matching
dictionary of the configuration.

The model: x = rms(embed[token]) w_e; every layer adds mixer(rms(x) w_1) + ff(rms(x) w_2), both read from the same x;
logits = logit_scale * embed @ (rms(x) w_f).
"""

from __future__ import annotations

import math

import torch


# ---- elementwise pieces ---------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def relu_squared(z):
    r = torch.clamp(z, min=0.0)
    return r * r


def clamped_glu(g, u, limit):
    """min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, -limit, limit) + 1)."""
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, min=-limit, max=limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)


def causal_conv(u, w):
    """y[t, c] = sum_j w[c, j] u[t - (taps - 1) + j, c], zeros before the start; the last tap is the current token's."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                y[t] = y[t] + w[:, j] * u[s]
    return y


def rotary_frequencies(base, dims, dtype=torch.float64):
    return torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=dtype)


def rotate(x, positions, base, dims, layout):
    """Turns the first ``dims`` channels of the last axis of x [T, ..., n] by position x base^(-2i/dims).  ``layout``
    "interleaved": channel 2i pairs with 2i + 1; "half": channel i pairs with i + dims / 2.  The other channels pass."""
    if dims == 0:
        return x
    f = rotary_frequencies(base, dims, x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]                 # [T, dims / 2]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    cs, sn = torch.cos(ang), torch.sin(ang)
    out = x.clone()
    if layout == "interleaved":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * cs - b * sn
        out[..., 1:dims:2] = b * cs + a * sn
    else:
        half = dims // 2
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * cs - b * sn
        out[..., half:dims] = b * cs + a * sn
    return out


# ---- mixers -----------------------------------------------------------------------------------------------------------
def gated_delta(h, p, m, eps):
    """Delta rule with one decay per head and token.  q, k (kv_heads x dim) and v (heads x vdim) pass a short causal
    convolution and silu; q, k become unit vectors per head (q also x dim^-1/2); per head
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;  then o / rms(o) x w x silu(gate), output projection."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ p["q"].T, p["q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ p["k"].T, p["k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ p["v"].T, p["v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ p["b"].T)                                # [T, H]
    decay = torch.exp(-torch.exp(p["A_log"]) * torch.nn.functional.softplus(h @ p["a"].T + p["dt_bias"]))
    out = torch.zeros((T, H, dv), dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros((d, dv), dtype=h.dtype)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hh] = S.T @ q[t, g]
    out = rms_unit(out, eps) * p["norm"]
    return (out.reshape(T, H * dv) * silu(h @ p["g"].T)) @ p["o"].T


def visible(i, j, window):
    """Key j is seen from query i when it is not in the future and less than ``window`` tokens back (None: all)."""
    return 0 <= i - j and (window is None or i - j < window)


def latent_attention(h, p, m, eps, positions=None):
    """Softmax attention whose per-head keys and values are up-projections of one normed latent per position, plus one
    rotated key part shared by all heads; queries through a normed latent of their own, laid out per head as
    [dim plain | rot_dim rotated]; a sliding window; output projection."""
    T = h.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    window = m["mask"]["size"] if m.get("mask") else None
    cq = rms_unit(h @ p["dq"].T, eps) * p["dq.norm"]
    q = (cq @ p["uq"].T).reshape(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], pos, rot["base"], rot["dims"], "interleaved")
    ckv = h @ p["dkv"].T
    c = rms_unit(ckv[:, :R], eps) * p["dkv.norm"]
    k_rot = rotate(ckv[:, R:], pos, rot["base"], rot["dims"], "interleaved")    # [T, dr], one for all heads
    k_plain = (c @ p["uk"].T).reshape(T, H, d)
    v = (c @ p["uv"].T).reshape(T, H, dv)
    gap = pos[:, None] - pos[None, :]                                  # the rule of `visible`, for all pairs at once
    seen = (gap >= 0) & (gap < (window if window is not None else T + 1))
    out = torch.zeros((T, H, dv), dtype=h.dtype)
    for hh in range(H):
        s = (q_plain[:, hh] @ k_plain[:, hh].T + q_rot[:, hh] @ k_rot.T) * m["scale"]
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        out[:, hh] = torch.softmax(s, dim=-1) @ v[:, hh]
    return out.reshape(T, H * dv) @ p["o"].T


def retention(h, p, m, eps, positions=None):
    """Linear attention with a fixed decay per head, no softmax and no denominator: q, k turn with the position
    ("half" pairs), k x dim^-1/2;  S_t = decay S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;  o / rms(o) per head, x silu(gate),
    output projection."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T) if positions is None else positions
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    q = rotate((h @ p["q"].T).reshape(T, H, d), pos, rot["base"], rot["dims"], "half")
    k = rotate((h @ p["k"].T).reshape(T, H, d), pos, rot["base"], rot["dims"], "half") * d ** -0.5
    v = (h @ p["v"].T).reshape(T, H, dv)
    out = torch.zeros((T, H, dv), dtype=h.dtype)
    for hh in range(H):
        S = torch.zeros((d, dv), dtype=h.dtype)
        for t in range(T):
            S = float(m["decay"][hh]) * S + torch.outer(k[t, hh], v[t, hh])
            out[t, hh] = S.T @ q[t, hh]
    out = rms_unit(out, eps)
    return (out.reshape(T, H * dv) * silu(h @ p["g"].T)) @ p["o"].T


# ---- feed-forwards ------------------------------------------------------------------------------------------------------
def dense_ff(h, p):
    return relu_squared(h @ p["up"].T) @ p["down"].T


def gated_unit(h, p, prefix, limit):
    return clamped_glu(h @ p[prefix + "gate"].T, h @ p[prefix + "up"].T, limit) @ p[prefix + "down"].T


def route(h, p, f, correction=True, groups=True):
    """Per token the chosen router outputs and their weights.  Scores = softmax over ALL router outputs (experts and
    identity experts); the choice is made on score + correction, inside the `keep` groups of neighbours whose largest
    choice score is largest; weights = the chosen scores (without the correction) / their sum x scale.  Ties go to the
    lower index.  ``correction`` / ``groups`` False leave that part out (what a test compares against)."""
    r = f["router"]
    n = r["experts"] + r.get("identity", 0)
    z = h @ p["router"].T
    s = torch.softmax(z, dim=-1)
    choice = s + p["correction"] if (correction and "correction" in p) else s.clone()
    gr = r.get("groups")
    picks, weights = [], []
    for t in range(h.shape[0]):
        allowed = [True] * n
        if groups and gr and gr["count"] > 1:
            size = n // gr["count"]
            best = sorted(range(gr["count"]), key=lambda g: (-float(choice[t, g * size:(g + 1) * size].max()), g))[:gr["keep"]]
            allowed = [(e // size) in best for e in range(n)]
        order = sorted((e for e in range(n) if allowed[e]), key=lambda e: (-float(choice[t, e]), e))[:r["top"]]
        w = s[t, order]
        picks.append(order)
        weights.append(w / (w.sum() + 1e-20) * r.get("scale", 1.0))
    return picks, weights


def moe_ff(h, p, f, correction=True, groups=True):
    """Weighted sum of the chosen experts (an identity expert returns its input), plus the shared unit x sigmoid(w_sg . h)."""
    picks, weights = route(h, p, f, correction, groups)
    E = f["router"]["experts"]
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        ht = h[t:t + 1]
        for e, w in zip(picks[t], weights[t]):
            y[t] = y[t] + w * (ht[0] if e >= E else gated_unit(ht, p, f"e{e}.", f["expert"]["limit"])[0])
    if f.get("shared"):
        y = y + torch.sigmoid(h @ p["shared.sg"].T) * gated_unit(h, p, "shared.", f["shared"]["limit"])
    return y


# ---- the model --------------------------------------------------------------------------------------------------------
def sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


MIXERS = {"delta": gated_delta, "latent_attention": latent_attention, "retention": retention}


def forward(cfg: dict, w: dict, tokens, keep_layers: bool = False, dtype=torch.float64):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    w = {k: v.to(dtype) for k, v in w.items()}
    x = rms_unit(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], eps) * w["embed.norm"]
    kept = []
    for i, lc in enumerate(cfg["layers"]):
        y = MIXERS[lc["type"]](rms_unit(x, eps) * w[f"l{i}.norm1"], sub(w, f"l{i}.mix."), lc["mixer"], eps)
        f = lc.get("mlp")
        if f:
            h2 = rms_unit(x, eps) * w[f"l{i}.norm2"]
            y = y + (dense_ff(h2, sub(w, f"l{i}.mlp.")) if f["kind"] == "dense" else moe_ff(h2, sub(w, f"l{i}.mlp."), f))
        x = x + y
        kept.append(x)
    logits = (rms_unit(x, eps) * w["final.norm"]) @ w["embed"].T * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(kept)) if keep_layers else logits


def greedy(cfg: dict, w: dict, prompt, n_new: int):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


def random_weights(cfg: dict, seed: int, spread: float = 1.0) -> dict:
    """Random float32 tensors that bfloat16 holds exactly, under the checkpoint's names."""
    g = torch.Generator().manual_seed(seed)
    D, w = cfg["width"], {}

    def mat(n_out, n_in, gain=1.0):
        return (torch.randn((n_out, n_in), generator=g) * (gain * spread / math.sqrt(n_in))).to(torch.bfloat16).float()

    def vec(n, mean=0.0, dev=0.1):
        return (mean + dev * torch.randn((n,), generator=g)).to(torch.bfloat16).float()

    def unit(prefix, ff):
        w[prefix + "gate"], w[prefix + "up"], w[prefix + "down"] = mat(ff, D, 1.5), mat(ff, D, 1.5), mat(D, ff)

    w["embed"] = (torch.randn((cfg["vocab"], D), generator=g) * spread).to(torch.bfloat16).float()
    w["embed.norm"], w["final.norm"] = vec(D, 1.0), vec(D, 1.0)
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        w[p + "norm1"] = vec(D, 1.0)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if lc["type"] == "delta":
            G = m.get("kv_heads") or H
            for name, n in (("q", G * d), ("k", G * d), ("v", H * dv)):
                w[p + "mix." + name] = mat(n, D, 1.5)
                w[p + f"mix.{name}.conv"] = (torch.randn((n, m["conv"]), generator=g) * 0.7).to(torch.bfloat16).float()
            w[p + "mix.b"], w[p + "mix.a"] = mat(H, D, 2.0), mat(H, D, 2.0)
            w[p + "mix.A_log"], w[p + "mix.dt_bias"] = vec(H, -0.5, 0.7), vec(H, -1.0, 1.0)
            w[p + "mix.norm"], w[p + "mix.g"] = vec(dv, 1.0), mat(H * dv, D, 1.5)
        elif lc["type"] == "latent_attention":
            dr = m.get("rot_dim", 0)
            w[p + "mix.dq"], w[p + "mix.dq.norm"] = mat(m["q_rank"], D), vec(m["q_rank"], 1.0)
            w[p + "mix.uq"] = mat(H * (d + dr), m["q_rank"], 2.0)
            w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(m["kv_rank"] + dr, D, 1.5), vec(m["kv_rank"], 1.0)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * d, m["kv_rank"], 2.0), mat(H * dv, m["kv_rank"])
        else:
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * d, D, 1.5), mat(H * d, D, 1.5), mat(H * dv, D)
            w[p + "mix.g"] = mat(H * dv, D, 1.5)
        w[p + "mix.o"] = mat(D, H * dv)
        f = lc.get("mlp")
        if f:
            w[p + "norm2"] = vec(D, 1.0)
            if f["kind"] == "dense":
                w[p + "mlp.up"], w[p + "mlp.down"] = mat(f["ff"], D, 1.5), mat(D, f["ff"])
            else:
                r = f["router"]
                n = r["experts"] + r.get("identity", 0)
                for e in range(r["experts"]):
                    unit(p + f"mlp.e{e}.", f["expert"]["ff"])
                w[p + "mlp.router"], w[p + "mlp.correction"] = mat(n, D, 3.0), vec(n, 0.0, 0.3 / n)
                if f.get("shared"):
                    unit(p + "mlp.shared.", f["shared"]["ff"])
                    w[p + "mlp.shared.sg"] = mat(1, D, 2.0)
    return w
