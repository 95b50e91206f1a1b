"""Plain, slow restatement of the Luketar decoder-only language model (test infrastructure only).

Torch on the CPU, one function per mechanism, whole sequences at once, no cache and no carried state: every position
is recomputed from the start of its sequence, and the recurrence is an explicit loop over time.  Nothing here is
imported by the product path and nothing of the product path is imported here.  The arithmetic type is the type of the
tensors handed in (float64 gives a reference whose own rounding is negligible).

Notation: matrices are ``[out, in]`` and applied as ``W @ x``; ``p`` maps the short tensor names of one mixer or
feed-forward (``dq``, ``dq.norm``, ``i.b``, ``e3.gate`` ...) to tensors, ``m`` is the matching size dictionary of the
configuration.  ``X [T, s, width]`` are the residual streams of a hyper-connected model.
"""

from __future__ import annotations

import math

import torch


# ---- elementwise pieces ---------------------------------------------------------------------------------------------
def layer_norm_w(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis (no bias), var = mean of squared deviations."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * w


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def log_sigmoid(z):
    return -torch.where(z < -30, -z, torch.log1p(torch.exp(-torch.clamp(z, min=-30))))


def clamped_glu(g, u, limit):
    """min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, -limit, limit) + 1)."""
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, min=-limit, max=limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)


# ---- hyper-connections ----------------------------------------------------------------------------------------------
def hyper_read(X, w_in):
    """u[t] = sum_s w_in[s] X[t, s]."""
    return torch.einsum("s,tsd->td", w_in, X)


def hyper_write(X, y, w_mix, w_out):
    """X'[t, j] = sum_s w_mix[s, j] X[t, s] + w_out[j] y[t]  (all streams at once from the old ones)."""
    return torch.einsum("sj,tsd->tjd", w_mix, X) + w_out[None, :, None] * y[:, None, :]


# ---- mixers -----------------------------------------------------------------------------------------------------------
def latent_attention(h, p, m, eps):
    """Causal softmax attention whose keys and values are up-projections of one normed latent per position, queries
    through a normed latent of their own, a value-less sink logit per head in the denominator, an elementwise sigmoid
    output gate read from the mixer's input."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cq = rms_unit(h @ p["dq"].T, eps) * p["dq.norm"]
    q = (cq @ p["uq"].T).reshape(T, H, d)
    c = rms_unit(h @ p["dkv"].T, eps) * p["dkv.norm"]
    k = (c @ p["uk"].T).reshape(T, H, d)
    v = (c @ p["uv"].T).reshape(T, H, dv)
    out = torch.zeros((T, H, dv), dtype=h.dtype)
    seen = torch.tril(torch.ones((T, T), dtype=torch.bool))
    for hh in range(H):
        s = (q[:, hh] @ k[:, hh].T) * m["scale"]                  # [query, key]
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        top = torch.maximum(s.max(dim=-1).values, p["sink"][hh])
        e = torch.exp(s - top[:, None])
        den = e.sum(dim=-1) + torch.exp(p["sink"][hh] - top)
        out[:, hh] = (e / den[:, None]) @ v[:, hh]
    gate = torch.sigmoid(h @ p["g"].T)
    return (out.reshape(T, H * dv) * gate) @ p["o"].T


def mlstm(h, p, m, eps, m0=0.0, floor=True):
    """Matrix-memory recurrence with exponential input gate and a running maximum that starts at 0.  Per head:
    m_t = max(f_t + m_(t-1), i_t);  S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T;  n_t the same with
    k_t alone;  o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ p["q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ p["k"].T).reshape(T, H, d)
    v = (h @ p["v"].T).reshape(T, H, dv)
    ig = cap * torch.tanh((h @ p["i"].T + p["i.b"]) / cap)
    fg = log_sigmoid(cap * torch.tanh((h @ p["f"].T + p["f.b"]) / cap))
    out = torch.zeros((T, H, dv), dtype=h.dtype)
    for hh in range(H):
        S = torch.zeros((d, dv), dtype=h.dtype)
        n = torch.zeros((d,), dtype=h.dtype)
        mx = torch.full((), m0, dtype=h.dtype)
        for t in range(T):
            new = torch.maximum(fg[t, hh] + mx, ig[t, hh])
            a, b = torch.exp(fg[t, hh] + mx - new), torch.exp(ig[t, hh] - new)
            S = a * S + b * torch.outer(k[t, hh], v[t, hh])
            n = a * n + b * k[t, hh]
            mx = new
            nq = torch.abs(n @ q[t, hh])
            den = (torch.maximum(nq, torch.exp(-mx)) if floor else nq) + 1e-6
            out[t, hh] = (S.T @ q[t, hh]) / den
    o = rms_unit(out, eps).reshape(T, H * dv) * p["norm"]
    return (o * torch.sigmoid(h @ p["g"].T)) @ p["o"].T


# ---- feed-forward -------------------------------------------------------------------------------------------------------
def gated_unit(h, gate, up, down, limit):
    return clamped_glu(h @ gate.T, h @ up.T, limit) @ down.T


def dense_ff(h, p, f):
    return gated_unit(h, p["gate"], p["up"], p["down"], f["limit"])


def route(z, top):
    """The ``top`` largest logits of every row (ties: the lower index) and the softmax over those alone."""
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.softmax(torch.gather(z, 1, order), dim=-1)


def expert_ff(h, p, f):
    z = h @ p["router"].T + p["router.b"]
    chosen, weight = route(z, f["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(chosen.shape[1]):
            e = int(chosen[t, j])
            out[t] = out[t] + weight[t, j] * gated_unit(h[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"],
                                                          f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + gated_unit(h, p["shared.gate"], p["shared.up"], p["shared.down"], f["shared"]["limit"])
    return out


# ---- the model ----------------------------------------------------------------------------------------------------------
def sub(w, prefix, dtype):
    return {k[len(prefix):]: v.to(dtype) for k, v in w.items() if k.startswith(prefix)}


def weight_layer(cfg, i):
    j = cfg["layers"][i].get("weights_of")
    return i if j is None else int(j)


def forward(cfg, w, tokens, dtype=torch.float64, keep_layers=False):
    """Logits [T, vocab] of one sequence (and, with ``keep_layers``, the summed streams after every layer)."""
    eps = cfg["norm"]["eps"]
    s = cfg.get("streams")
    embed = w["embed"].to(dtype)
    x = embed[torch.as_tensor(tokens, dtype=torch.long)] * cfg.get("embedding", {}).get("scale", 1.0)
    X = x[:, None, :].repeat(1, s, 1) if s else None
    kept = []

    def sublayer(q, src, fn):
        nonlocal x, X
        nw = w[f"l{src}.norm{q}"].to(dtype)
        if s:
            hc = sub(w, f"l{src}.hc{q}.", dtype)
            y = fn(layer_norm_w(hyper_read(X, hc["in"]), nw, eps))
            X = hyper_write(X, y, hc["mix"], hc["out"])
        else:
            x = x + fn(layer_norm_w(x, nw, eps))

    for i, lc in enumerate(cfg["layers"]):
        src = weight_layer(cfg, i)
        pm = sub(w, f"l{src}.mix.", dtype)
        mixer = latent_attention if lc["type"] == "latent_attention" else mlstm
        sublayer(1, src, lambda h: mixer(h, pm, lc["mixer"], eps))
        if lc.get("mlp"):
            pf = sub(w, f"l{src}.mlp.", dtype)
            ff = dense_ff if lc["mlp"]["kind"] == "dense" else expert_ff
            sublayer(2, src, lambda h: ff(h, pf, lc["mlp"]))
        if keep_layers:
            kept.append(X.sum(dim=1) if s else x.clone())
    if s:
        x = X.sum(dim=1)
    logits = layer_norm_w(x, w["final.norm"].to(dtype), eps) @ embed.T
    return (logits, torch.stack(kept)) if keep_layers else logits


MIXERS = {"latent_attention": latent_attention, "mlstm": mlstm}


def greedy(cfg, w, prompt, n_new, dtype=torch.float64):
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(cfg, w, toks, dtype)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out


def random_weights(cfg, seed, spread=1.0):
    """bfloat16-representable random weights for a configuration dictionary (float32 tensors)."""
    g = torch.Generator().manual_seed(seed)
    D, w = cfg["width"], {}
    s = cfg.get("streams")

    def mat(n_out, n_in, gain=1.0):
        return (torch.randn((n_out, n_in), generator=g) * (gain * spread / math.sqrt(n_in))).to(torch.bfloat16).float()

    def vec(n, mean=0.0, dev=0.1):
        return (mean + dev * torch.randn((n,), generator=g)).to(torch.bfloat16).float()

    def unit(prefix, ff):
        w[prefix + "gate"], w[prefix + "up"], w[prefix + "down"] = mat(ff, D, 1.5), mat(ff, D, 1.5), mat(D, ff)

    w["embed"] = (torch.randn((cfg["vocab"], D), generator=g) * spread).to(torch.bfloat16).float()
    w["final.norm"] = vec(D, 1.0)
    for i, lc in enumerate(cfg["layers"]):
        if lc.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", lc["mixer"]
        w[p + "norm1"] = vec(D, 1.0)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if lc["type"] == "latent_attention":
            w[p + "mix.dq"], w[p + "mix.dq.norm"] = mat(m["q_rank"], D), vec(m["q_rank"], 1.0)
            w[p + "mix.uq"] = mat(H * d, m["q_rank"], 2.0)
            w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(m["kv_rank"], D), vec(m["kv_rank"], 1.0)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * d, m["kv_rank"], 2.0), mat(H * dv, m["kv_rank"])
            w[p + "mix.sink"] = vec(H, 0.0, 1.0)
        else:
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * d, D), mat(H * d, D), mat(H * dv, D)
            w[p + "mix.i"], w[p + "mix.f"] = mat(H, D, 2.0), mat(H, D, 2.0)
            w[p + "mix.i.b"], w[p + "mix.f.b"] = vec(H, 0.0, 1.0), vec(H, 2.0, 1.0)
            w[p + "mix.norm"] = vec(H * dv, 1.0)
        w[p + "mix.g"], w[p + "mix.o"] = mat(H * dv, D), mat(D, H * dv)
        f = lc.get("mlp")
        if f:
            w[p + "norm2"] = vec(D, 1.0)
            if f["kind"] == "dense":
                unit(p + "mlp.", f["ff"])
            else:
                for e in range(f["router"]["experts"]):
                    unit(p + f"mlp.e{e}.", f["expert"]["ff"])
                w[p + "mlp.router"], w[p + "mlp.router.b"] = mat(f["router"]["experts"], D, 3.0), vec(f["router"]["experts"], 0.0, 0.5)
                if f.get("shared"):
                    unit(p + "mlp.shared.", f["shared"]["ff"])
        if s:
            for q in (1, 2) if f else (1,):
                w[p + f"hc{q}.in"] = vec(s, 1.0 / s, 0.2)
                w[p + f"hc{q}.out"] = vec(s, 1.0, 0.3)
                w[p + f"hc{q}.mix"] = (torch.eye(s) + 0.2 * torch.randn((s, s), generator=g)).to(torch.bfloat16).float()
    return w
