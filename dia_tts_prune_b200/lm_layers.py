"""Mechanisms of the decoder-only language-model path, as parameter holders that describe themselves to the kernels.

Beside ``layers.py`` (Dia's RMSNorm / rotary attention / gated MLP modules) this file adds
  * :class:`DynamicTanh` - a norm without statistics, ``tanh(alpha x) w + b``;
  * :class:`TapMix` - a causal per-channel short convolution over time added to its input, with a per-sequence tail;
  * :class:`SinkAttention` - grouped-query softmax attention whose values are the projected keys, with whole-projection
    q / k RMS norms, per-head temperature, tanh score cap, linear distance bias, a sliding window that keeps the first
    tokens, and a value-less sink logit in the denominator;
  * :class:`RoutedExperts` - sigmoid-scored top-k mixture of gated units whose score multiplies the expert's INPUT,
    plus an optional shared unit.
  * :class:`LayerNorm` - mean / variance norm with weight and bias;
  * :class:`TalkingAttention` - grouped-query softmax attention with biased projections, per-head q / k RMS norms, rotary
    positions on the leading channels of every head (interleaved pairs, optional wavelength-band rescaling), scores
    mixed across heads before the softmax, a value-less sink logit and a per-head sigmoid output gate;
  * :class:`Hgrn2` - gated linear recurrence whose forget gate (with a learned lower bound) also sets the write strength;
  * :class:`ChannelDelta` - gated delta rule with a decay per head and key channel, short causal convolutions on q, k, v,
    unit-vector q and k, and a low-rank sigmoid output gate;
  * :class:`DenseXielu` - up projection, xIELU activation, down projection;
  * :class:`HyperConnection` - read, mix and write weights of one sublayer over several residual streams;
  * :class:`LatentAttention` - softmax attention whose keys and values are up-projections of ONE cached normed latent per
    token (the queries go through a normed latent of their own), with a value-less sink logit and an elementwise sigmoid
    output gate;
  * :class:`MLstm` - matrix memory with an exponential input gate, capped gate pre-activations, a running maximum that
    keeps the exponentials in range and a normaliser state;
  * :class:`GatedUnit` - gate / up / down unit with the clamped activation ``g' sigmoid(1.702 g') (u' + 1)``; the same
    activation, a logit bias and softmax-over-the-chosen output weights are options of :class:`RoutedExperts`;
  * :class:`RmsNorm` - ``x / sqrt(mean(x^2) + eps) w``, as a sublayer norm of the stream form, the final norm and the
    norm of the embedding output;
  * :class:`GatedDelta` - gated delta rule with ONE decay per head and token (single-step decay and gate projections, a
    silu output gate), beside :class:`ChannelDelta`;
  * :class:`Retention` - linear attention with a fixed decay per head, rotary q and k ("half" pairs), no softmax and no
    denominator;
  * options of :class:`LatentAttention`: a turned key part shared by all heads behind the cached latent (the query heads
    carry a turned part of their own), a sliding window, no sink, no gate;
  * :class:`DenseRelu2` - up projection, squared relu, down projection;
  * options of :class:`RoutedExperts`: scores from the softmax over ALL router outputs, a correction that only the choice
    sees, choice inside the best groups of neighbouring outputs, normalised and scaled weights, identity experts, a
    sigmoid gate number on the shared unit.
All constants are constructor arguments; a design picks and combines them per layer (:class:`MixLayer` runs its
sublayers one after the other, :class:`ParallelLayer` feeds one norm to mixer and feed-forward and adds both,
:class:`StreamLayer` runs pre-norm sublayers over hyper-connected streams - with ``parallel`` both sublayers read the
streams before either writes).  The arithmetic lives in
``csrc/lm_kernels.cu``, ``csrc/lm_mixers.cu`` and ``csrc/lm_streams.cu``; these classes only keep device tensors alive
and fill ``lm_b200_layer``.
"""

from __future__ import annotations

import math

import torch

from .lm_state import StateSpec


def _f32(t: torch.Tensor, device) -> torch.Tensor:
    return t.detach().to(device=device, dtype=torch.float32).contiguous()


def _bf16(t: torch.Tensor, device) -> torch.Tensor:
    return t.detach().to(device=device, dtype=torch.bfloat16).contiguous()


class DynamicTanh:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor, alpha: float, device):
        self.w, self.b, self.alpha = _f32(weight, device), _f32(bias, device), float(alpha)

    def fill(self, rec) -> None:
        rec.w, rec.b, rec.alpha = self.w.data_ptr(), self.b.data_ptr(), self.alpha


class TapMix:
    def __init__(self, taps: torch.Tensor, device):
        """``taps [width, n]``: out_t = h_t + sum_j taps[:, j] * h_(t - n + 1 + j)."""
        self.w = _f32(taps, device)
        self.n = int(taps.shape[1])


class SinkAttention:
    def __init__(self, w_q, w_k, q_norm, k_norm, w_o, *, heads: int, kv_heads: int, dim: int, scale: float,
                 temp=None, slopes=None, sink=None, softcap: float | None = None, window: int | None = None,
                 keep_first: int = 0, device=None):
        self.heads, self.kv_heads, self.dim = int(heads), int(kv_heads), int(dim)
        self.scale, self.softcap = float(scale), float(softcap) if softcap else 0.0
        self.window, self.keep_first = int(window) if window else 0, int(keep_first or 0)
        if tuple(w_q.shape)[0] != heads * dim or tuple(w_k.shape)[0] != kv_heads * dim:
            raise ValueError("projection shapes do not match heads x dim")
        self.w_qk = _bf16(torch.cat([w_q, w_k], dim=0), device)          # one GEMM for both projections
        self.q_norm, self.k_norm = _f32(q_norm, device), _f32(k_norm, device)
        self.temp = None if temp is None else _f32(temp, device)
        self.slopes = None if slopes is None else _f32(slopes, device)
        self.sink = None if sink is None else _f32(sink, device)
        self.w_o = _bf16(w_o, device)


class RoutedExperts:
    def __init__(self, router, gates: list, ups: list, downs: list, *, top: int, shared=None, device=None,
                 router_bias=None, softmax_top: bool = False, limit: float | None = None, shared_limit: float | None = None,
                 softmax_all: bool = False, identity: int = 0, correction=None, groups: tuple[int, int] | None = None,
                 route_scale: float = 1.0, shared_gate=None):
        """``gates[e] / ups[e]: [ff, width]``, ``downs[e]: [width, ff]``; ``shared``: (gate, up, down) or None.
        ``softmax_top``: the softmax over the chosen logits weighs the experts' OUTPUTS (otherwise sigmoid scores scale
        their inputs); ``limit`` / ``shared_limit``: the clamped activation instead of silu(g) u.
        ``softmax_all``: scores are the softmax over all router outputs; the choice is made on score + ``correction``,
        inside the ``groups = (count, keep)`` best groups of neighbouring outputs; the chosen scores, divided by their sum and
        times ``route_scale``, weigh the outputs.  The last ``identity`` router outputs have no weights: their expert
        returns its input.  ``shared_gate [1, width]``: the shared unit's output is times sigmoid(shared_gate . h)."""
        self.router_bias = None if router_bias is None else _f32(router_bias, device)
        self.softmax_top, self.softmax_all = bool(softmax_top), bool(softmax_all)
        self.identity, self.route_scale = int(identity), float(route_scale)
        self.groups = (int(groups[0]), int(groups[1])) if groups else (1, 1)
        self.correction = None if correction is None else _f32(correction, device)
        self.limit = None if limit is None else float(limit)
        self.shared_limit = float(shared_limit) if shared_limit is not None else self.limit
        self.experts, self.top, self.ff = len(gates), int(top), int(gates[0].shape[0])
        if tuple(router.shape)[0] != self.experts + self.identity:
            raise ValueError("the router needs one row per expert and identity expert")
        self.has_shared_gate = shared_gate is not None
        if self.has_shared_gate:                                  # the gate's row rides behind the router's: one product
            if shared is None or not softmax_all:
                raise ValueError("a shared gate needs a shared unit and the softmax-over-all router")
            router = torch.cat([router, shared_gate.reshape(1, -1)], dim=0)
        self.w_router = _bf16(router, device)
        self.w_gate_up = _bf16(torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]), device)
        self.w_down = _bf16(torch.stack(list(downs)), device)
        self.shared_ff = 0
        self.ws_gate_up = self.ws_down = None
        if shared is not None:
            g, u, d = shared
            self.shared_ff = int(g.shape[0])
            self.ws_gate_up, self.ws_down = _bf16(torch.cat([g, u], dim=0), device), _bf16(d, device)


class MixLayer:
    """x += norm_out(mixer(tap(norm_in(x))));  x += norm_out'(ff(tap'(norm_in'(x))))  (the second line only with ``ff``)."""

    def __init__(self, mixer: SinkAttention, norm_mix_in: DynamicTanh, norm_mix_out: DynamicTanh, tap_mix: TapMix | None,
                 ff: RoutedExperts | None = None, norm_ff_in: DynamicTanh | None = None,
                 norm_ff_out: DynamicTanh | None = None, tap_ff: TapMix | None = None):
        self.mixer, self.ff = mixer, ff
        self.norm_mix_in, self.norm_mix_out, self.norm_ff_in, self.norm_ff_out = norm_mix_in, norm_mix_out, norm_ff_in, norm_ff_out
        self.tap_mix, self.tap_ff = tap_mix, tap_ff

    def state_spec(self) -> StateSpec:
        return StateSpec(kv=(self.mixer.kv_heads, self.mixer.dim, self.mixer.dim), tap_tails=2)

    def fill(self, rec, st) -> None:
        from ._lm_lib import FF_NONE, FF_ROUTED_EXPERTS, MIXER_SINK_ATTENTION
        k_pages, v_pages, (tail_mix, tail_ff) = st.k_pages, st.v_pages, st.tails
        a = self.mixer
        rec.mixer = MIXER_SINK_ATTENTION
        rec.heads, rec.kv_heads, rec.dim = a.heads, a.kv_heads, a.dim
        rec.window, rec.keep_first, rec.scale, rec.softcap = a.window, a.keep_first, a.scale, a.softcap
        self.norm_mix_in.fill(rec.norm_mix_in)
        self.norm_mix_out.fill(rec.norm_mix_out)
        rec.tap_mix = self.tap_mix.w.data_ptr() if self.tap_mix is not None else None
        rec.w_qk, rec.q_norm, rec.k_norm, rec.w_o = a.w_qk.data_ptr(), a.q_norm.data_ptr(), a.k_norm.data_ptr(), a.w_o.data_ptr()
        rec.temp = a.temp.data_ptr() if a.temp is not None else None
        rec.slopes = a.slopes.data_ptr() if a.slopes is not None else None
        rec.sink = a.sink.data_ptr() if a.sink is not None else None
        rec.k_pages, rec.v_pages = k_pages.data_ptr(), v_pages.data_ptr()
        rec.tail_mix, rec.tail_ff = tail_mix.data_ptr(), tail_ff.data_ptr()
        rec.ff = FF_NONE
        f = self.ff
        if f is not None:
            rec.ff = FF_ROUTED_EXPERTS
            rec.experts, rec.top, rec.expert_ff, rec.shared_ff = f.experts, f.top, f.ff, f.shared_ff
            self.norm_ff_in.fill(rec.norm_ff_in)
            self.norm_ff_out.fill(rec.norm_ff_out)
            rec.tap_ff = self.tap_ff.w.data_ptr() if self.tap_ff is not None else None
            rec.w_router, rec.w_gate_up, rec.w_down = f.w_router.data_ptr(), f.w_gate_up.data_ptr(), f.w_down.data_ptr()
            if f.shared_ff:
                rec.ws_gate_up, rec.ws_down = f.ws_gate_up.data_ptr(), f.ws_down.data_ptr()


# ---- the parallel form ------------------------------------------------------------------------------------------------
class LayerNorm:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None, device):
        self.w, self.b = _f32(weight, device), None if bias is None else _f32(bias, device)

    def fill(self, rec) -> None:
        from ._lm_lib import NORM_LAYER
        rec.w, rec.b, rec.alpha, rec.kind = self.w.data_ptr(), self.b.data_ptr() if self.b is not None else None, 0.0, NORM_LAYER


def rotary_angles(base: float, dims: int, scaling=None) -> torch.Tensor:
    """Angle per position of each of the ``dims / 2`` rotary pairs: ``base^(-2i/dims)``.  ``scaling`` (factor, low, high,
    original) stretches long waves: a pair whose wavelength exceeds ``original / low`` turns ``factor`` times slower, one
    below ``original / high`` is kept, and in between the two rates are blended linearly in ``original / wavelength``."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = (float(getattr(scaling, k)) for k in ("factor", "low", "high", "original"))
            turns = orig * f / (2.0 * math.pi)                    # original / wavelength
            if turns < low:
                f = f / factor
            elif turns <= high:
                t = (turns - low) / (high - low)
                f = (1.0 - t) * f / factor + t * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


class TalkingAttention:
    kind = "talk_attention"

    def __init__(self, w_q, w_k, w_v, w_o, q_norm, k_norm, *, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 b_q=None, b_k=None, b_v=None, w_gate=None, talk=None, sink=None, rot_angles=None, device=None):
        self.heads, self.kv_heads, self.dim, self.vdim, self.scale = int(heads), int(kv_heads), int(dim), int(vdim), float(scale)
        if tuple(w_q.shape)[0] != heads * dim or tuple(w_k.shape)[0] != kv_heads * dim or tuple(w_v.shape)[0] != kv_heads * vdim:
            raise ValueError("projection shapes do not match heads x dim")
        zeros = lambda n: torch.zeros(n, dtype=torch.float32)    # noqa: E731
        gate_bias = zeros(heads)
        if w_gate is None:                                        # no gate: zero rows with a bias whose sigmoid is 1.0f
            w_gate, gate_bias = torch.zeros((heads, w_q.shape[1]), dtype=w_q.dtype), torch.full((heads,), 40.0)
        self.in_rows = [w_q, w_k, w_v, w_gate]
        self.in_bias = [b if b is not None else zeros(w.shape[0]) for b, w in ((b_q, w_q), (b_k, w_k), (b_v, w_v))] + [gate_bias]
        self.has_bias = any(b is not None for b in (b_q, b_k, b_v)) or bool(gate_bias.any())
        self.w_o = w_o
        self.q_norm, self.k_norm = _f32(q_norm, device), _f32(k_norm, device)
        self.talk = None if talk is None else _f32(talk, device)
        self.sink = None if sink is None else _f32(sink, device)
        self.rot = None if rot_angles is None or rot_angles.numel() == 0 else _f32(rot_angles, device)

    def out_columns(self) -> int:
        return self.heads * self.vdim

    def state_spec(self) -> StateSpec:
        return StateSpec(kv=(self.kv_heads, self.dim, self.vdim))

    def fill(self, rec, st) -> None:
        from ._lm_lib import MIXER_TALK_ATTENTION
        rec.mixer = MIXER_TALK_ATTENTION
        rec.heads, rec.kv_heads, rec.dim, rec.vdim, rec.scale = self.heads, self.kv_heads, self.dim, self.vdim, self.scale
        rec.q_norm, rec.k_norm = self.q_norm.data_ptr(), self.k_norm.data_ptr()
        rec.talk = self.talk.data_ptr() if self.talk is not None else None
        rec.sink = self.sink.data_ptr() if self.sink is not None else None
        rec.rot_dims = 2 * self.rot.numel() if self.rot is not None else 0
        rec.rot_freq = self.rot.data_ptr() if self.rot is not None else None
        rec.k_pages, rec.v_pages = st.k_pages.data_ptr(), st.v_pages.data_ptr()


class Hgrn2:
    kind = "hgrn2"

    def __init__(self, w_q, w_f, w_v, w_o, head_norm, *, heads: int, dim: int, vdim: int, b_f=None, lower=None, device=None):
        self.heads, self.dim, self.vdim = int(heads), int(dim), int(vdim)
        if tuple(w_q.shape)[0] != heads * dim or tuple(w_f.shape)[0] != heads * dim or tuple(w_v.shape)[0] != heads * vdim:
            raise ValueError("projection shapes do not match heads x dim")
        self.in_rows = [w_q, w_f, w_v]
        zeros = lambda n: torch.zeros(n, dtype=torch.float32)    # noqa: E731
        self.in_bias = [zeros(heads * dim), b_f if b_f is not None else zeros(heads * dim), zeros(heads * vdim)]
        self.has_bias = b_f is not None
        self.w_o = w_o
        self.head_norm = _f32(head_norm, device)
        self.lower = None if lower is None else _f32(lower, device)

    def out_columns(self) -> int:
        return self.heads * self.vdim

    def state_spec(self) -> StateSpec:
        return StateSpec(recurrent=(self.heads, self.vdim, self.dim))

    def fill(self, rec, st) -> None:
        from ._lm_lib import MIXER_HGRN2
        rec.mixer = MIXER_HGRN2
        rec.heads, rec.kv_heads, rec.dim, rec.vdim = self.heads, self.heads, self.dim, self.vdim
        rec.head_norm = self.head_norm.data_ptr()
        rec.lower = self.lower.data_ptr() if self.lower is not None else None
        rec.rec_state = st.rec_state.data_ptr()


class ChannelDelta:
    kind = "channel_delta"

    def __init__(self, w_q, w_k, w_v, w_beta, w_a1, w_a2, w_g1, w_g2, w_o, conv_q, conv_k, conv_v, a_log, dt_bias, head_norm, *,
                 heads: int, kv_heads: int, dim: int, vdim: int, unit_eps: float = 1e-6, device=None):
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        if tuple(w_q.shape)[0] != kv_heads * dim or tuple(w_k.shape)[0] != kv_heads * dim or tuple(w_v.shape)[0] != heads * vdim:
            raise ValueError("projection shapes do not match heads x dim")
        self.taps = int(conv_q.shape[1])
        self.rank_a, self.rank_g = int(w_a1.shape[0]), int(w_g1.shape[0])
        if tuple(w_a2.shape) != (heads * dim, self.rank_a) or tuple(w_g2.shape) != (heads * vdim, self.rank_g):
            raise ValueError("the second steps of the decay / gate projections do not match heads x dim / heads x vdim")
        self.in_rows = [w_q, w_k, w_v, w_beta, w_a1, w_g1]
        self.in_bias, self.has_bias = None, False
        self.w_o = w_o
        self.conv_w = _f32(torch.cat([conv_q, conv_k, conv_v], dim=0), device)
        self.a_log, self.dt_bias = _f32(a_log, device), _f32(dt_bias, device)
        self.w_a2, self.w_g2 = _bf16(w_a2, device), _bf16(w_g2, device)
        self.head_norm = _f32(head_norm, device)
        self.unit_eps = float(unit_eps)

    def out_columns(self) -> int:
        return self.heads * self.vdim

    def state_spec(self) -> StateSpec:
        return StateSpec(recurrent=(self.heads, self.vdim, self.dim),
                         conv=(self.taps, 2 * self.kv_heads * self.dim + self.heads * self.vdim))

    def fill(self, rec, st) -> None:
        from ._lm_lib import MIXER_CHANNEL_DELTA
        rec.mixer = MIXER_CHANNEL_DELTA
        rec.heads, rec.kv_heads, rec.dim, rec.vdim = self.heads, self.kv_heads, self.dim, self.vdim
        rec.conv_taps, rec.rank_a, rec.rank_g, rec.unit_eps = self.taps, self.rank_a, self.rank_g, self.unit_eps
        rec.conv_w, rec.a_log, rec.dt_bias = self.conv_w.data_ptr(), self.a_log.data_ptr(), self.dt_bias.data_ptr()
        rec.w_a2, rec.w_g2, rec.head_norm = self.w_a2.data_ptr(), self.w_g2.data_ptr(), self.head_norm.data_ptr()
        rec.rec_state, rec.conv_tail = st.rec_state.data_ptr(), st.conv_tail.data_ptr()


def _softplus(z: float) -> float:
    return z if z > 30.0 else math.log1p(math.exp(z))


class DenseXielu:
    def __init__(self, w_up, w_down, act):
        """``act``: the two raw numbers (p, q) of the activation; z > 0: softplus(p) z^2 + z / 2, z <= 0:
        (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
        self.w_up, self.w_down, self.ff = w_up, w_down, int(w_up.shape[0])
        p, q = (float(v) for v in act.detach().to(torch.float64).reshape(-1)[:2])
        self.act_p, self.act_q = _softplus(p), 0.5 + _softplus(q)


class ParallelLayer:
    """h = norm(x);  x += mixer(h) + ff(h).  Every projection that reads h is one stacked matrix, and the mixer's output
    projection stands beside the feed-forward's down projection in one matrix, so a layer is two products around its
    mixer kernels."""

    def __init__(self, norm: LayerNorm, mixer, ff: DenseXielu | None, device):
        self.norm, self.mixer, self.ff = norm, mixer, ff
        rows = [_bf16(r, device) for r in list(mixer.in_rows) + ([ff.w_up] if ff is not None else [])]
        n = sum(int(r.shape[0]) for r in rows)
        self.n_in = (n + 3) & ~3
        width = int(rows[0].shape[1])
        if self.n_in > n:
            rows.append(torch.zeros((self.n_in - n, width), dtype=torch.bfloat16, device=device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.in_bias = None
        if mixer.has_bias:
            b = torch.cat([_f32(x, device).reshape(-1) for x in mixer.in_bias])
            self.in_bias = torch.cat([b, torch.zeros(self.n_in - b.numel(), dtype=torch.float32, device=device)]).contiguous()
        outs = [_bf16(o, device) for o in [mixer.w_o] + ([ff.w_down] if ff is not None else [])]
        self.w_out = torch.cat(outs, dim=1).contiguous()
        self.k_out = int(self.w_out.shape[1])

    def state_spec(self) -> StateSpec:
        return self.mixer.state_spec()

    def fill(self, rec, st) -> None:
        from ._lm_lib import ACT_XIELU, FF_DENSE, FF_NONE, FORM_PARALLEL
        rec.form = FORM_PARALLEL
        self.norm.fill(rec.norm_mix_in)
        self.mixer.fill(rec, st)
        rec.n_in, rec.k_out = self.n_in, self.k_out
        rec.w_in, rec.w_out = self.w_in.data_ptr(), self.w_out.data_ptr()
        rec.in_bias = self.in_bias.data_ptr() if self.in_bias is not None else None
        rec.ff = FF_NONE
        if self.ff is not None:
            rec.ff, rec.dense_ff, rec.act = FF_DENSE, self.ff.ff, ACT_XIELU
            rec.act_p, rec.act_q = self.ff.act_p, self.ff.act_q


class LayerRun:
    """One execution of a layer: the layer's weights with a state of its own, and optionally the input mix
    ``x <- W [x; embedding output]`` in front of it (the first layer of a pass over a repeated block)."""

    def __init__(self, layer, pre: torch.Tensor | None = None, device=None):
        self.layer = layer
        self.pre = None if pre is None else _bf16(pre, device)
        self.mixer, self.ff = layer.mixer, layer.ff

    def state_spec(self) -> StateSpec:
        return self.layer.state_spec()

    def fill(self, rec, st) -> None:
        self.layer.fill(rec, st)
        rec.w_pre = self.pre.data_ptr() if self.pre is not None else None


# ---- the stream form ----------------------------------------------------------------------------------------------------
class HyperConnection:
    """One sublayer's weights over ``s`` residual streams: it reads ``u = sum_s w_in[s] x_s`` and writes
    ``x_j <- sum_s w_mix[s, j] x_s + w_out[j] y``.  :meth:`residual` is the plain residual sum as one stream."""

    def __init__(self, w_in, w_out, w_mix, device):
        self.streams = int(w_in.numel())
        if tuple(w_out.shape) != (self.streams,) or tuple(w_mix.shape) != (self.streams, self.streams):
            raise ValueError("hyper-connection weights do not match the number of streams")
        self.w_in, self.w_out, self.w_mix = _f32(w_in, device), _f32(w_out, device), _f32(w_mix, device)

    @classmethod
    def residual(cls, device) -> "HyperConnection":
        return cls(torch.ones(1), torch.ones(1), torch.ones((1, 1)), device)


class LatentAttention:
    kind = "latent_attention"

    def __init__(self, w_dq, q_lat_norm, w_uq, w_dkv, kv_lat_norm, w_uk, w_uv, w_gate, w_o, *, heads: int, dim: int, vdim: int,
                 scale: float, sink=None, device=None, rot_dim: int = 0, rot_angles=None, rot_half: bool = False,
                 window: int | None = None):
        """``rot_dim`` > 0: every query head is ``[dim plain | rot_dim turned]`` (``w_uq`` has heads x (dim + rot_dim) rows) and
        ``w_dkv`` has ``rot_dim`` more rows behind the latent's: one turned key part for all heads, cached beside the
        latent.  ``rot_angles``: angle per position of the turning pairs (the first 2 x len channels of the turned part).
        ``window``: a position sees itself and the ``window - 1`` before it.  ``w_gate`` None: no output gate."""
        self.heads, self.dim, self.vdim, self.scale = int(heads), int(dim), int(vdim), float(scale)
        self.rot_dim, self.rot_half, self.window = int(rot_dim), bool(rot_half), int(window) if window else 0
        self.q_rank, self.kv_rank = int(w_dq.shape[0]), int(w_dkv.shape[0]) - self.rot_dim
        if (tuple(w_uq.shape) != (heads * (dim + self.rot_dim), self.q_rank) or tuple(w_uk.shape) != (heads * dim, self.kv_rank)
                or tuple(w_uv.shape) != (heads * vdim, self.kv_rank) or (w_gate is not None and tuple(w_gate.shape)[0] != heads * vdim)):
            raise ValueError("projection shapes do not match heads x dim and the latent sizes")
        self.gated = w_gate is not None
        self.in_rows, self.in_bias, self.w_o = [w_dq, w_dkv] + ([w_gate] if self.gated else []), None, w_o
        self.rot = None if rot_angles is None or rot_angles.numel() == 0 else _f32(rot_angles, device)
        if self.rot is not None and 2 * self.rot.numel() > self.rot_dim:
            raise ValueError("more turning channels than the turned part has")
        self.q_lat_norm, self.kv_lat_norm = _f32(q_lat_norm, device), _f32(kv_lat_norm, device)
        self.w_uq = _bf16(w_uq, device)
        # scores are taken in the latent space: q_h . (W_uk,h c) = (W_uk,h^T q_h) . c, so the kernels want W_uk,h^T
        self.w_uk_t = _bf16(w_uk.reshape(heads, dim, self.kv_rank).transpose(1, 2), device)
        self.w_uv = _bf16(w_uv, device)                           # [heads][vdim][kv_rank] as stored
        self.sink = None if sink is None else _f32(sink, device)

    def state_spec(self) -> StateSpec:
        return StateSpec(latent=self.kv_rank + self.rot_dim)

    def fill(self, rec, st) -> None:
        from ._lm_lib import GATE_NONE, GATE_SIGMOID, MIXER_LATENT_ATTENTION, ROT_HALF, ROT_INTERLEAVED
        rec.mixer = MIXER_LATENT_ATTENTION
        rec.mixer_gate = GATE_SIGMOID if self.gated else GATE_NONE
        rec.rot_dim, rec.window = self.rot_dim, self.window
        rec.rot_dims = 2 * self.rot.numel() if self.rot is not None else 0
        rec.rot_freq = self.rot.data_ptr() if self.rot is not None else None
        rec.rot_layout = ROT_HALF if self.rot_half else ROT_INTERLEAVED
        rec.heads, rec.kv_heads, rec.dim, rec.vdim, rec.scale = self.heads, 1, self.dim, self.vdim, self.scale
        rec.q_rank, rec.kv_rank = self.q_rank, self.kv_rank
        rec.q_lat_norm, rec.kv_lat_norm = self.q_lat_norm.data_ptr(), self.kv_lat_norm.data_ptr()
        rec.w_uq, rec.w_uk_t, rec.w_uv = self.w_uq.data_ptr(), self.w_uk_t.data_ptr(), self.w_uv.data_ptr()
        rec.sink = self.sink.data_ptr() if self.sink is not None else None
        rec.latent_pages = st.latent_pages.data_ptr()


class MLstm:
    kind = "mlstm"

    def __init__(self, w_q, w_k, w_v, w_i, w_f, w_gate, w_o, head_norm, *, heads: int, dim: int, vdim: int, gate_cap: float,
                 b_i=None, b_f=None, device=None):
        self.heads, self.dim, self.vdim, self.gate_cap = int(heads), int(dim), int(vdim), float(gate_cap)
        if (tuple(w_q.shape)[0] != heads * dim or tuple(w_k.shape)[0] != heads * dim or tuple(w_v.shape)[0] != heads * vdim
                or tuple(w_i.shape)[0] != heads or tuple(w_f.shape)[0] != heads or tuple(w_gate.shape)[0] != heads * vdim):
            raise ValueError("projection shapes do not match heads x dim")
        self.in_rows, self.w_o = [w_q, w_k, w_v, w_i, w_f, w_gate], w_o
        zeros = lambda n: torch.zeros(n, dtype=torch.float32)    # noqa: E731
        self.in_bias = None
        if b_i is not None or b_f is not None:
            self.in_bias = [zeros(2 * heads * dim + heads * vdim), b_i if b_i is not None else zeros(heads),
                            b_f if b_f is not None else zeros(heads), zeros(heads * vdim)]
        self.head_norm = _f32(head_norm, device)                 # [heads * vdim]

    def state_spec(self) -> StateSpec:
        # the normaliser rides as one more value column of the matrix state; the running maximum per head beside it
        return StateSpec(recurrent=(self.heads, self.vdim + 1, self.dim), aux=self.heads)

    def fill(self, rec, st) -> None:
        from ._lm_lib import MIXER_MLSTM
        rec.mixer = MIXER_MLSTM
        rec.heads, rec.kv_heads, rec.dim, rec.vdim, rec.gate_cap = self.heads, self.heads, self.dim, self.vdim, self.gate_cap
        rec.head_norm = self.head_norm.data_ptr()
        rec.rec_state, rec.rec_aux = st.rec_state.data_ptr(), st.rec_aux.data_ptr()


def _gate_kind(gate: str | None) -> int:
    from ._lm_lib import GATE_NONE, GATE_SIGMOID, GATE_SILU
    return {None: GATE_NONE, "sigmoid": GATE_SIGMOID, "silu": GATE_SILU}[gate]


class GatedDelta:
    kind = "gated_delta"

    def __init__(self, w_q, w_k, w_v, w_beta, w_a, w_gate, w_o, conv_q, conv_k, conv_v, a_log, dt_bias, head_norm, *, heads: int,
                 kv_heads: int, dim: int, vdim: int, unit_eps: float = 1e-6, gate: str | None = "silu", device=None):
        """Per head S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q with ONE decay g = exp(-exp(a_log) softplus(w_a . h
        + dt_bias)) per head and token; q, k, v pass a short causal convolution and silu, q and k become unit vectors (q
        also x dim^-1/2); o / rms(o) x head_norm [vdim] x gate(w_gate h)."""
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        if (tuple(w_q.shape)[0] != kv_heads * dim or tuple(w_k.shape)[0] != kv_heads * dim or tuple(w_v.shape)[0] != heads * vdim
                or tuple(w_beta.shape)[0] != heads or tuple(w_a.shape)[0] != heads or heads % kv_heads):
            raise ValueError("projection shapes do not match heads x dim")
        self.taps, self.gate = int(conv_q.shape[1]), gate
        self.in_rows = [w_q, w_k, w_v, w_beta, w_a] + ([w_gate] if gate is not None else [])
        self.in_bias, self.w_o = None, w_o
        self.conv_w = _f32(torch.cat([conv_q, conv_k, conv_v], dim=0), device)
        self.a_log, self.dt_bias = _f32(a_log, device), _f32(dt_bias, device)
        self.head_norm = _f32(head_norm, device)
        self.unit_eps = float(unit_eps)

    def state_spec(self) -> StateSpec:
        return StateSpec(recurrent=(self.heads, self.vdim, self.dim),
                         conv=(self.taps, 2 * self.kv_heads * self.dim + self.heads * self.vdim))

    def fill(self, rec, st) -> None:
        from ._lm_lib import MIXER_GATED_DELTA
        rec.mixer, rec.mixer_gate = MIXER_GATED_DELTA, _gate_kind(self.gate)
        rec.heads, rec.kv_heads, rec.dim, rec.vdim = self.heads, self.kv_heads, self.dim, self.vdim
        rec.conv_taps, rec.unit_eps = self.taps, self.unit_eps
        rec.conv_w, rec.a_log, rec.dt_bias = self.conv_w.data_ptr(), self.a_log.data_ptr(), self.dt_bias.data_ptr()
        rec.head_norm = self.head_norm.data_ptr()
        rec.rec_state, rec.conv_tail = st.rec_state.data_ptr(), st.conv_tail.data_ptr()


class Retention:
    kind = "retention"

    def __init__(self, w_q, w_k, w_v, w_gate, w_o, decay, *, heads: int, dim: int, vdim: int, rot_angles=None, rot_half: bool = True,
                 head_norm=None, gate: str | None = "silu", device=None):
        """Per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with a fixed ``decay`` per head; q and k turn with the
        position (``rot_angles`` per pair), k also x dim^-1/2; o / rms(o) per head (x ``head_norm [vdim]`` if given) x
        gate(w_gate h)."""
        self.heads, self.dim, self.vdim = int(heads), int(dim), int(vdim)
        if (tuple(w_q.shape)[0] != heads * dim or tuple(w_k.shape)[0] != heads * dim or tuple(w_v.shape)[0] != heads * vdim
                or len(decay) != heads):
            raise ValueError("projection shapes do not match heads x dim")
        self.gate, self.rot_half = gate, bool(rot_half)
        self.in_rows = [w_q, w_k, w_v] + ([w_gate] if gate is not None else [])
        self.in_bias, self.w_o = None, w_o
        self.decay = _f32(torch.tensor([float(d) for d in decay], dtype=torch.float64), device)
        self.rot = None if rot_angles is None or rot_angles.numel() == 0 else _f32(rot_angles, device)
        self.head_norm = None if head_norm is None else _f32(head_norm, device)

    def state_spec(self) -> StateSpec:
        return StateSpec(recurrent=(self.heads, self.vdim, self.dim))

    def fill(self, rec, st) -> None:
        from ._lm_lib import MIXER_RETENTION, ROT_HALF, ROT_INTERLEAVED
        rec.mixer, rec.mixer_gate = MIXER_RETENTION, _gate_kind(self.gate)
        rec.heads, rec.kv_heads, rec.dim, rec.vdim = self.heads, self.heads, self.dim, self.vdim
        rec.head_decay = self.decay.data_ptr()
        rec.head_norm = self.head_norm.data_ptr() if self.head_norm is not None else None
        rec.rot_dims = 2 * self.rot.numel() if self.rot is not None else 0
        rec.rot_freq = self.rot.data_ptr() if self.rot is not None else None
        rec.rot_layout = ROT_HALF if self.rot_half else ROT_INTERLEAVED
        rec.rec_state = st.rec_state.data_ptr()


class DenseRelu2:
    def __init__(self, w_up, w_down, device=None):
        """``down(max(up h, 0)^2)``."""
        self.ff = int(w_up.shape[0])
        self.w_up, self.w_down = _bf16(w_up, device), _bf16(w_down, device)


class RmsNorm:
    def __init__(self, weight: torch.Tensor, device):
        self.w = _f32(weight, device)

    def fill(self, rec) -> None:
        from ._lm_lib import NORM_RMS
        rec.w, rec.b, rec.alpha, rec.kind = self.w.data_ptr(), None, 0.0, NORM_RMS


class GatedUnit:
    def __init__(self, w_gate, w_up, w_down, *, limit: float | None, device=None):
        """``down(act(gate h, up h))``; with ``limit`` the clamped activation, without it silu(g) u."""
        self.ff, self.limit = int(w_gate.shape[0]), None if limit is None else float(limit)
        self.w_gate_up, self.w_down = _bf16(torch.cat([w_gate, w_up], dim=0), device), _bf16(w_down, device)


class StreamLayer:
    """Pre-norm sublayers over hyper-connected residual streams: for the mixer and then the feed-forward,
    ``u = sum_s in[s] x_s;  y = sublayer(layernorm(u) w);  x_j <- sum_s mix[s, j] x_s + out[j] y``.  Every projection that
    reads the mixer's input is one stacked matrix.  The same object may stand in several layer records (a layer that runs
    with another layer's weights): each record gets a state of its own."""

    def __init__(self, norm1, hc1: HyperConnection, mixer, ff=None, norm2=None, hc2: HyperConnection | None = None, device=None,
                 parallel: bool = False, rms: bool = False):
        """``parallel``: the feed-forward reads the streams as they were before the mixer's write, and both outputs are
        written at once (with one stream: x += mixer(norm1 x) + ff(norm2 x)).  ``rms``: the norms are RMS norms."""
        self.mixer, self.ff, self.hc1, self.hc2 = mixer, ff, hc1, hc2
        self.parallel, self.rms = bool(parallel), bool(rms)
        self.norm1 = _f32(norm1, device)
        self.norm2 = None if norm2 is None else _f32(norm2, device)
        if ff is not None and (norm2 is None or hc2 is None or hc2.streams != hc1.streams):
            raise ValueError("a feed-forward sublayer needs its norm and hyper-connection weights")
        rows = [_bf16(r, device) for r in mixer.in_rows]
        n = sum(int(r.shape[0]) for r in rows)
        self.n_in = (n + 3) & ~3
        if self.n_in > n:
            rows.append(torch.zeros((self.n_in - n, int(rows[0].shape[1])), dtype=torch.bfloat16, device=device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.in_bias = None
        if mixer.in_bias is not None:
            b = torch.cat([_f32(x, device).reshape(-1) for x in mixer.in_bias])
            self.in_bias = torch.cat([b, torch.zeros(self.n_in - b.numel(), dtype=torch.float32, device=device)]).contiguous()
        self.w_o = _bf16(mixer.w_o, device)

    def state_spec(self) -> StateSpec:
        return self.mixer.state_spec()

    def fill(self, rec, st) -> None:
        from ._lm_lib import (ACT_CLAMPED_GLU, ACT_RELU2, ACT_SILU_GLU, FF_DENSE, FF_NONE, FF_ROUTED_EXPERTS, FORM_STREAMS,
                              NORM_LAYER, NORM_RMS, ROUTER_SIGMOID_INPUT, ROUTER_SOFTMAX_GROUPED, ROUTER_SOFTMAX_TOP)
        norm_kind = NORM_RMS if self.rms else NORM_LAYER
        rec.form, rec.streams, rec.parallel = FORM_STREAMS, self.hc1.streams, 1 if self.parallel else 0
        rec.norm_mix_in.w, rec.norm_mix_in.b, rec.norm_mix_in.kind = self.norm1.data_ptr(), None, norm_kind
        for q, hc in enumerate((self.hc1, self.hc2)):
            if hc is not None:
                rec.hc_in[q], rec.hc_out[q], rec.hc_mix[q] = hc.w_in.data_ptr(), hc.w_out.data_ptr(), hc.w_mix.data_ptr()
        self.mixer.fill(rec, st)
        rec.n_in, rec.w_in, rec.w_o = self.n_in, self.w_in.data_ptr(), self.w_o.data_ptr()
        rec.in_bias = self.in_bias.data_ptr() if self.in_bias is not None else None
        rec.ff = FF_NONE
        f = self.ff
        if f is None:
            return
        rec.norm_ff_in.w, rec.norm_ff_in.b, rec.norm_ff_in.kind = self.norm2.data_ptr(), None, norm_kind
        if isinstance(f, DenseRelu2):
            rec.ff, rec.dense_ff, rec.act = FF_DENSE, f.ff, ACT_RELU2
            rec.ws_gate_up, rec.ws_down = f.w_up.data_ptr(), f.w_down.data_ptr()
            return
        rec.act = ACT_CLAMPED_GLU if f.limit is not None else ACT_SILU_GLU
        rec.act_limit = f.limit if f.limit is not None else 0.0
        if isinstance(f, GatedUnit):
            rec.ff, rec.dense_ff = FF_DENSE, f.ff
            rec.ws_gate_up, rec.ws_down = f.w_gate_up.data_ptr(), f.w_down.data_ptr()
            return
        rec.ff = FF_ROUTED_EXPERTS
        rec.experts, rec.top, rec.expert_ff, rec.shared_ff = f.experts, f.top, f.ff, f.shared_ff
        rec.router = ROUTER_SOFTMAX_GROUPED if f.softmax_all else ROUTER_SOFTMAX_TOP if f.softmax_top else ROUTER_SIGMOID_INPUT
        rec.identity_experts, rec.route_scale, rec.shared_gate = f.identity, f.route_scale, 1 if f.has_shared_gate else 0
        rec.group_count, rec.group_keep = f.groups
        rec.route_correction = f.correction.data_ptr() if f.correction is not None else None
        rec.router_bias = f.router_bias.data_ptr() if f.router_bias is not None else None
        rec.shared_limit = f.shared_limit if f.shared_limit is not None else 0.0
        rec.w_router, rec.w_gate_up, rec.w_down = f.w_router.data_ptr(), f.w_gate_up.data_ptr(), f.w_down.data_ptr()
        if f.shared_ff:
            rec.ws_gate_up, rec.ws_down = f.ws_gate_up.data_ptr(), f.ws_down.data_ptr()
