"""``CausalLM``: the decoder-only language models behind the framework's serving interface.

``CausalLM.from_pretrained(folder)`` reads ``config.json`` + ``model.safetensors``, builds the layer stack out of the
mechanisms of ``lm_layers.py`` and binds it to an :class:`~.lm_engine.LMEngine` with a paged sequence state.  Requests
then go through one scheduler (:class:`Scheduler`): it admits waiting requests while slots and pages last, feeds prompt
portions and decode rows of all running requests to the SAME step function as one flat batch, samples, and gives the
state of finished requests back.  ``generate`` (token ids in, token ids out - these models ship no tokenizer) and the
teacher-forced ``run_step`` of the trace replayer both sit on it.
"""

from __future__ import annotations

import json
from collections import deque
from dataclasses import dataclass, field
from pathlib import Path

import torch

from .checkpoint import load_safetensors
from .lm_config import FipadraConfig, KupelixConfig, LuketarConfig, PubopelConfig, load_config
from .lm_engine import LMEngine
from .lm_layers import (ChannelDelta, DenseRelu2, DenseXielu, DynamicTanh, GatedDelta, GatedUnit, Hgrn2, HyperConnection,
                        LatentAttention, LayerNorm, LayerRun, MixLayer, MLstm, ParallelLayer, Retention, RmsNorm, RoutedExperts,
                        SinkAttention, StreamLayer, TalkingAttention, TapMix, rotary_angles)
from .lm_state import OutOfPages, PagedState, Sequence


def distance_slopes(heads: int) -> torch.Tensor:
    """Per-head slope of the linear distance bias of the Pubopel design: 2^(-8 (h + 1) / heads)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float64).to(torch.float32)


def build_pubopel_layers(cfg: PubopelConfig, w: dict[str, torch.Tensor], device) -> tuple[list[MixLayer], DynamicTanh]:
    """The layer stack of a Pubopel checkpoint (tensor names ``l<i>.norm1``, ``l<i>.mix.q``, ``l<i>.mlp.e<j>.gate`` ...)."""

    def norm(name: str) -> DynamicTanh:
        return DynamicTanh(w[name], w[name + ".b"], float(w[name + ".alpha"].float().item()), device)

    layers = []
    for i, lc in enumerate(cfg.layers):
        p, m = f"l{i}.", lc.mixer
        attn = SinkAttention(w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.q.norm"], w[p + "mix.k.norm"], w[p + "mix.o"],
                             heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, scale=m.scale, temp=w[p + "mix.temp"],
                             slopes=distance_slopes(m.heads), sink=w[p + "mix.sink"], softcap=m.softcap,
                             window=m.mask.size if m.mask else None, keep_first=m.mask.keep_first if m.mask else 0,
                             device=device)
        ff = n2 = n2b = t2 = None
        if lc.mlp is not None:
            E = lc.mlp.router.experts
            shared = None
            if lc.mlp.shared is not None:
                shared = (w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"], w[p + "mlp.shared.down"])
            ff = RoutedExperts(w[p + "mlp.router"], [w[p + f"mlp.e{e}.gate"] for e in range(E)],
                               [w[p + f"mlp.e{e}.up"] for e in range(E)], [w[p + f"mlp.e{e}.down"] for e in range(E)],
                               top=lc.mlp.router.top, shared=shared, device=device)
            n2, n2b, t2 = norm(p + "norm2"), norm(p + "norm2b"), TapMix(w[p + "canon2"], device)
        layers.append(MixLayer(attn, norm(p + "norm1"), norm(p + "norm1b"), TapMix(w[p + "canon1"], device), ff, n2, n2b, t2))
    return layers, norm("final.norm")


def build_kupelix_layers(cfg: KupelixConfig, w: dict[str, torch.Tensor], device) -> tuple[list[LayerRun], LayerNorm]:
    """The layer records of a Kupelix checkpoint in execution order (tensor names ``l<i>.norm1``, ``l<i>.mix.*``,
    ``l<i>.mlp.*``, ``loop.in``): every layer is built once, and a layer inside the repeated block appears once per pass,
    the first layer of each pass with the input mix in front."""
    built = []
    for i, lc in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", lc.mixer
        t = lambda name: w[p + name]                             # noqa: E731
        if lc.type == "attention":
            rot = rotary_angles(m.rot.base, m.rot.dims, m.rot.scaling) if m.rot is not None and m.rot.dims > 0 else None
            mixer = TalkingAttention(t("q"), t("k"), t("v"), t("o"), t("q.norm"), t("k.norm"), heads=m.heads,
                                     kv_heads=m.kv_heads or m.heads, dim=m.dim, vdim=m.vdim, scale=m.scale, b_q=t("q.b"),
                                     b_k=t("k.b"), b_v=t("v.b"), w_gate=t("g"), talk=t("talk"), sink=t("sink"), rot_angles=rot,
                                     device=device)
        elif lc.type == "hgrn2":
            mixer = Hgrn2(t("q"), t("f"), t("v"), t("o"), t("norm"), heads=m.heads, dim=m.dim, vdim=m.vdim, b_f=t("f.b"),
                          lower=t("lower"), device=device)
        else:
            mixer = ChannelDelta(t("q"), t("k"), t("v"), t("b"), t("a1"), t("a2"), t("g1"), t("g2"), t("o"), t("q.conv"),
                                 t("k.conv"), t("v.conv"), t("A_log"), t("dt_bias"), t("norm"), heads=m.heads,
                                 kv_heads=m.kv_heads or m.heads, dim=m.dim, vdim=m.vdim, device=device)
        ff = None
        if lc.mlp is not None:
            ff = DenseXielu(w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"], w[f"l{i}.mlp.act"])
        built.append(ParallelLayer(LayerNorm(w[f"l{i}.norm1"], w[f"l{i}.norm1.b"], device), mixer, ff, device))
    pre = w["loop.in"] if cfg.loop is not None else None
    runs = [LayerRun(built[i], pre if starts else None, device) for i, starts in cfg.runs()]
    return runs, LayerNorm(w["final.norm"], w["final.norm.b"], device)


def build_luketar_layers(cfg: LuketarConfig, w: dict[str, torch.Tensor], device) -> tuple[list[StreamLayer], LayerNorm]:
    """The layer records of a Luketar checkpoint in execution order (tensor names ``l<i>.norm1``, ``l<i>.hc1.in``,
    ``l<i>.mix.*``, ``l<i>.mlp.*``): a layer with weights of its own is built once; a layer that names another layer's
    weights is that layer's object again, and gets its own state record by its place in the list."""
    built: dict[int, StreamLayer] = {}

    def hyper(prefix: str) -> HyperConnection:
        if cfg.streams is None:
            return HyperConnection.residual(device)
        return HyperConnection(w[prefix + "in"], w[prefix + "out"], w[prefix + "mix"], device)

    def build(i: int) -> StreamLayer:
        lc, p = cfg.layers[i], f"l{i}.mix."
        m = lc.mixer
        t = lambda name: w[p + name]                             # noqa: E731
        if lc.type == "latent_attention":
            mixer = LatentAttention(t("dq"), t("dq.norm"), t("uq"), t("dkv"), t("dkv.norm"), t("uk"), t("uv"), t("g"), t("o"),
                                    heads=m.heads, dim=m.dim, vdim=m.vdim, scale=m.scale, sink=t("sink"), device=device)
        else:
            mixer = MLstm(t("q"), t("k"), t("v"), t("i"), t("f"), t("g"), t("o"), t("norm"), heads=m.heads, dim=m.dim,
                          vdim=m.vdim, gate_cap=m.gate_cap, b_i=t("i.b"), b_f=t("f.b"), device=device)
        ff = norm2 = hc2 = None
        f, q = lc.mlp, f"l{i}.mlp."
        if f is not None:
            norm2, hc2 = w[f"l{i}.norm2"], hyper(f"l{i}.hc2.")
            if f.kind == "dense":
                ff = GatedUnit(w[q + "gate"], w[q + "up"], w[q + "down"], limit=f.limit, device=device)
            else:
                E = f.router.experts
                shared = (w[q + "shared.gate"], w[q + "shared.up"], w[q + "shared.down"]) if f.shared is not None else None
                ff = RoutedExperts(w[q + "router"], [w[q + f"e{e}.gate"] for e in range(E)], [w[q + f"e{e}.up"] for e in range(E)],
                                   [w[q + f"e{e}.down"] for e in range(E)], top=f.router.top, shared=shared, device=device,
                                   router_bias=w[q + "router.b"], softmax_top=True, limit=f.expert.limit,
                                   shared_limit=f.shared.limit if f.shared is not None else None)
        return StreamLayer(w[f"l{i}.norm1"], hyper(f"l{i}.hc1."), mixer, ff, norm2, hc2, device=device)

    runs = []
    for i in range(len(cfg.layers)):
        j = cfg.weight_layer(i)
        if j not in built:
            built[j] = build(j)
        runs.append(built[j])
    return runs, LayerNorm(w["final.norm"], None, device)


def build_fipadra_layers(cfg: FipadraConfig, w: dict[str, torch.Tensor], device) -> tuple[list[StreamLayer], RmsNorm]:
    """The layer records of a Fipadra checkpoint (tensor names ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
    ``l<i>.mlp.*``): stream records with one plain residual stream, RMS norms, and both sublayers reading the same x."""
    residual = HyperConnection.residual(device)                   # one object: both sublayers read with the same weights
    layers = []
    for i, lc in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", lc.mixer
        t = lambda name: w[p + name]                             # noqa: E731
        rot = getattr(m, "rot", None)
        angles = rotary_angles(rot.base, rot.dims, rot.scaling) if rot is not None and rot.dims > 0 else None
        if lc.type == "delta":
            mixer = GatedDelta(t("q"), t("k"), t("v"), t("b"), t("a"), t("g"), t("o"), t("q.conv"), t("k.conv"), t("v.conv"),
                               t("A_log"), t("dt_bias"), t("norm"), heads=m.heads, kv_heads=m.kv_heads or m.heads, dim=m.dim,
                               vdim=m.vdim, gate="silu", device=device)
        elif lc.type == "latent_attention":
            mixer = LatentAttention(t("dq"), t("dq.norm"), t("uq"), t("dkv"), t("dkv.norm"), t("uk"), t("uv"), None, t("o"),
                                    heads=m.heads, dim=m.dim, vdim=m.vdim, scale=m.scale, sink=None, rot_dim=m.rot_dim,
                                    rot_angles=angles, rot_half=False, window=m.mask.size if m.mask else None, device=device)
        else:
            mixer = Retention(t("q"), t("k"), t("v"), t("g"), t("o"), m.decay, heads=m.heads, dim=m.dim, vdim=m.vdim,
                              rot_angles=angles, rot_half=True, head_norm=None, gate="silu", device=device)
        ff = norm2 = None
        f, q = lc.mlp, f"l{i}.mlp."
        if f is not None:
            norm2 = w[f"l{i}.norm2"]
            if f.kind == "dense":
                ff = DenseRelu2(w[q + "up"], w[q + "down"], device=device)
            else:
                E, r = f.router.experts, f.router
                shared = (w[q + "shared.gate"], w[q + "shared.up"], w[q + "shared.down"]) if f.shared is not None else None
                ff = RoutedExperts(w[q + "router"], [w[q + f"e{e}.gate"] for e in range(E)], [w[q + f"e{e}.up"] for e in range(E)],
                                   [w[q + f"e{e}.down"] for e in range(E)], top=r.top, shared=shared, device=device,
                                   limit=f.expert.limit, shared_limit=f.shared.limit if f.shared is not None else None,
                                   softmax_all=True, identity=r.identity, correction=w.get(q + "correction"),
                                   groups=(r.groups.count, r.groups.keep) if r.groups is not None else None, route_scale=r.scale,
                                   shared_gate=w.get(q + "shared.sg") if f.shared is not None else None)
        layers.append(StreamLayer(w[f"l{i}.norm1"], residual, mixer, ff, norm2, residual if ff is not None else None, device=device,
                                  parallel=True, rms=True))
    return layers, RmsNorm(w["final.norm"], device)


@dataclass
class Request:
    name: str
    prompt: list[int]
    max_new_tokens: int
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int | None = None
    eos: int | None = None
    output: list[int] = field(default_factory=list)
    fed: int = 0                      # prompt tokens already in the state
    seq: Sequence | None = None
    done: bool = False


class Scheduler:
    """Continuous batching over one engine: every iteration is one ``LMEngine.step`` over the decode rows of the running
    requests and as many prompt rows (whole prompts or portions) as ``max_step_tokens`` leaves room for."""

    def __init__(self, model: "CausalLM", max_step_tokens: int | None = None):
        self.model = model
        self.max_step_tokens = int(max_step_tokens or model.engine.max_rows)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []

    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError("a request needs at least one prompt token")
        self.waiting.append(req)

    def _admit(self) -> None:
        st = self.model.state
        while self.waiting and st.free_slots > 0:
            req = self.waiting[0]
            # room for the whole prompt and the tokens it may generate, so a running request never starves
            if st.pages_needed(None, len(req.prompt) + req.max_new_tokens) > st.free_pages - self._promised():
                break
            self.waiting.popleft()
            req.seq = st.open(req.name)
            self.running.append(req)

    def _promised(self) -> int:
        st = self.model.state
        return sum(st.pages_needed(r.seq, len(r.prompt) + r.max_new_tokens - r.seq.length) for r in self.running)

    def iterate(self) -> list[Request]:
        """One engine step; returns the requests that finished in it."""
        self._admit()
        if not self.running:
            if self.waiting:
                raise OutOfPages("the first waiting request does not fit the sequence state")
            return []
        budget, entries, sampled = self.max_step_tokens, [], []
        for req in self.running:                               # decode rows first: they are one token each
            if req.fed == len(req.prompt) and budget > 0:
                entries.append((req.seq, [req.output[-1]], [0]))
                sampled.append(req)
                budget -= 1
        for req in self.running:
            if req.fed < len(req.prompt) and budget > 0:
                n = min(budget, len(req.prompt) - req.fed)
                last = req.fed + n == len(req.prompt)
                entries.append((req.seq, req.prompt[req.fed:req.fed + n], [n - 1] if last else []))
                req.fed += n
                budget -= n
                if last:
                    sampled.append(req)
        logits = self.model.engine.step(entries)
        tokens = self.model.sample(logits, sampled).tolist() if sampled else []
        finished = []
        for req, tok in zip(sampled, tokens):
            req.output.append(int(tok))
            if len(req.output) >= req.max_new_tokens or (req.eos is not None and tok == req.eos):
                req.done = True
                finished.append(req)
        for req in finished:
            self.running.remove(req)
            self.model.state.close(req.name)
        return finished

    def run(self) -> None:
        while self.waiting or self.running:
            self.iterate()


class CausalLM:
    def __init__(self, cfg: PubopelConfig | KupelixConfig | LuketarConfig | FipadraConfig, weights: dict[str, torch.Tensor], dtype: str = "bfloat16", device=None,
                 max_tokens: int = 4096, max_sequences: int = 8, page_size: int = 16, max_rows: int = 1024,
                 max_sequence_tokens: int | None = None, step_graphs: bool = True):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        if not torch.cuda.is_available():
            raise RuntimeError("the language-model path needs a CUDA device (sm_100a); there is no CPU fallback")
        cfg.check()
        self.config, self.dtype = cfg, dtype
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        # a design is its layer records (in execution order), its final norm and the constants around them
        embed_scale, head, embed_norm = 1.0, weights.get("head"), None
        if isinstance(cfg, FipadraConfig):
            self.layers, final_norm = build_fipadra_layers(cfg, weights, self.device)
            taps, logit_scale = 0, cfg.logit_scale
            head, embed_norm = weights["embed"], weights["embed.norm"]    # logits against the table itself; a norm behind the lookup
        elif isinstance(cfg, KupelixConfig):
            self.layers, final_norm = build_kupelix_layers(cfg, weights, self.device)
            taps, logit_scale = 0, cfg.logit_scale
        elif isinstance(cfg, LuketarConfig):
            self.layers, final_norm = build_luketar_layers(cfg, weights, self.device)
            taps, logit_scale, embed_scale = 0, 1.0, cfg.embedding.scale
            head = weights["embed"]                             # the logits are taken against the embedding table itself
        else:
            self.layers, final_norm = build_pubopel_layers(cfg, weights, self.device)
            taps, logit_scale = cfg.canon.taps, 1.0
        self.state = PagedState([layer.state_spec() for layer in self.layers], cfg.width, taps, max_tokens, self.device,
                                page_size=page_size, max_sequences=max_sequences, max_sequence_tokens=max_sequence_tokens)
        # float32: every product is fp32 arithmetic on the stored (bfloat16) weights.  bfloat16: the products of prompt
        # portions run on the tensor cores with bfloat16 operands and fp32 accumulation.  Norms, scores, the router, the
        # pages, recurrent states and the residual stream are float32 in both.
        self.engine = LMEngine(self.layers, weights["embed"], head, final_norm, width=cfg.width, vocab=cfg.vocab,
                               taps=taps, eps=cfg.norm.eps, state=self.state, max_rows=max_rows, precision=dtype,
                               step_graphs=step_graphs, logit_scale=logit_scale, embed_scale=embed_scale, embed_norm=embed_norm)
        self._draws = 0

    @classmethod
    def from_pretrained(cls, folder: str | Path, dtype: str = "bfloat16", device=None, **kw) -> "CausalLM":
        folder = Path(folder)
        cfg = load_config(json.loads((folder / "config.json").read_text(encoding="utf-8")))
        return cls(cfg, load_safetensors(folder / "model.safetensors"), dtype=dtype, device=device, **kw)

    # ---- teacher-forced stepping (trace replay, scoring) -------------------------------------------------------
    def run_step(self, entries: list[dict], end: list[str] = (), keep_layers: bool = False):
        """``entries``: ``{"id", "tokens", "want"}`` per request - its next tokens and the places among them whose logits
        are wanted.  A new id opens a sequence; ids in ``end`` are closed after the step.  Returns float32 logits
        ``[wanted, vocab]`` on the device."""
        rows, opened = [], []
        try:
            for ent in entries:
                seq = self.state.sequences.get(ent["id"])
                if seq is None:
                    seq = self.state.open(ent["id"])
                    opened.append(ent["id"])
                rows.append((seq, [int(t) for t in ent["tokens"]], [int(k) for k in ent.get("want", [])]))
            out = self.engine.step(rows, keep_layers=keep_layers)
        except OutOfPages:
            for name in opened:                                 # a request that does not fit leaves nothing behind
                self.state.close(name)
            raise
        for name in end:
            if name in self.state.sequences:
                self.state.close(name)
        return out

    # ---- sampling ------------------------------------------------------------------------------------------------
    def sample(self, logits: torch.Tensor, reqs: list[Request]) -> torch.Tensor:
        """Greedy rows through the argmax kernel; the others through the framework's sampling helper."""
        out = self.engine.argmax(logits)
        hot = [i for i, r in enumerate(reqs) if r.temperature > 0.0]
        if hot:
            from .model import _sample_next_token
            for i in hot:
                r = reqs[i]
                out[i] = _sample_next_token(logits[i:i + 1], r.temperature, r.top_p, r.top_k)[0].to(torch.int32)
        return out

    # ---- generation ------------------------------------------------------------------------------------------------
    @torch.inference_mode()
    def generate(self, prompts: list[list[int]], max_new_tokens: int = 16, temperature: float = 0.0, top_p: float = 1.0,
                 top_k: int | None = None, eos: int | None = None, seed: int | None = None,
                 max_step_tokens: int | None = None) -> list[list[int]]:
        """Continues every prompt (token ids) by up to ``max_new_tokens`` tokens; greedy when ``temperature`` is 0."""
        if seed is not None:
            torch.manual_seed(seed)
        sched = Scheduler(self, max_step_tokens)
        reqs = [Request(name=f"g{self._draws}_{i}", prompt=[int(t) for t in p], max_new_tokens=int(max_new_tokens),
                        temperature=float(temperature), top_p=float(top_p), top_k=top_k, eos=eos) for i, p in enumerate(prompts)]
        self._draws += 1
        for r in reqs:
            sched.add(r)
        sched.run()
        return [r.output for r in reqs]
