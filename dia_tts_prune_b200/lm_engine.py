"""Python face of ``liblm_b200.so``: the step function of the decoder-only language-model path.

``LMEngine.step`` takes the rows the scheduler picked - for each scheduled sequence its next tokens, a prompt portion
or one decoded token alike - lays them out as one flat batch, and runs them through the kernels in portions of at most
``max_rows`` rows.  All arithmetic is in ``csrc/``; there is no eager / CPU fallback here.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lm_lib
from .lm_layers import DynamicTanh, LayerNorm, MixLayer, RmsNorm
from .lm_state import PagedState, Sequence


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def launch_count() -> int:
    return int(_lm_lib.load().lm_b200_launch_count())


class LMEngine:
    def __init__(self, layers: list, embed: torch.Tensor, head: torch.Tensor, final_norm: DynamicTanh | LayerNorm | RmsNorm, *,
                 width: int, vocab: int, taps: int, eps: float, state: PagedState, max_rows: int = 1024,
                 precision: str = "bfloat16", step_graphs: bool = True, logit_scale: float = 1.0, embed_scale: float = 1.0,
                 embed_norm: torch.Tensor | None = None):
        """``layers``: the layer records in execution order (a layer that runs twice per token appears twice, each time
        with the state record of its own index)."""
        if not torch.cuda.is_available():
            raise RuntimeError("the language-model path needs a CUDA device (sm_100a); there is no CPU fallback")
        self.lib = _lm_lib.load()
        self.device = state.device
        if self.device.type != "cuda":
            raise RuntimeError("the sequence state must live on a CUDA device")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.layers, self.state = layers, state
        self.embed = embed.detach().to(device=self.device, dtype=torch.bfloat16).contiguous()
        self.head = head.detach().to(device=self.device, dtype=torch.bfloat16).contiguous()
        self.final_norm = final_norm
        self.width, self.vocab, self.max_rows = int(width), int(vocab), int(max_rows)
        m = _lm_lib.Model()
        m.n_layer, m.width, m.vocab, m.taps = len(layers), self.width, self.vocab, int(taps)
        m.page_size, m.max_pages, m.n_slots, m.max_rows = state.page_size, state.max_pages, state.n_slots, self.max_rows
        m.eps = float(eps)
        if precision not in ("bfloat16", "float32"):
            raise ValueError("precision must be 'bfloat16' or 'float32'")
        self.precision = precision
        m.precision = _lm_lib.PRECISION_BF16 if precision == "bfloat16" else _lm_lib.PRECISION_FP32
        m.embed, m.head = self.embed.data_ptr(), self.head.data_ptr()
        final_norm.fill(m.final_norm)
        m.page_table = state.page_table.data_ptr()
        m.step_graphs = 1 if step_graphs else 0
        m.logit_scale = float(logit_scale)
        m.embed_scale = float(embed_scale)
        # an RMS norm weight on the embedding rows (stream records only)
        self.embed_norm = None if embed_norm is None else embed_norm.detach().to(device=self.device, dtype=torch.float32).contiguous()
        m.embed_norm = self.embed_norm.data_ptr() if self.embed_norm is not None else None
        recs = (_lm_lib.Layer * len(layers))()
        for i, layer in enumerate(layers):
            layer.fill(recs[i], state.record_state(i))
        self._h = C.c_void_p()
        _lm_lib.check(self.lib.lm_b200_engine_create(C.byref(m), recs, self.device.index, C.byref(self._h)), "engine_create")
        self.workspace_bytes = int(self.lib.lm_b200_engine_workspace_bytes(self._h))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self.lib.lm_b200_engine_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- one launch sequence over <= max_rows rows -----------------------------------------------------------
    def _pack(self, parts: list[tuple[Sequence, list[int], int, list[int]]]) -> tuple[torch.Tensor, int, int, int]:
        """parts: (sequence, tokens, position of the first token, wanted indexes into tokens) -> the step buffer."""
        n_rows = sum(len(t) for _, t, _, _ in parts)
        S = len(parts)
        want = [k for _, _, _, w in parts for k in w]
        buf = np.empty(4 * n_rows + 3 * S + len(want), dtype=np.int32)
        tok, slot, pos, start = (buf[i * n_rows:(i + 1) * n_rows] for i in range(4))
        meta, r0, at = buf[4 * n_rows:], 0, 0
        for s, (seq, tokens, p0, w) in enumerate(parts):
            n = len(tokens)
            tok[r0:r0 + n] = tokens
            slot[r0:r0 + n] = seq.slot
            pos[r0:r0 + n] = np.arange(p0, p0 + n, dtype=np.int32)
            start[r0:r0 + n] = p0
            meta[s], meta[S + s], meta[2 * S + s] = seq.slot, r0, n
            for k in w:
                meta[3 * S + at] = r0 + k
                at += 1
            r0 += n
        t = torch.from_numpy(buf)
        if buf.size > 4096:                                     # a long step: asynchronous copy from pinned memory
            t = t.pin_memory()
        return t.to(self.device, non_blocking=True), n_rows, S, len(want)

    def _forward(self, parts, logits_out: torch.Tensor | None, layers_out: torch.Tensor | None = None) -> None:
        buf, M, S, W = self._pack(parts)
        self.state.sync_table()
        _lm_lib.check(self.lib.lm_b200_forward(
            self._h, buf.data_ptr(), M, S, W, logits_out.data_ptr() if W else None,
            layers_out.data_ptr() if layers_out is not None else None, _stream(self.device)), "forward")
        self._keep = buf                                        # stays alive until the next call is queued behind it

    def step(self, entries: list[tuple[Sequence, list[int], list[int]]], keep_layers: bool = False):
        """entries: (sequence, its next tokens, indexes among them whose logits are wanted).  Appends the tokens to the
        sequences' state and returns float32 logits ``[wanted, vocab]`` in the order of the entries (and, with
        ``keep_layers``, the residual stream after every layer for all rows)."""
        n_want = sum(len(w) for _, _, w in entries)
        total = sum(len(t) for _, t, _ in entries)
        logits = torch.empty((n_want, self.vocab), dtype=torch.float32, device=self.device)
        streams = torch.empty((len(self.layers), total, self.width), dtype=torch.float32, device=self.device) if keep_layers else None
        if keep_layers and total > self.max_rows:
            raise ValueError("keep_layers needs the whole step in one portion")
        for seq, tokens, _ in entries:
            self.state.reserve(seq, len(tokens))
        parts, rows, done = [], 0, 0

        def flush():
            nonlocal parts, rows, done
            if not parts:
                return
            w = sum(len(p[3]) for p in parts)
            self._forward(parts, logits[done:done + w] if w else None, streams)
            done += w
            parts, rows = [], 0

        order, base = [], 0                                     # logits are produced in row order; `want` may not be
        for _, _, want in entries:
            order += [base + k for k in sorted(range(len(want)), key=lambda i: want[i])]
            base += len(want)
        for seq, tokens, want in entries:
            at, want = 0, sorted(want)
            if want and (want[0] < 0 or want[-1] >= len(tokens)):
                raise ValueError("a wanted place lies outside the entry's tokens")
            while at < len(tokens):
                n = min(len(tokens) - at, self.max_rows - rows)
                parts.append((seq, list(tokens[at:at + n]), seq.length, [k - at for k in want if at <= k < at + n]))
                self.state.advance(seq, n)
                rows += n
                at += n
                if rows == self.max_rows:
                    flush()
        flush()
        if order != list(range(n_want)):
            inverse = [0] * n_want
            for produced, asked in enumerate(order):
                inverse[asked] = produced
            logits = logits[torch.tensor(inverse, device=self.device)]
        return (logits, streams) if keep_layers else logits

    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        if logits.shape[0]:
            _lm_lib.check(self.lib.lm_b200_argmax_rows(logits.data_ptr(), logits.shape[0], logits.shape[1], out.data_ptr(),
                                                       _stream(self.device)), "argmax_rows")
        return out

    # ---- operator boundaries (one mechanism at a time; used by the parity tests) ----------------------------------
    def op_norm_tapmix(self, layer: int, sub: int, x: torch.Tensor, parts) -> torch.Tensor:
        buf, M, S, _ = self._pack([(s, [0] * n, p0, []) for s, n, p0 in parts])
        x = x.to(device=self.device, dtype=torch.float32).contiguous()
        out = torch.empty_like(x)
        _lm_lib.check(self.lib.lm_b200_op_norm_tapmix(self._h, layer, sub, x.data_ptr(), buf.data_ptr(), M, S, out.data_ptr(),
                                                      _stream(self.device)), "op_norm_tapmix")
        return out

    def op_mixer(self, layer: int, h: torch.Tensor, parts) -> torch.Tensor:
        buf, M, S, _ = self._pack([(s, [0] * n, p0, []) for s, n, p0 in parts])
        self.state.sync_table()
        h = h.to(device=self.device, dtype=torch.float32).contiguous()
        y = torch.empty((M, self.width), dtype=torch.float32, device=self.device)
        _lm_lib.check(self.lib.lm_b200_op_mixer(self._h, layer, h.data_ptr(), buf.data_ptr(), M, S, y.data_ptr(),
                                                _stream(self.device)), "op_mixer")
        return y

    def op_attention(self, layer: int, qk: torch.Tensor, parts) -> torch.Tensor:
        """Attention of ``layer`` alone on projected rows ``qk [M, (heads + kv_heads) * dim]`` (queries, then keys), which
        are appended to the pages of their sequences; ``parts``: (sequence, rows, first position) like ``op_mixer``."""
        buf, M, S, _ = self._pack([(s, [0] * n, p0, []) for s, n, p0 in parts])
        self.state.sync_table()
        a = self.layers[layer].mixer
        qk = qk.to(device=self.device, dtype=torch.float32).contiguous().clone()
        out = torch.empty((M, a.heads * a.dim), dtype=torch.float32, device=self.device)
        _lm_lib.check(self.lib.lm_b200_op_attention(self._h, layer, qk.data_ptr(), buf.data_ptr(), M, S, out.data_ptr(),
                                                    _stream(self.device)), "op_attention")
        return out

    def op_mixer_kernels(self, layer: int, proj: torch.Tensor, parts) -> torch.Tensor:
        """The mixer kernels of a parallel-form record alone on stacked projections ``proj [M, n_in]`` (its attention or
        recurrence without the products around it); the state of the sequences in ``parts`` is appended to."""
        buf, M, S, _ = self._pack([(s, [0] * n, p0, []) for s, n, p0 in parts])
        self.state.sync_table()
        m = self.layers[layer].mixer
        proj = proj.to(device=self.device, dtype=torch.float32).contiguous().clone()
        out = torch.empty((M, m.heads * m.vdim), dtype=torch.float32, device=self.device)
        _lm_lib.check(self.lib.lm_b200_op_mixer_kernels(self._h, layer, proj.data_ptr(), buf.data_ptr(), M, S, out.data_ptr(),
                                                        _stream(self.device)), "op_mixer_kernels")
        return out

    def op_ff(self, layer: int, h: torch.Tensor) -> torch.Tensor:
        h = h.to(device=self.device, dtype=torch.float32).contiguous()
        y = torch.empty_like(h)
        _lm_lib.check(self.lib.lm_b200_op_ff(self._h, layer, h.data_ptr(), h.shape[0], y.data_ptr(), _stream(self.device)), "op_ff")
        return y


def linear(a: torch.Tensor, w_bf16: torch.Tensor, tensor_cores: bool = False) -> torch.Tensor:
    """``a [M, K] float32 @ w [N, K]^T bfloat16`` on the path's own linear kernels: fp32 FMA arithmetic, or (with
    ``tensor_cores``) ``a`` rounded to bfloat16 and the tcgen05 kernel."""
    lib = _lm_lib.load()
    a = a.to(torch.float32).contiguous()
    w = w_bf16.to(torch.bfloat16).contiguous()
    y = torch.empty((a.shape[0], w.shape[0]), dtype=torch.float32, device=a.device)
    if tensor_cores:
        ab = torch.empty(a.shape, dtype=torch.bfloat16, device=a.device)
        _lm_lib.check(lib.lm_b200_op_linear_tc(a.data_ptr(), w.data_ptr(), y.data_ptr(), ab.data_ptr(), a.shape[0], w.shape[0],
                                               a.shape[1], _stream(a.device)), "op_linear_tc")
        return y
    _lm_lib.check(lib.lm_b200_op_linear(a.data_ptr(), w.data_ptr(), y.data_ptr(), a.shape[0], w.shape[0], a.shape[1],
                                        _stream(a.device)), "op_linear")
    return y
