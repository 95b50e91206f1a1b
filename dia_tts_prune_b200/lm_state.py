"""Sequence state of the language-model path: paged K/V storage, per-sequence slots, short-convolution tails and
recurrent states.

Same role as ``state.py`` has for Dia (``KVCache`` / ``DecoderInferenceState``), but for any number of concurrent
sequences of unknown final length: a sequence owns a *slot* (a row of the page table, of every layer's tail buffers
and of every recurrent layer's state) and a list of fixed-size *pages* of the shared K/V pool, taken when its length
crosses a page border and given back when it ends.  Slots and pages are recycled last-freed-first; nothing is cleared
on reuse, because the kernels take a sequence's state as zero when its first row of a step is position 0.  What a layer
record keeps is described by a :class:`StateSpec`; a layer that runs several times per token has one record, and so
one state, per run.  The kernels read the device copy of the page table; the bookkeeping is host-side and never reads
a device tensor.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass(frozen=True)
class StateSpec:
    """What one layer record keeps per sequence (every part optional)."""
    kv: tuple[int, int, int] | None = None          # (kv_heads, key size, value size): paged keys and values
    tap_tails: int = 0                              # [taps - 1][width] tails of tap-mix sublayers
    recurrent: tuple[int, int, int] | None = None   # (heads, value size, key size): fp32 matrix state per slot
    conv: tuple[int, int] | None = None             # (taps, channels): the last taps - 1 inputs of a short convolution
    latent: int | None = None                       # size of a paged latent vector per token (keys and values are made from it)
    aux: int = 0                                    # fp32 numbers per slot beside a recurrent state (running maxima)


class OutOfPages(RuntimeError):
    """The pool cannot hold the tokens asked for (the scheduler keeps the request waiting instead)."""


@dataclass
class Sequence:
    """One live request: its slot, how many tokens its state holds, and the pages that hold them."""
    name: str
    slot: int
    length: int = 0
    pages: list[int] = field(default_factory=list)


@dataclass
class RecordState:
    k_pages: torch.Tensor | None
    v_pages: torch.Tensor | None
    tails: tuple
    rec_state: torch.Tensor | None
    conv_tail: torch.Tensor | None
    latent_pages: torch.Tensor | None = None
    rec_aux: torch.Tensor | None = None


class PagedState:
    def __init__(self, layers: list, width: int, taps: int, max_tokens: int, device: torch.device,
                 page_size: int = 16, max_sequences: int = 8, max_sequence_tokens: int | None = None):
        """``layers``: a :class:`StateSpec` per layer record, or ``(kv_heads, dim)`` for a record with keys and values of
        one size and two tap-mix tails.  ``max_tokens``: the most tokens all live sequences hold at one time; the pool gets
        that many tokens' worth of pages plus one partly filled page per slot."""
        if page_size <= 0 or max_tokens <= 0 or max_sequences <= 0:
            raise ValueError("page_size, max_tokens and max_sequences must be positive")
        self.device = torch.device(device)
        self.page_size, self.n_slots = int(page_size), int(max_sequences)
        longest = int(max_sequence_tokens or max_tokens)
        self.max_pages = -(-longest // self.page_size)
        self.n_pages = -(-int(max_tokens) // self.page_size) + self.n_slots
        self.taps = int(taps)
        self.specs = [sp if isinstance(sp, StateSpec) else StateSpec(kv=(sp[0], sp[1], sp[1]), tap_tails=2) for sp in layers]
        f32 = dict(dtype=torch.float32, device=self.device)
        # K and V pages per record: [page][kv head][page_size][size], float32 (None for a record without attention)
        self.k_pages = [torch.zeros((self.n_pages, sp.kv[0], self.page_size, sp.kv[1]), **f32) if sp.kv else None
                        for sp in self.specs]
        self.v_pages = [torch.zeros((self.n_pages, sp.kv[0], self.page_size, sp.kv[2]), **f32) if sp.kv else None
                        for sp in self.specs]
        # the last taps - 1 normed inputs of the tap-mix sublayers of every record: [slot][taps - 1][width]
        t1 = max(self.taps - 1, 1)
        self.tails = [tuple(torch.zeros((self.n_slots, t1, width), **f32) for _ in range(sp.tap_tails)) for sp in self.specs]
        # recurrent matrix states [slot][head][value channel][key channel] and short-convolution tails [slot][taps - 1][channels]
        self.rec_states = [torch.zeros((self.n_slots, sp.recurrent[0], sp.recurrent[1], sp.recurrent[2]), **f32)
                           if sp.recurrent else None for sp in self.specs]
        self.conv_tails = [torch.zeros((self.n_slots, max(sp.conv[0] - 1, 1), sp.conv[1]), **f32) if sp.conv else None
                           for sp in self.specs]
        # latent pages [page][page_size][size] share the page table with the K/V pages; per-slot numbers [slot][aux]
        self.latent_pages = [torch.zeros((self.n_pages, self.page_size, sp.latent), **f32) if sp.latent else None for sp in self.specs]
        self.rec_aux = [torch.zeros((self.n_slots, sp.aux), **f32) if sp.aux else None for sp in self.specs]
        self._table_host = torch.zeros((self.n_slots, self.max_pages), dtype=torch.int32).pin_memory() \
            if self.device.type == "cuda" else torch.zeros((self.n_slots, self.max_pages), dtype=torch.int32)
        self.page_table = torch.zeros((self.n_slots, self.max_pages), dtype=torch.int32, device=self.device)
        self._dirty = False
        self._free_pages = list(range(self.n_pages - 1, -1, -1))        # pop() takes page 0 first
        self._free_slots = list(range(self.n_slots - 1, -1, -1))
        self.sequences: dict[str, Sequence] = {}

    def record_state(self, i: int) -> "RecordState":
        """The buffers of layer record ``i`` (what its ``fill`` points the kernels at)."""
        return RecordState(self.k_pages[i], self.v_pages[i], self.tails[i], self.rec_states[i], self.conv_tails[i],
                           self.latent_pages[i], self.rec_aux[i])

    # ---- bookkeeping -----------------------------------------------------------------------------------------
    @property
    def free_pages(self) -> int:
        return len(self._free_pages)

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def pages_needed(self, seq: Sequence | None, new_tokens: int) -> int:
        have = len(seq.pages) if seq is not None else 0
        length = seq.length if seq is not None else 0
        return max(0, -(-(length + new_tokens) // self.page_size) - have)

    def open(self, name: str) -> Sequence:
        if name in self.sequences:
            raise ValueError(f"sequence {name!r} is already open")
        if not self._free_slots:
            raise OutOfPages("no free sequence slot")
        seq = Sequence(name=name, slot=self._free_slots.pop())
        self.sequences[name] = seq
        return seq

    def reserve(self, seq: Sequence, new_tokens: int) -> None:
        """Make room for ``new_tokens`` more tokens of ``seq`` (takes pages; the length moves in :meth:`advance`)."""
        need = self.pages_needed(seq, new_tokens)
        if len(seq.pages) + need > self.max_pages:
            raise OutOfPages(f"sequence {seq.name!r} would exceed {self.max_pages * self.page_size} tokens")
        if need > len(self._free_pages):
            raise OutOfPages(f"{need} pages needed, {len(self._free_pages)} free")
        for _ in range(need):
            p = self._free_pages.pop()
            self._table_host[seq.slot, len(seq.pages)] = p
            seq.pages.append(p)
            self._dirty = True

    def advance(self, seq: Sequence, new_tokens: int) -> None:
        seq.length += int(new_tokens)

    def close(self, name: str) -> None:
        """Give a finished sequence's pages and slot back."""
        seq = self.sequences.pop(name)
        self._free_pages.extend(reversed(seq.pages))
        self._free_slots.append(seq.slot)
        seq.pages = []

    def sync_table(self) -> torch.Tensor:
        """The device page table, refreshed if pages were taken since the last call (stream-ordered copy)."""
        if self._dirty:
            self.page_table.copy_(self._table_host, non_blocking=True)
            self._dirty = False
        return self.page_table
