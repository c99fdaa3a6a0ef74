"""The rows of one step and their metadata, on the host and on the device.

A step is a list of (request, its next tokens, wanted places).  All rows are laid end
to end, ``[T]``; per sequence the step records where its rows start, how many
positions the cache already holds, its state slot and its block-table row.  Everything
is packed into ONE int32 staging block in pinned host memory and copied to the device
with one transfer; the kernels read slices of that block.  The layout depends only on
(T, S, table width), so a captured step of the same shape finds every array at the same
address.

The reference uploads ids, positions and bounds as three small arrays and packs page
tables with device-to-device copies (crates/shiso-engine/src/stack.rs:513-544,843-870;
crates/shiso-engine/src/rows.rs:92-111), always after pages were claimed and before any
launch (stack.rs:1018-1033); the same order is kept here.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places (indices into
    ``tokens``) whose logits are wanted."""

    request: object
    tokens: Sequence[int]
    want: Sequence[int] = ()
    # The entry's one token is not known on the host: the device reads it from this index of the
    # engine's ``fed_tokens`` buffer (where a sampler left it a step earlier); ``tokens`` then
    # holds a placeholder.
    feed: Optional[int] = None
    # Values of the model's further per-row inputs (``ModelPlan.row_inputs``): name -> one int per
    # token of this entry.  A name that is left out gets the rows' positions.
    extras: Optional[dict] = None


@dataclass
class StepMeta:
    """Device arrays (int32) of one step plus the host facts kernels are launched with."""

    num_tokens: int
    num_seqs: int
    num_wanted: int
    token_ids: torch.Tensor  # [T]
    positions: torch.Tensor  # [T] absolute position of each row
    seq_of_token: torch.Tensor  # [T] index of the row's sequence in this step
    q_start: torch.Tensor  # [S + 1] first row of each sequence
    start_pos: torch.Tensor  # [S] positions the cache held before this step
    state_slots: torch.Tensor  # [S]
    want_rows: torch.Tensor  # [W] rows whose logits are wanted
    block_tables: list  # per paged group: [S, width]
    max_q_len: int
    max_context: int  # most positions any sequence can see after this step
    all_decode: bool  # every sequence brings exactly one token
    wants_every_row: bool = False  # want_rows is 0, 1, .. T-1: logits of all rows, in order
    feed_index: Optional[torch.Tensor] = None  # [T] index into fed_tokens, or -1: the id in token_ids stands
    fed_tokens: Optional[torch.Tensor] = None  # the engine's buffer of tokens picked on the device
    extras: dict = field(default_factory=dict)  # name -> [T] int32, the model's further per-row inputs
    h_q_start: list = field(default_factory=list)
    h_start_pos: list = field(default_factory=list)
    h_state_slots: list = field(default_factory=list)
    requests: list = field(default_factory=list)


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class MetaLayout:
    """Offsets (in int32 elements) of every array inside the staging block."""

    def __init__(self, num_tokens: int, num_seqs: int, num_wanted_cap: int, num_groups: int, width: int, num_extras: int = 0):
        t, s = _align(num_tokens), _align(num_seqs)
        self.token_ids = 0
        self.positions = t
        self.seq_of_token = 2 * t
        self.feed_index = 3 * t
        self.q_start = 4 * t
        self.start_pos = self.q_start + _align(num_seqs + 1)
        self.state_slots = self.start_pos + s
        self.want_rows = self.state_slots + s
        self.tables = self.want_rows + _align(num_wanted_cap)
        self.table_elems = _align(num_seqs * width)
        self.extras = self.tables + num_groups * self.table_elems  # num_extras arrays of t entries
        self.extra_elems = t
        self.total = self.extras + num_extras * t


class StepBuilder:
    """Builds ``StepMeta`` from entries and the cache manager's holdings."""

    def __init__(self, cache, device, max_tokens: int, max_seqs: int, fixed_table_width: Optional[int] = None,
                 row_inputs: Sequence[str] = ()):
        self.cache = cache
        self.row_inputs = tuple(row_inputs)
        self.device = torch.device(device)
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs
        self.num_groups = len(cache.groups)
        self.fixed_width = fixed_table_width
        width = fixed_table_width or cache.max_blocks
        cap = MetaLayout(max_tokens, max_seqs, max_tokens, self.num_groups, width, len(self.row_inputs)).total
        pin = self.device.type == "cuda"
        self._staging = [torch.zeros(cap, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._events = [None, None]
        self._turn = 0
        self.device_block = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self._arange = np.arange(max_seqs + 2, dtype=np.int32)
        self.fed_tokens: Optional[torch.Tensor] = None  # set by the engine; None: steps carry no feed arrays
        self.ops = None  # set by the engine: the kernels, whose ``words_from_host`` (if any) moves small blocks

    KERNEL_COPY_MAX_WORDS = 16384  # larger blocks (long prompt steps) take the copy engine

    def _to_device(self, stage: torch.Tensor, words: int) -> None:
        """The step's block from its pinned staging buffer to the device, in the stream: a small
        block as loads of a kernel that reads the host's memory in place (no turn of the copy
        engine before the step's first kernel), a large one or any the kernel refuses as a copy."""
        from_host = getattr(self.ops, "words_from_host", None) if self.ops is not None else None
        if from_host is not None and words <= self.KERNEL_COPY_MAX_WORDS and from_host(stage, self.device_block[:words]):
            return
        self.device_block[:words].copy_(stage[:words], non_blocking=True)

    def _iota(self, n: int) -> np.ndarray:
        return self._arange[:n]

    def _fill_extras(self, host, lay, entries, q_start, num_tokens: int) -> None:
        """The model's further per-row inputs: the rows' positions unless an entry brings values."""
        for j, name in enumerate(self.row_inputs):
            at = lay.extras + j * lay.extra_elems
            host[at : at + num_tokens] = host[lay.positions : lay.positions + num_tokens]
            for i, e in enumerate(entries):
                values = e.extras.get(name) if e.extras else None
                if values is None:
                    continue
                a, b = int(q_start[i]), int(q_start[i + 1])
                if len(values) != b - a:
                    raise ValueError(f"request {e.request!r}: {len(values)} values of {name!r} for {b - a} tokens")
                host[at + a : at + b] = values

    def _extras(self, part, lay, num_tokens: int) -> dict:
        return {name: part(lay.extras + j * lay.extra_elems, num_tokens) for j, name in enumerate(self.row_inputs)}

    def build(self, entries: Sequence[StepEntry], starts: Sequence[int], pad=None) -> StepMeta:
        """``starts[i]`` = positions the cache held for entry ``i`` before this step.

        ``pad = (tokens, sequences, wanted)`` fills the step up to a captured shape: behind the
        entries come made-up sequences (token 0 from position 0) that read and write only the
        cache manager's scratch pages and scratch slot, all but the last of one row; wanted rows
        are filled up with row 0.  The entries' rows, sequences and wanted rows keep their
        places, so the first ``sum(len(e.want))`` rows of the logits are theirs."""
        if pad is not None:
            return self._build_padded(entries, starts, pad)
        num_seqs = len(entries)
        lens = [len(e.tokens) for e in entries]
        num_tokens = sum(lens)
        num_wanted = sum(len(e.want) for e in entries)
        if num_seqs == 0 or num_tokens == 0:
            raise ValueError("a step needs at least one token")
        if num_tokens > self.max_tokens or num_seqs > self.max_seqs:
            raise ValueError(
                f"step of {num_tokens} tokens in {num_seqs} sequences exceeds the engine's "
                f"limits ({self.max_tokens} tokens, {self.max_seqs} sequences)"
            )
        requests = [e.request for e in entries]
        width = self.fixed_width or self.cache.max_blocks_held(requests)
        lay = MetaLayout(num_tokens, num_seqs, num_wanted, self.num_groups, width, len(self.row_inputs))

        turn = self._turn
        self._turn ^= 1
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        stage = self._staging[turn]
        host = stage.numpy()

        slots = [self.cache.slot_of(r) for r in requests]
        host[lay.start_pos : lay.start_pos + num_seqs] = starts
        host[lay.state_slots : lay.state_slots + num_seqs] = slots
        single = num_tokens == num_seqs  # every sequence brings one token: rows and sequences coincide
        every_row = False
        if single:
            rows = self._iota(num_seqs + 1)
            q_start = rows
            host[lay.q_start : lay.q_start + num_seqs + 1] = rows
            host[lay.token_ids : lay.token_ids + num_seqs] = [e.tokens[0] for e in entries]
            host[lay.positions : lay.positions + num_seqs] = starts
            host[lay.seq_of_token : lay.seq_of_token + num_seqs] = rows[:num_seqs]
            host[lay.feed_index : lay.feed_index + num_seqs] = [-1 if e.feed is None else e.feed for e in entries]
            want_at = lay.want_rows
            every_row = num_wanted == num_seqs and all(len(e.want) == 1 and e.want[0] == 0 for e in entries)
            if every_row:
                host[want_at : want_at + num_seqs] = rows[:num_seqs]
            else:
                for i, e in enumerate(entries):
                    for w in e.want:
                        if w != 0:
                            raise ValueError(f"request {e.request!r}: wanted place {w} is outside its 1 tokens")
                        host[want_at] = i
                        want_at += 1
        else:
            q_start = np.zeros(num_seqs + 1, dtype=np.int32)
            np.cumsum(lens, out=q_start[1:])
            host[lay.q_start : lay.q_start + num_seqs + 1] = q_start
        want_at = lay.want_rows
        for i, e in enumerate(entries if not single else ()):
            a, b = int(q_start[i]), int(q_start[i + 1])
            host[lay.token_ids + a : lay.token_ids + b] = e.tokens
            host[lay.positions + a : lay.positions + b] = np.arange(starts[i], starts[i] + lens[i], dtype=np.int32)
            host[lay.seq_of_token + a : lay.seq_of_token + b] = i
            host[lay.feed_index + a : lay.feed_index + b] = -1
            if e.feed is not None:
                if lens[i] != 1:
                    raise ValueError(f"request {e.request!r}: only a single token can be fed from the device")
                host[lay.feed_index + a] = e.feed
            for w in e.want:
                if not 0 <= w < lens[i]:
                    raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {lens[i]} tokens")
                host[want_at] = a + w
                want_at += 1
        for g in range(self.num_groups):
            at = lay.tables + g * lay.table_elems
            self.cache.fill_block_tables(requests, g, host[at : at + num_seqs * width].reshape(num_seqs, width))

        if self.row_inputs:
            self._fill_extras(host, lay, entries, q_start, num_tokens)
        dev = self.device_block
        self._to_device(stage, lay.total)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._events[turn] = ev

        def part(at, n):
            return dev[at : at + n]

        return StepMeta(
            num_tokens=num_tokens,
            num_seqs=num_seqs,
            num_wanted=num_wanted,
            token_ids=part(lay.token_ids, num_tokens),
            positions=part(lay.positions, num_tokens),
            seq_of_token=part(lay.seq_of_token, num_tokens),
            q_start=part(lay.q_start, num_seqs + 1),
            start_pos=part(lay.start_pos, num_seqs),
            state_slots=part(lay.state_slots, num_seqs),
            want_rows=part(lay.want_rows, num_wanted),
            block_tables=[
                part(lay.tables + g * lay.table_elems, num_seqs * width).view(num_seqs, width)
                for g in range(self.num_groups)
            ],
            max_q_len=max(lens),
            max_context=max(s + n for s, n in zip(starts, lens)),
            all_decode=all(n == 1 for n in lens),
            wants_every_row=single and every_row,
            feed_index=part(lay.feed_index, num_tokens) if self.fed_tokens is not None else None,
            fed_tokens=self.fed_tokens,
            extras=self._extras(part, lay, num_tokens),
            h_q_start=q_start.tolist(),
            h_start_pos=list(starts),
            h_state_slots=slots,
            requests=requests,
        )

    def _build_padded(self, entries, starts, pad) -> StepMeta:
        pad_tokens, pad_seqs, pad_wanted = pad
        cache = self.cache
        # a step of single tokens that all want their row stays one when every made-up sequence
        # brings one row too: the kernels for such steps serve it
        decode = pad_tokens == pad_seqs == pad_wanted and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        if self.fixed_width is None or cache.scratch_slot is None:
            raise RuntimeError("a padded step needs a builder with a fixed table width and a cache with scratch pages")
        real_seqs = len(entries)
        lens = [len(e.tokens) for e in entries]
        real_tokens = sum(lens)
        real_wanted = sum(len(e.want) for e in entries)
        made_up = pad_seqs - real_seqs
        spare = pad_tokens - real_tokens
        fits = (made_up == 0 and spare == 0) or (made_up >= 1 and spare >= made_up)
        if not fits or pad_wanted < real_wanted or pad_tokens > self.max_tokens or pad_seqs > self.max_seqs:
            raise ValueError(f"a step of {real_tokens} tokens in {real_seqs} sequences does not fit the shape {pad}")
        last = spare - (made_up - 1) if made_up else 0  # rows of the last made-up sequence
        if last > len(cache.scratch_pages) * cache.page_size:
            raise ValueError(f"{last} padding rows in one sequence exceed the cache's scratch pages")
        lens = lens + ([1] * (made_up - 1) + [last] if made_up else [])
        starts = list(starts) + [0] * made_up
        width = self.fixed_width
        lay = MetaLayout(pad_tokens, pad_seqs, pad_wanted, self.num_groups, width, len(self.row_inputs))

        turn = self._turn
        self._turn ^= 1
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        stage = self._staging[turn]
        host = stage.numpy()
        requests = [e.request for e in entries]
        slots = [cache.slot_of(r) for r in requests] + [cache.scratch_slot] * made_up
        host[lay.start_pos : lay.start_pos + pad_seqs] = starts
        host[lay.state_slots : lay.state_slots + pad_seqs] = slots
        q_start = np.zeros(pad_seqs + 1, dtype=np.int32)
        np.cumsum(lens, out=q_start[1:])
        host[lay.q_start : lay.q_start + pad_seqs + 1] = q_start
        host[lay.token_ids + real_tokens : lay.token_ids + pad_tokens] = 0
        host[lay.feed_index : lay.feed_index + pad_tokens] = -1
        want_at = lay.want_rows
        for i in range(pad_seqs):
            a, b = int(q_start[i]), int(q_start[i + 1])
            host[lay.positions + a : lay.positions + b] = np.arange(starts[i], starts[i] + lens[i], dtype=np.int32)
            host[lay.seq_of_token + a : lay.seq_of_token + b] = i
            if i >= real_seqs:
                continue
            e = entries[i]
            host[lay.token_ids + a : lay.token_ids + b] = e.tokens
            if e.feed is not None:
                if lens[i] != 1:
                    raise ValueError(f"request {e.request!r}: only a single token can be fed from the device")
                host[lay.feed_index + a] = e.feed
            for w in e.want:
                if not 0 <= w < lens[i]:
                    raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {lens[i]} tokens")
                host[want_at] = a + w
                want_at += 1
        if decode:
            host[lay.want_rows : lay.want_rows + pad_wanted] = self._iota(pad_wanted) if pad_wanted <= len(self._arange) else np.arange(pad_wanted)
        else:
            host[want_at : lay.want_rows + pad_wanted] = 0
        scratch = np.resize(np.asarray(cache.scratch_pages, dtype=np.int32), width)
        for g in range(self.num_groups):
            at = lay.tables + g * lay.table_elems
            tables = host[at : at + pad_seqs * width].reshape(pad_seqs, width)
            cache.fill_block_tables(requests, g, tables[:real_seqs])
            tables[real_seqs:] = scratch

        if self.row_inputs:
            self._fill_extras(host, lay, entries, q_start, pad_tokens)
        dev = self.device_block
        self._to_device(stage, lay.total)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._events[turn] = ev

        def part(at, n):
            return dev[at : at + n]

        return StepMeta(
            num_tokens=pad_tokens,
            num_seqs=pad_seqs,
            num_wanted=pad_wanted,
            token_ids=part(lay.token_ids, pad_tokens),
            positions=part(lay.positions, pad_tokens),
            seq_of_token=part(lay.seq_of_token, pad_tokens),
            q_start=part(lay.q_start, pad_seqs + 1),
            start_pos=part(lay.start_pos, pad_seqs),
            state_slots=part(lay.state_slots, pad_seqs),
            want_rows=part(lay.want_rows, pad_wanted),
            block_tables=[
                part(lay.tables + g * lay.table_elems, pad_seqs * width).view(pad_seqs, width)
                for g in range(self.num_groups)
            ],
            max_q_len=max(lens),
            max_context=max(s + n for s, n in zip(starts, lens)),
            all_decode=decode,
            wants_every_row=decode,
            feed_index=part(lay.feed_index, pad_tokens) if self.fed_tokens is not None else None,
            fed_tokens=self.fed_tokens,
            extras=self._extras(part, lay, pad_tokens),
            h_q_start=[],  # a captured step sizes its launches by capacity, not by this step's lengths
            h_start_pos=[],
            h_state_slots=[],
            requests=requests,
        )
