"""The caller's side of the paged KV cache: which physical page holds which positions, and the integer inputs of a step.

Mirrors the behaviour of the reference's serving backend, not its code: the page pool of one model instance
(triton/backend/sequence_mode.h:315-336: page 0 is never handed out, it is where the block tables of padding rows
point; pages are taken lowest first; a shared page goes back only when its last holder returns it) and the
derivation of a step's inputs from the sequences in it (triton/backend/sequence_mode.cc:2584-2604: tokens
right-aligned in their row, `slot = pages[pos // bs] * bs + pos % bs`, `tables[r] = pages`, `lens[r] = position + n`;
padding rows use slot -1, length 1 and page 0, ir/.../DecodeGraphSpec.kt:989-1004).  Host-side NumPy only: the
arrays go to `Decoder.set_inputs` or straight into the operators' device buffers.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

PADDING_PAGE = 0
PADDING_SLOT = -1
PADDING_LENGTH = 1


class PagePool:
    """The physical pages 1 .. num_blocks - 1 of one KV pool."""

    def __init__(self, num_blocks: int):
        if num_blocks < 2:
            raise ValueError("a pool needs page 0 (padding) and at least one page to hand out")
        self.capacity = num_blocks - 1
        self._free = set(range(1, num_blocks))
        self._extra_holders: dict[int, int] = {}

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self, n: int) -> list[int] | None:
        """`n` pages, lowest ids first; None (and nothing taken) when fewer are free."""
        if n < 0:
            raise ValueError("cannot take a negative number of pages")
        if n > len(self._free):
            return None
        pages = sorted(self._free)[:n]
        self._free.difference_update(pages)
        return pages

    def share(self, pages) -> None:
        """One more holder of each page (a cached prefix, or a sequence that starts from one)."""
        for p in pages:
            self._check_held(p)
            self._extra_holders[p] = self._extra_holders.get(p, 0) + 1

    def give(self, pages) -> None:
        """Returns pages; a shared page becomes free only when its last holder gives it back."""
        for p in pages:
            self._check_held(p)
            extra = self._extra_holders.get(p, 0)
            if extra > 0:
                if extra == 1:
                    del self._extra_holders[p]
                else:
                    self._extra_holders[p] = extra - 1
            else:
                self._free.add(p)

    def _check_held(self, p: int) -> None:
        if p == PADDING_PAGE or not 0 < p <= self.capacity:
            raise ValueError(f"page {p} is not one this pool hands out")
        if p in self._free:
            raise ValueError(f"page {p} is free: nobody holds it")


@dataclass
class Sequence:
    """One sequence's pages (logical block b lives on pages[b]) and how many tokens have their KV in the pool."""

    pages: list[int] = field(default_factory=list)
    length: int = 0

    def reserve(self, pool: PagePool, tokens: int, block_size: int) -> bool:
        """Makes room for `tokens` more tokens; False (and nothing taken) if the pool cannot supply the pages."""
        need = -(-(self.length + tokens) // block_size) - len(self.pages)
        if need <= 0:
            return True
        got = pool.take(need)
        if got is None:
            return False
        self.pages.extend(got)
        return True

    def release(self, pool: PagePool) -> None:
        pool.give(self.pages)
        self.pages, self.length = [], 0


@dataclass
class StepInputs:
    """The integer operands of one step for a batch of `rows` rows, `width` token columns each."""

    token_ids: np.ndarray     # i32 [rows, width]
    positions: np.ndarray     # i32 [rows, width]
    slot_mapping: np.ndarray  # i32 [rows, width]; -1 = no write
    block_tables: np.ndarray  # i32 [rows, max_blocks]
    seq_lens: np.ndarray      # i32 [rows]


def stage_step(work, *, rows: int, width: int, max_blocks: int, block_size: int) -> StepInputs:
    """`work` = [(sequence, tokens)] with len(work) <= rows and 1 <= len(tokens) <= width: the sequence runs `tokens`
    at positions sequence.length .. (its pages must already cover them, see Sequence.reserve).  Tokens sit
    right-aligned in their row, so the last column is always the row's newest token; rows past len(work) and the
    columns left of a short row are padding."""
    if len(work) > rows:
        raise ValueError(f"{len(work)} sequences do not fit a batch of {rows} rows")
    ids = np.zeros((rows, width), np.int32)
    pos = np.zeros((rows, width), np.int32)
    slots = np.full((rows, width), PADDING_SLOT, np.int32)
    tables = np.full((rows, max_blocks), PADDING_PAGE, np.int32)
    lens = np.full((rows,), PADDING_LENGTH, np.int32)
    for r, (seq, tokens) in enumerate(work):
        n = len(tokens)
        if not 1 <= n <= width:
            raise ValueError(f"row {r}: {n} tokens do not fit {width} columns")
        end = seq.length + n
        if end > len(seq.pages) * block_size:
            raise ValueError(f"row {r}: positions up to {end - 1} but its {len(seq.pages)} pages cover {len(seq.pages) * block_size}")
        if len(seq.pages) > max_blocks and end > max_blocks * block_size:
            raise ValueError(f"row {r}: {end} positions exceed the table width {max_blocks} x {block_size}")
        p = np.arange(seq.length, end, dtype=np.int64)
        pages = np.asarray(seq.pages, np.int64)
        ids[r, width - n:] = np.asarray(tokens, np.int32)
        pos[r, width - n:] = p
        slots[r, width - n:] = pages[p // block_size] * block_size + p % block_size
        k = min(len(seq.pages), max_blocks)
        tables[r, :k] = pages[:k]
        lens[r] = end
    return StepInputs(ids, pos, slots, tables, lens)


def commit_step(work) -> None:
    """After the step ran: the tokens' KV is in the pool."""
    for seq, tokens in work:
        seq.length += len(tokens)
