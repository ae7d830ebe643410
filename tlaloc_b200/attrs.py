"""The PAGED_ATTENTION operand/attribute contract, host side.

Mirrors ``io.tlaloc.ir.PagedAttentionAttrs`` (ir/src/commonMain/kotlin/io/tlaloc/ir/PagedAttentionAttrs.kt:79-286):
one parser every caller goes through, deriving the shape story from operand shapes (never from attrs) and
refusing by name what the reference refuses.  Operates on anything with ``.shape`` and ``.dtype``
(torch tensors, NumPy arrays), so it runs without a GPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

FORBIDDEN_ATTRS = ("block_size", "blockSize", "num_kv_heads", "numKvHeads")


@dataclass(frozen=True)
class PagedAttentionShape:
    """``PagedAttentionAttrs.Parsed`` (:79-138): every field derived or checked."""

    num_seqs: int
    num_heads: int
    head_dim: int
    num_blocks: int
    block_size: int
    num_kv_heads: int
    max_blocks_per_seq: int
    scale: float
    sliding_window: int | None = None
    num_tables: int | None = None
    keep_chunk: int | None = None
    return_lse: bool = False

    @property
    def rows_per_table(self) -> int:
        return self.num_seqs // self.num_tables

    def table_of(self, row: int) -> int:
        return row // self.rows_per_table

    def first_live(self, seq_len: int) -> int:
        return 0 if self.sliding_window is None else max(0, seq_len - self.sliding_window)

    @property
    def group(self) -> int:
        return self.num_heads // self.num_kv_heads

    @property
    def max_context_len(self) -> int:
        return self.max_blocks_per_seq * self.block_size


def _is_integral(dtype) -> bool:
    return str(dtype).replace("torch.", "") in ("int32", "int64")


def parse_paged_attention(query, key_cache, value_cache, block_tables, seq_lens, *, scale, sliding_window=None,
                          keep=None, return_lse=False, layer="tlaloc_b200", **other_attrs) -> PagedAttentionShape:
    """Validate the operands and attrs of one PAGED_ATTENTION and return the derived shape story."""
    q, k, v, t, l = (tuple(x.shape) for x in (query, key_cache, value_cache, block_tables, seq_lens))
    if len(q) != 3:
        raise ValueError(f"{layer}: PAGED_ATTENTION query must be rank-3 [numSeqs, numHeads, headDim], got {list(q)}")
    if len(k) != 4:
        raise ValueError(f"{layer}: PAGED_ATTENTION keyCache must be rank-4 [numBlocks, blockSize, numKvHeads, headDim], got {list(k)}")
    if v != k:
        raise ValueError(f"{layer}: PAGED_ATTENTION valueCache shape {list(v)} must match keyCache {list(k)} "
                         "(the two pools are indexed by the SAME block table)")
    if len(t) != 2:
        raise ValueError(f"{layer}: PAGED_ATTENTION blockTables must be rank-2 [numTables, maxBlocksPerSeq], got {list(t)}")
    if len(l) != 1:
        raise ValueError(f"{layer}: PAGED_ATTENTION seqLens must be rank-1 [numSeqs], got {list(l)}")
    if not _is_integral(block_tables.dtype):
        raise ValueError(f"{layer}: PAGED_ATTENTION blockTables must be an integer tensor, got {block_tables.dtype}")
    if not _is_integral(seq_lens.dtype):
        raise ValueError(f"{layer}: PAGED_ATTENTION seqLens must be an integer tensor, got {seq_lens.dtype}")
    num_seqs, num_heads, head_dim = q
    num_blocks, block_size, num_kv_heads, kd = k
    num_tables, max_blocks = t
    if kd != head_dim:
        raise ValueError(f"{layer}: PAGED_ATTENTION keyCache headDim {kd} must match query headDim {head_dim}")
    if num_tables < 1 or num_seqs % num_tables != 0:
        raise ValueError(f"{layer}: PAGED_ATTENTION blockTables has {num_tables} rows but query has {num_seqs} rows; "
                         "the tables must be one per row or one per equal group of consecutive rows")
    if l[0] != num_seqs:
        raise ValueError(f"{layer}: PAGED_ATTENTION seqLens has {l[0]} entries but query has {num_seqs} sequences")
    if num_kv_heads <= 0 or num_heads % num_kv_heads != 0:
        raise ValueError(f"{layer}: PAGED_ATTENTION numHeads {num_heads} must be a positive multiple of numKvHeads "
                         f"{num_kv_heads} (GQA grouping is derived, never an attr)")
    if block_size <= 0 or num_blocks <= 0 or max_blocks <= 0:
        raise ValueError(f"{layer}: PAGED_ATTENTION needs positive numBlocks/blockSize/maxBlocksPerSeq, got "
                         f"{num_blocks}/{block_size}/{max_blocks}")
    if scale is None or not isinstance(scale, (int, float)):
        raise ValueError(f"{layer}: PAGED_ATTENTION requires a 'scale' attr (the softmax temperature, typically "
                         f"1/sqrt(headDim)); got {scale}")
    if not math.isfinite(scale):
        raise ValueError(f"{layer}: PAGED_ATTENTION scale must be finite, got {scale}")
    for name in FORBIDDEN_ATTRS:
        if name in other_attrs:
            raise ValueError(f"{layer}: PAGED_ATTENTION attr '{name}' is refused by name: it is derived from keyCache's "
                             f"shape {list(k)}")
    if other_attrs.get("ring"):
        raise ValueError(f"{layer}: PAGED_ATTENTION 'ring' tables are outside this library's decode path")
    window = None
    if sliding_window is not None:
        if not isinstance(sliding_window, (int, float)) or sliding_window != int(sliding_window) or int(sliding_window) < 1:
            raise ValueError(f"{layer}: PAGED_ATTENTION 'sliding_window' must be a whole number >= 1, got {sliding_window}")
        window = int(sliding_window)
    if return_lse and (window is not None or keep is not None):
        raise ValueError(f"{layer}: PAGED_ATTENTION 'return_lse' is for full-attention tables, without "
                         "'sliding_window' and without a keep operand")
    keep_chunk = None
    if keep is not None:
        kt = tuple(keep.shape)
        ctx = max_blocks * block_size
        if len(kt) != 2 or kt[0] != num_seqs or not _is_integral(keep.dtype):
            raise ValueError(f"{layer}: PAGED_ATTENTION keep must be an integer [{num_seqs}, numChunks], got "
                             f"{keep.dtype}{list(kt)}")
        if kt[1] < 1 or ctx % kt[1] != 0:
            raise ValueError(f"{layer}: PAGED_ATTENTION keep has {kt[1]} chunks, which do not divide the {ctx} positions")
        keep_chunk = ctx // kt[1]
    return PagedAttentionShape(num_seqs, num_heads, head_dim, num_blocks, block_size, num_kv_heads, max_blocks,
                               float(scale), window, num_tables, keep_chunk, bool(return_lse))
