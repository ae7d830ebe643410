"""Tensor-parallel partition of the decode step across the GPUs of one box (host logic, NumPy only).

The reference never built multi-GPU serving (docs/design/SHARDED_SERVING.md:3,30-33); its design note and its
training preset agree on the split used here (SHARDED_SERVING.md:74-77 "shard the pool by head", DISTRIBUTED.md:75
tensorParallel: q/k/v/gate/up by column, o/down by row):

  q, k, v      column blocks by head: rank r owns query heads [r*H/g, (r+1)*H/g) and kv heads [r*Hkv/g, ...)
  KV pools     the Hkv axis: [P, bs, Hkv/g, D] per rank; block tables, lengths and slots are replicated
  o_proj       rows (its input is the rank's heads); partial sums meet in an all-reduce
  gate, up     column blocks of the FFN; down: the matching rows; partial sums meet in an all-reduce
  scales       follow the output axis: sliced for column blocks, whole for row blocks
  embedding, norm gains: replicated;  head: column blocks of the vocabulary, greedy candidates merged

Weights are in the reference's staged layout: int8 codes [in, out] and f32 scales [out]
(ir/src/jvmMain/.../HfStagedWeights.kt:396-461).
"""
from __future__ import annotations

import numpy as np


def check_world(num_heads: int, num_kv_heads: int, ffn: int, vocab: int, world: int) -> None:
    if world < 1 or num_heads % world or num_kv_heads % world or ffn % world:
        raise ValueError(f"tensor parallel {world} must divide heads {num_heads}, kv heads {num_kv_heads} and ffn {ffn}")
    if vocab % world:
        raise ValueError(f"tensor parallel {world} must divide the vocabulary {vocab} (pad the head)")


def _cols(codes_scales, lo, hi):
    codes, scales = codes_scales
    return np.ascontiguousarray(codes[:, lo:hi]), np.ascontiguousarray(scales[lo:hi])


def _rows(codes_scales, lo, hi):
    codes, scales = codes_scales
    return np.ascontiguousarray(codes[lo:hi, :]), scales


def shard_layer(layer: dict, num_heads: int, num_kv_heads: int, head_dim: int, ffn: int, rank: int, world: int,
                fuse_swiglu: bool = False) -> dict:
    """One layer's weights for `rank`; q|k|v and gate|up are returned fused along the output axis (gate|up as two halves,
    or, with `fuse_swiglu`, interleaved in blocks of 128 for the projection that applies SwiGLU in its epilogue)."""
    hq, hk, f = num_heads // world, num_kv_heads // world, ffn // world
    q = _cols(layer["q"], rank * hq * head_dim, (rank + 1) * hq * head_dim)
    k = _cols(layer["k"], rank * hk * head_dim, (rank + 1) * hk * head_dim)
    v = _cols(layer["v"], rank * hk * head_dim, (rank + 1) * hk * head_dim)
    gate = _cols(layer["gate"], rank * f, (rank + 1) * f)
    up = _cols(layer["up"], rank * f, (rank + 1) * f)
    return {
        "qkv": (np.concatenate([q[0], k[0], v[0]], axis=1), np.concatenate([q[1], k[1], v[1]])),
        "o": _rows(layer["o"], rank * hq * head_dim, (rank + 1) * hq * head_dim),
        "gate_up": (interleave_gate_up(gate, up) if fuse_swiglu
                    else (np.concatenate([gate[0], up[0]], axis=1), np.concatenate([gate[1], up[1]]))),
        "down": _rows(layer["down"], rank * f, (rank + 1) * f),
        "ln1": layer["ln1"], "ln2": layer["ln2"],
    }


def interleave_gate_up(gate, up):
    """gate and up as (codes [K, F], scales [F]) -> the fused-SwiGLU layout of tlaloc_b200_int8_gemm_swiglu: one
    (codes [K, 2F], scales [2F]) whose column blocks of 256 hold 128 gate columns then the same 128 up columns.
    F must be a multiple of 128."""
    (gc, gs), (uc, us) = gate, up
    k, f = gc.shape
    if uc.shape != gc.shape or f % 128:
        raise ValueError(f"interleave_gate_up: gate and up must both be [K, F] with F a multiple of 128, got {gc.shape}, {uc.shape}")
    codes = np.stack([gc.reshape(k, f // 128, 128), uc.reshape(k, f // 128, 128)], axis=2).reshape(k, 2 * f)
    scales = np.stack([np.asarray(gs).reshape(f // 128, 128), np.asarray(us).reshape(f // 128, 128)], axis=1).reshape(2 * f)
    return np.ascontiguousarray(codes), np.ascontiguousarray(scales)


def shard_head(head, vocab: int, rank: int, world: int):
    """The rank's block of vocabulary columns: (codes, scales) for a quantized head, else the [d, V/g] matrix."""
    lo, hi = rank * (vocab // world), (rank + 1) * (vocab // world)
    if isinstance(head, tuple):
        return _cols(head, lo, hi)
    return np.ascontiguousarray(head[:, lo:hi])


def merge_greedy(values: np.ndarray, ids: np.ndarray, vocab_per_rank: int) -> np.ndarray:
    """Greedy token from per-rank candidates: values [g, B] (each rank's best logit), ids [g, B] (its local index).
    The largest value wins and, among equals, the lowest global id: the first-maximum rule of
    DxirInterpreter.kt:2414-2426 carried across the vocabulary blocks."""
    g, b = values.shape
    glob = ids.astype(np.int64) + (np.arange(g, dtype=np.int64) * vocab_per_rank)[:, None]
    best = np.zeros(b, np.int64)
    for r in range(1, g):
        better = values[r] > values[best, np.arange(b)]
        best = np.where(better, r, best)
    return glob[best, np.arange(b)].astype(np.int32)


def slot_mapping(block_tables: np.ndarray, positions: np.ndarray, block_size: int) -> np.ndarray:
    """The flat KV slot of each sequence's token at `positions`: pages[pos / bs] * bs + pos % bs
    (triton/backend/sequence_mode.cc:2584-2604)."""
    pos = np.asarray(positions, np.int64)
    pages = block_tables[np.arange(len(pos)), pos // block_size].astype(np.int64)
    return (pages * block_size + pos % block_size).astype(np.int32)
