"""The hot-path operators on torch CUDA tensors, through the C ABI.

PyTorch is plumbing here (device memory, the current stream); every operator is one call into
libtlaloc_kernels.so with raw device pointers, enqueued on torch's current stream.  There is no CPU path:
a tensor that is not on a CUDA device is refused.
"""
from __future__ import annotations

import torch

from . import _native as N
from .attrs import PagedAttentionShape, parse_paged_attention

_DT = {torch.float32: N.F32, torch.bfloat16: N.BF16, torch.int8: N.S8, torch.int32: N.S32, torch.float8_e4m3fn: N.F8E4M3FN}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def _dev(*ts) -> None:
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("operands must be contiguous CUDA tensors (there is no CPU path)")


def _out(name: str, t, shape, dtypes, like: torch.Tensor) -> None:
    """A caller-supplied result or scratch tensor is written through its raw pointer: refuse one that is not exactly
    the contiguous CUDA tensor of that shape the kernel will write."""
    if t is None:
        return
    if not isinstance(dtypes, (tuple, list)):
        dtypes = (dtypes,)
    if (not t.is_cuda or not t.is_contiguous() or t.device != like.device or t.dtype not in dtypes
            or (shape is not None and tuple(t.shape) != tuple(shape))):
        want = "x".join(str(d) for d in shape) if shape is not None else "any shape"
        raise ValueError(f"{name} must be a contiguous {'/'.join(str(d) for d in dtypes)} tensor [{want}] on {like.device}, "
                         f"got {t.dtype} {tuple(t.shape)} on {t.device}")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor) -> int:
    """The current stream of the tensor's own device (not of whichever device happens to be current)."""
    return torch.cuda.current_stream(t.device).cuda_stream


def init() -> None:
    """Kernel set-up for the current CUDA device (call once per device, before any graph capture)."""
    N.check(N.lib().tlaloc_b200_init())


def set_order_faithful(on: bool) -> bool:
    """Parity mode of the whole library (tlaloc_b200_set_order_faithful); returns the previous setting."""
    return bool(N.lib().tlaloc_b200_set_order_faithful(1 if on else 0))


def paged_attention_scratch(shape: PagedAttentionShape, device, splits: int | None = None) -> torch.Tensor:
    """The f32 scratch [S, R, H, D + 2] a call of this shape wants (S as the reference's emitter sizes it)."""
    lib = N.lib()
    if splits is None:
        splits = lib.tlaloc_b200_paged_attention_splits(shape.num_seqs, shape.num_kv_heads, shape.num_tables,
                                                        shape.max_blocks_per_seq, shape.block_size)
    return torch.empty((splits, shape.num_seqs, shape.num_heads, shape.head_dim + 2), dtype=torch.float32, device=device)


def paged_attention(query, key_cache, value_cache, block_tables, seq_lens, *, scale, sliding_window=None, keep=None,
                    return_lse=False, out=None, scratch=None):
    """PAGED_ATTENTION: operands and attrs as ir/.../PagedAttentionAttrs.kt; see include/tlaloc_b200.h."""
    p = parse_paged_attention(query, key_cache, value_cache, block_tables, seq_lens, scale=scale,
                              sliding_window=sliding_window, keep=keep, layer="tlaloc_b200.ops")
    _dev(query, key_cache, value_cache, block_tables, seq_lens, keep)
    if block_tables.dtype != torch.int32 or seq_lens.dtype != torch.int32 or (keep is not None and keep.dtype != torch.int32):
        raise TypeError("PAGED_ATTENTION: the kernels read blockTables, seqLens and keep as int32")
    if out is None:
        out = torch.empty_like(query)
    if scratch is None:
        scratch = paged_attention_scratch(p, query.device)
    _out("PAGED_ATTENTION out", out, (p.num_seqs, p.num_heads, p.head_dim), (torch.float32, torch.bfloat16), query)
    if scratch.dim() != 4 or scratch.shape[0] < 1:
        raise ValueError("PAGED_ATTENTION scratch must be f32 [S, R, H, D + 2] with S >= 1")
    _out("PAGED_ATTENTION scratch", scratch, (scratch.shape[0], p.num_seqs, p.num_heads, p.head_dim + 2), torch.float32, query)
    lse = torch.empty((p.num_seqs, p.num_heads), dtype=torch.float32, device=query.device) if return_lse else None
    N.check(N.lib().tlaloc_b200_paged_attention(
        _ptr(query), _dt(query), _ptr(key_cache), _ptr(value_cache), _dt(key_cache), _ptr(block_tables),
        _ptr(seq_lens), _ptr(keep), 0 if keep is None else keep.shape[1], _ptr(out), _dt(out), _ptr(lse),
        _ptr(scratch), scratch.shape[0], p.num_seqs, p.num_heads, p.head_dim, p.num_blocks, p.block_size,
        p.num_kv_heads, p.max_blocks_per_seq, p.num_tables, float(scale), int(sliding_window or 0), _stream(query)))
    return (out, lse) if return_lse else out


def kv_cache_write(pool, new_kv, slot_mapping):
    """KV_CACHE_WRITE in place: pool [P, bs, Hkv, D], new_kv [T, Hkv, D], slot_mapping i32 [T]."""
    _dev(pool, new_kv, slot_mapping)
    P, bs, Hkv, D = pool.shape
    T = slot_mapping.shape[0]
    if new_kv.numel() != T * Hkv * D:
        raise ValueError(f"KV_CACHE_WRITE: newKv must be [T, {Hkv}, {D}] for the pool, got {tuple(new_kv.shape)}")
    N.check(N.lib().tlaloc_b200_kv_cache_write(_ptr(pool), _dt(pool), _ptr(new_kv), _dt(new_kv), _ptr(slot_mapping), T,
                                               Hkv * D, P * bs, _stream(pool)))
    return pool


def int8_gemm(x, codes, scales, *, residual=None, out=None, out_dtype=torch.float32, exact=False, x_f32_exact=False,
              scratch=None, weights_const=False, i8_mma=False, x_planes=False):
    """y = (cast(x) @ cast(codes)) * scales (+ residual): x [M, K], codes int8 [K, N] (in, out), scales f32 [N].
    `weights_const`: no kernel queued just before this call writes codes or scales (true of a loaded model).
    `i8_mma`: 17 to 128 rows take the int8 tensor-core kernel (codes straight to the tensor core, activations as 16-bit
    fixed point per row, exact int32 sums) instead of the bf16 one (f32 accumulation of exact products).
    `x_planes`: `scratch` already holds x's activation planes (rmsnorm(..., planes=scratch) wrote them)."""
    _dev(x, codes, scales, residual)
    M, K = x.shape
    K2, Nn = codes.shape
    if K2 != K or codes.dtype != torch.int8 or (scales is not None and tuple(scales.shape) != (Nn,)):
        raise ValueError(f"INT8_PROJ: x [M, K] x codes int8 [K, N] with scales [N]; got {tuple(x.shape)}, {tuple(codes.shape)}")
    if out is None:
        out = torch.empty((M, Nn), dtype=out_dtype, device=x.device)
    _out("INT8_PROJ out", out, (M, Nn), (torch.float32, torch.bfloat16), x)
    _out("INT8_PROJ residual", residual, (M, Nn), torch.float32, x)
    # an f32 x is cast to bf16 in the scratch; the int8 tensor-core kernel leaves the activations' int8 planes there
    if scratch is None and not exact and (x.dtype == torch.float32 or (i8_mma and 17 <= M <= 128)):
        scratch = torch.empty((N.lib().tlaloc_b200_int8_gemm_scratch_bytes(M, K, Nn) + 3) // 4, dtype=torch.float32,
                              device=x.device)
    _out("INT8_PROJ scratch", scratch, None, torch.float32, x)
    flags = ((N.GEMM_EXACT if exact else 0) | (N.GEMM_X_F32_EXACT if x_f32_exact else 0)
             | (N.GEMM_WEIGHTS_CONST if weights_const else 0) | (N.GEMM_I8_MMA if i8_mma else 0)
             | (N.GEMM_X_PLANES if x_planes else 0))
    N.check(N.lib().tlaloc_b200_int8_gemm(_ptr(x), _dt(x), _ptr(codes), _ptr(scales), _ptr(residual), _ptr(out), _dt(out),
                                          _ptr(scratch), 0 if scratch is None else scratch.numel() * 4, M, K, Nn, flags,
                                          _stream(x)))
    return out


def int8_gemm_swiglu(x, codes, scales, *, out=None, out_dtype=torch.bfloat16, exact=False, scratch=None, weights_const=False,
                     i8_mma=False, x_planes=False):
    """silu(x @ gate) * (x @ up) with gate and up interleaved in `codes` [K, 2F] in column blocks of 128 + 128
    (sharding.interleave_gate_up); returns [M, F]."""
    _dev(x, codes, scales)
    M, K = x.shape
    K2, Nn = codes.shape
    if K2 != K or codes.dtype != torch.int8 or Nn % 256 or (scales is not None and tuple(scales.shape) != (Nn,)):
        raise ValueError(f"INT8_PROJ_SWIGLU: x [M, K] x codes int8 [K, 2F] (2F a multiple of 256) with scales [2F]; got "
                         f"{tuple(x.shape)}, {tuple(codes.shape)}")
    if out is None:
        out = torch.empty((M, Nn // 2), dtype=out_dtype, device=x.device)
    _out("INT8_PROJ_SWIGLU out", out, (M, Nn // 2), (torch.float32, torch.bfloat16), x)
    if scratch is None and not exact and (x.dtype == torch.float32 or (i8_mma and 17 <= M <= 128)):
        scratch = torch.empty((N.lib().tlaloc_b200_int8_gemm_scratch_bytes(M, K, Nn) + 3) // 4, dtype=torch.float32, device=x.device)
    _out("INT8_PROJ_SWIGLU scratch", scratch, None, torch.float32, x)
    flags = ((N.GEMM_EXACT if exact else 0) | (N.GEMM_WEIGHTS_CONST if weights_const else 0) | (N.GEMM_I8_MMA if i8_mma else 0)
             | (N.GEMM_X_PLANES if x_planes else 0))
    N.check(N.lib().tlaloc_b200_int8_gemm_swiglu(_ptr(x), _dt(x), _ptr(codes), _ptr(scales), _ptr(out), _dt(out), _ptr(scratch),
                                                 0 if scratch is None else scratch.numel() * 4, M, K, Nn, flags, _stream(x)))
    return out


def int8_gemm_scratch_bytes(m: int, k: int, n: int) -> int:
    return int(N.lib().tlaloc_b200_int8_gemm_scratch_bytes(m, k, n))


def dense_gemm_exact(x, w, *, x_f32_exact=False):
    """The interpreter's MATMUL order over an unquantized weight w [K, N]; returns f32 [M, N]."""
    _dev(x, w)
    M, K = x.shape
    out = torch.empty((M, w.shape[1]), dtype=torch.float32, device=x.device)
    N.check(N.lib().tlaloc_b200_dense_gemm_exact(_ptr(x), _dt(x), _ptr(w), _dt(w), _ptr(out), M, K, w.shape[1],
                                                 N.GEMM_X_F32_EXACT if x_f32_exact else 0, _stream(x)))
    return out


def embedding(table, ids, *, out=None):
    _dev(table, ids)
    ids = ids.reshape(-1)
    if out is None:
        out = torch.empty((ids.shape[0], table.shape[1]), dtype=torch.float32, device=table.device)
    _out("EMBEDDING out", out, (ids.shape[0], table.shape[1]), torch.float32, table)
    N.check(N.lib().tlaloc_b200_embedding(_ptr(table), _dt(table), _ptr(ids), _ptr(out), ids.shape[0], table.shape[0],
                                          table.shape[1], _stream(table)))
    return out


def rmsnorm(x, gain, eps, *, out=None, out_dtype=torch.float32, planes=None):
    """x * rsqrt(mean(x^2) + eps) * gain.  `planes` (an f32 scratch of int8_gemm_scratch_bytes(rows, n, 0) bytes; out must
    be bf16, n a multiple of 16) also receives the normalised rows as the activation planes of the int8 tensor-core
    projection that reads `out`: call that projection with the same scratch and x_planes=True."""
    _dev(x, gain)
    rows, n = x.shape
    if out is None:
        out = torch.empty((rows, n), dtype=torch.bfloat16 if planes is not None else out_dtype, device=x.device)
    _out("RMSNORM out", out, (rows, n), (torch.float32, torch.bfloat16), x)
    if planes is not None:
        _out("RMSNORM planes", planes, None, torch.float32, x)
        if out.dtype != torch.bfloat16 or planes.numel() * 4 < int8_gemm_scratch_bytes(rows, n, 0):
            raise ValueError("RMSNORM: planes need a bf16 out and int8_gemm_scratch_bytes(rows, n, 0) bytes")
        N.check(N.lib().tlaloc_b200_rmsnorm_planes(_ptr(x), _ptr(gain), _ptr(out), _ptr(planes), planes.numel() * 4, rows, n, float(eps), _stream(x)))
        return out
    N.check(N.lib().tlaloc_b200_rmsnorm(_ptr(x), _ptr(gain), _ptr(out), _dt(out), rows, n, float(eps), _stream(x)))
    return out


def rope_kv_write(q, k, v, positions, cos_table, sin_table, slot_mapping, key_cache, value_cache, *, q_out=None,
                  q_dtype=torch.float32):
    """RoPE on q [T,H,hd] and k [T,Hkv,hd], then K/V rows into the pools at slot_mapping; returns rotated q."""
    _dev(positions, cos_table, sin_table, slot_mapping, key_cache, value_cache)
    for t in (q, k, v):
        if not t.is_cuda or t.dtype != torch.float32 or t.stride(2) != 1 or t.stride(1) != t.shape[2]:
            raise ValueError("ROPE_KV_WRITE: q, k and v must be f32 CUDA tensors [T, heads, hd] with dense heads")
    T, H, hd = q.shape
    Hkv = k.shape[1]
    P, bs = key_cache.shape[0], key_cache.shape[1]
    if q_out is None:
        q_out = torch.empty((T, H, hd), dtype=q_dtype, device=q.device)
    _out("ROPE_KV_WRITE q_out", q_out, (T, H, hd), (torch.float32, torch.bfloat16), q)
    N.check(N.lib().tlaloc_b200_rope_kv_write(_ptr(q), _ptr(k), _ptr(v), _ptr(positions), _ptr(cos_table), _ptr(sin_table),
                                              _ptr(slot_mapping), _ptr(q_out), _dt(q_out), _ptr(key_cache),
                                              _ptr(value_cache), _dt(key_cache), T, H, Hkv, hd, P * bs,
                                              cos_table.shape[0], q.stride(0), k.stride(0), v.stride(0), _stream(q)))
    return q_out


def swiglu(gate, up, *, out=None, out_dtype=torch.float32):
    """silu(gate) * up; gate and up may be column slices of one [rows, ld] matrix (a fused gate|up projection)."""
    if not gate.is_cuda or gate.stride(1) != 1 or up.stride(1) != 1 or gate.stride(0) != up.stride(0):
        raise ValueError("SWIGLU: gate and up must be CUDA row-major views with the same row stride")
    rows, n = gate.shape
    if out is None:
        out = torch.empty((rows, n), dtype=out_dtype, device=gate.device)
    _out("SWIGLU out", out, (rows, n), (torch.float32, torch.bfloat16), gate)
    N.check(N.lib().tlaloc_b200_swiglu(_ptr(gate), _ptr(up), gate.stride(0), _ptr(out), _dt(out), rows, n, _stream(gate)))
    return out


def argmax(logits, out=None):
    _dev(logits)
    rows, n = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _out("ARGMAX out", out, (rows,), torch.int32, logits)
    N.check(N.lib().tlaloc_b200_argmax(_ptr(logits), _ptr(out), rows, n, _stream(logits)))
    return out
