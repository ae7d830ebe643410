"""CPU oracle: TEST INFRASTRUCTURE, not product code.

ctypes bindings over ``oracle/oracle.c`` (a C restatement of the reference's
host interpreter for the decode hot path) plus a NumPy composition of one
Llama-style decode step out of those primitives.  Only ``tests/``, the smoke
check and the benchmark's CPU-baseline leg may import this package; the CUDA
product path never does.

Reference lines each primitive follows are cited in ``oracle.c``; the step
composition follows ``ir/.../inference/HfDecoderGraph.kt`` (attention()
``:1162-1274``, mlp ``:953-1009``, layer loop ``:1553-1588``, tail
``:2093-2137``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` with the Makefile beside it (gcc, -ffp-contract=off)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_num_threads.restype = ctypes.c_int
        for name in ("orc_paged_attention", "orc_paged_attention_bf16", "orc_kv_cache_write", "orc_embedding"):
            getattr(_lib, name).restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def host_threads() -> int:
    return int(lib().orc_num_threads())


def snap_bf16(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_snap_bf16(_p(x), _p(out), ctypes.c_int64(x.size))
    return out


def bf16_bits(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16_bits(_p(x), _p(out), ctypes.c_int64(x.size))
    return out


def bf16_widen(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().orc_bf16_bits_to_f32(_p(bits), _p(out), ctypes.c_int64(bits.size))
    return out


def e4m3_bits(x) -> np.ndarray:
    """f32 -> e4m3fn bytes as an f8e4m3fn KV pool stores them: clamped to +-448, rounded to nearest even."""
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().orc_f32_to_e4m3_bits(_p(x), _p(out), ctypes.c_int64(x.size))
    return out


def e4m3_widen(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint8)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().orc_e4m3_bits_to_f32(_p(bits), _p(out), ctypes.c_int64(bits.size))
    return out


def snap_e4m3(x) -> np.ndarray:
    """saturateToF8e4m3fn elementwise: the f32 values an e4m3fn pool holds after a write of x."""
    return e4m3_widen(e4m3_bits(x))


class OracleRefusal(ValueError):
    """The interpreter would have refused these operands by name."""


def paged_attention(q, key_cache, value_cache, block_tables, seq_lens, scale, *, sliding_window=None, keep=None,
                    return_lse=False, threads=1):
    """``DxirInterpreter.evalPagedAttention`` on widened f32 arrays.

    q [R,H,D]; pools [P,bs,Hkv,D]; block_tables [Tb,M]; seq_lens [R]; keep [R,C] or None.
    ``scale`` is taken as a double (the interpreter multiplies the f64 dot by the attr's double value).
    """
    q, kc, vc = _f32(q), _f32(key_cache), _f32(value_cache)
    tables, lens = _i32(block_tables), _i32(seq_lens)
    R, H, D = q.shape
    P, bs, Hkv, Dk = kc.shape
    Tb, M = tables.shape
    if Dk != D or vc.shape != kc.shape or lens.shape != (R,) or R % Tb or H % Hkv:
        raise OracleRefusal("shape story refused (PagedAttentionAttrs.parse)")
    keep_arr, chunks = None, 0
    if keep is not None:
        keep_arr = _i32(keep)
        chunks = keep_arr.shape[1]
        if keep_arr.shape[0] != R or (M * bs) % chunks:
            raise OracleRefusal("keep must be [R, C] with C dividing the context")
    if sliding_window is not None and sliding_window < 1:
        raise OracleRefusal("sliding_window must be a whole number >= 1")
    out = np.empty_like(q)
    lse = np.empty((R, H), dtype=np.float32) if return_lse else None
    rc = lib().orc_paged_attention(_p(q), _p(kc), _p(vc), _p(tables), _p(lens), _p(keep_arr), chunks, _p(out), _p(lse),
                                   R, H, D, P, bs, Hkv, M, Tb, ctypes.c_double(float(scale)),
                                   int(sliding_window or 0), int(threads))
    if rc == -1:
        raise OracleRefusal("seqLens outside [0, maxBlocksPerSeq * blockSize]")
    if rc == -2:
        raise OracleRefusal("blockTables names a page outside [0, numBlocks)")
    return (out, lse) if return_lse else out


def paged_attention_bf16(q_bits, kc_bits, vc_bits, block_tables, seq_lens, scale, threads=1):
    """The same walk reading bf16 bit patterns (uint16) directly; used by the timed CPU leg."""
    tables, lens = _i32(block_tables), _i32(seq_lens)
    R, H, D = q_bits.shape
    P, bs, Hkv, _ = kc_bits.shape
    Tb, M = tables.shape
    out = np.empty((R, H, D), dtype=np.float32)
    rc = lib().orc_paged_attention_bf16(_p(q_bits), _p(kc_bits), _p(vc_bits), _p(tables), _p(lens), _p(out), R, H, D,
                                        P, bs, Hkv, M, Tb, ctypes.c_double(float(scale)), int(threads))
    if rc:
        raise OracleRefusal(f"paged walk refused ({rc})")
    return out


def matmul_f32(a, b, threads=1) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_matmul_f32(_p(a), _p(b), _p(out), m, k, n, int(threads))
    return out


def proj_int8(x, codes, scales, round_x_bf16=True, threads=1) -> np.ndarray:
    """``HfDecoderGraph.proj`` over an int8 weight: (cast(x) @ cast(codes)) * scale."""
    x = _f32(x)
    codes = np.ascontiguousarray(codes, dtype=np.int8)
    scales = _f32(scales)
    m, k = x.shape
    k2, n = codes.shape
    assert k == k2 and scales.shape == (n,)
    y = np.empty((m, n), dtype=np.float32)
    lib().orc_proj_int8(_p(x), _p(codes), _p(scales), _p(y), m, k, n, int(bool(round_x_bf16)), int(threads))
    return y


def quantize_int8(w_out_in) -> tuple[np.ndarray, np.ndarray]:
    """``HfStagedWeights.quantize`` INT8: w [out,in] f32 -> codes [in,out] int8, scales [out] f32."""
    w = _f32(w_out_in)
    o, i = w.shape
    codes = np.empty((i, o), dtype=np.int8)
    scales = np.empty((o,), dtype=np.float32)
    lib().orc_quantize_int8(_p(w), o, i, _p(codes), _p(scales))
    return codes, scales


def kv_cache_write(pool, new_kv, slots) -> np.ndarray:
    """Functional ``KV_CACHE_WRITE``: returns the updated pool [P,bs,Hkv,D]."""
    out = _f32(pool).copy()
    new_kv, slots = _f32(new_kv), _i32(slots)
    P, bs, Hkv, D = out.shape
    rc = lib().orc_kv_cache_write(_p(out), _p(new_kv), _p(slots), slots.shape[0], Hkv * D, P * bs)
    if rc == -1:
        raise OracleRefusal("a slot past the pool is an allocator bug, not padding")
    if rc == -2:
        raise OracleRefusal("the non-negative slots must be distinct")
    return out


def kv_cache_write_inplace(pool: np.ndarray, new_kv, slots) -> None:
    """KV_CACHE_WRITE on a caller-owned f32 pool (no copy); same refusals."""
    assert pool.dtype == np.float32 and pool.flags.c_contiguous
    new_kv, slots = _f32(new_kv), _i32(slots)
    P, bs, Hkv, D = pool.shape
    rc = lib().orc_kv_cache_write(_p(pool), _p(new_kv), _p(slots), slots.shape[0], Hkv * D, P * bs)
    if rc:
        raise OracleRefusal("KV_CACHE_WRITE refused the slots")


def rmsnorm(x, gain, eps) -> np.ndarray:
    x = _f32(x)
    g = None if gain is None else _f32(gain)
    out = np.empty_like(x)
    rows = int(np.prod(x.shape[:-1]))
    lib().orc_rmsnorm(_p(x), _p(g), _p(out), rows, x.shape[-1], ctypes.c_float(np.float32(eps)))
    return out


def rope_tables(theta, head_dim, positions):
    cos = np.empty((positions, head_dim), dtype=np.float32)
    sin = np.empty_like(cos)
    lib().orc_rope_tables(ctypes.c_double(theta), head_dim, positions, _p(cos), _p(sin))
    return cos, sin


def rope(x, pos, cos, sin) -> np.ndarray:
    x, pos = _f32(x), _i32(pos)
    rows, heads, hd = x.shape
    out = np.empty_like(x)
    lib().orc_rope(_p(x), _p(pos), _p(_f32(cos)), _p(_f32(sin)), _p(out), rows, heads, hd)
    return out


def swiglu(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().orc_swiglu(_p(gate), _p(up), _p(out), ctypes.c_int64(gate.size))
    return out


def argmax(x) -> np.ndarray:
    x = _f32(x)
    rows = int(np.prod(x.shape[:-1]))
    out = np.empty((rows,), dtype=np.int32)
    lib().orc_argmax(_p(x), _p(out), rows, x.shape[-1])
    return out.reshape(x.shape[:-1])


def embedding(table, ids) -> np.ndarray:
    table, ids = _f32(table), _i32(ids).reshape(-1)
    out = np.empty((ids.shape[0], table.shape[1]), dtype=np.float32)
    if lib().orc_embedding(_p(table), _p(ids), _p(out), ids.shape[0], table.shape[0], table.shape[1]):
        raise OracleRefusal("EMBEDDING index out of bounds")
    return out


# --------------------------------------------------------------------------------------------
# A Llama-style decode step composed from the primitives above.


@dataclass
class DecoderShape:
    """The fields of the reference's HfDecoderConfig this path reads."""

    num_layers: int
    d_model: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    block_size: int = 16
    # HfDecoderConfig.weightDType: BF16 rounds activations to bf16 before each projection and keeps the
    # embedding table / head / norm gains as bf16 values; F32 leaves everything f32.
    weight_dtype: str = "bf16"
    kv_dtype: str = "f32"  # "f32" | "bf16" | "e4m3": values are snapped on write (bf16 RNE; e4m3fn clamped to 448, RNE)
    head_quant: bool = False  # WeightQuant.kt:21-22: the head stays in weight dtype unless quantized
    # The Granite family's four scalars (HfDecoderGraph.kt:546,915,1000,2129): h *= embed_scale after the embedding;
    # the attention scale replaces 1/sqrt(head_dim); each sub-layer's output is multiplied by residual_multiplier
    # before its residual add; the logits by logit_multiplier.  Every one a MUL by the f32 constant.
    embed_scale: float | None = None
    attention_scale: float | None = None
    residual_multiplier: float = 1.0
    logit_multiplier: float = 1.0


@dataclass
class DecoderWeights:
    """Weights in the staged layout: int8 codes [in,out] + f32 scales [out] per projection."""

    embed: np.ndarray  # [vocab, d] f32 values (bf16-representable when weight_dtype is bf16)
    layers: list = field(default_factory=list)  # dicts: q,k,v,o,gate,up,down -> (codes, scales); ln1, ln2 gains
    final_norm: np.ndarray | None = None
    head: tuple | np.ndarray | None = None  # (codes, scales) when head_quant else [d, vocab] f32 values


def make_weights(shape: DecoderShape, seed: int = 0, std: float = 0.02) -> DecoderWeights:
    """Random-init N(0, std) weights, quantized per output channel as the exporter does; norm gains are ones."""
    rng = np.random.default_rng(seed)
    d, qo, kvo = shape.d_model, shape.num_heads * shape.head_dim, shape.num_kv_heads * shape.head_dim

    def lin(out_f, in_f):
        return quantize_int8((rng.standard_normal((out_f, in_f)) * std).astype(np.float32))

    def plain(a):
        a = a.astype(np.float32)
        return snap_bf16(a) if shape.weight_dtype == "bf16" else a

    w = DecoderWeights(embed=plain(rng.standard_normal((shape.vocab, d)) * std))
    for _ in range(shape.num_layers):
        w.layers.append({
            "q": lin(qo, d), "k": lin(kvo, d), "v": lin(kvo, d), "o": lin(d, qo),
            "gate": lin(shape.ffn, d), "up": lin(shape.ffn, d), "down": lin(d, shape.ffn),
            "ln1": np.ones(d, np.float32), "ln2": np.ones(d, np.float32),
        })
    w.final_norm = np.ones(d, np.float32)
    head = (rng.standard_normal((shape.vocab, d)) * std).astype(np.float32)
    w.head = quantize_int8(head) if shape.head_quant else plain(head.T.copy())
    return w


def decode_step(shape: DecoderShape, w: DecoderWeights, key_pools, value_pools, token_ids, positions, block_tables,
                seq_lens, slot_mapping, threads=1):
    """One decode step (one token per sequence); pools are updated in place. Returns logits [B, vocab] f32.

    HfDecoderGraph.kt: embed :904-909 -> per layer [rmsNorm -> q/k/v proj -> rope -> KV_CACHE_WRITE x2 ->
    PAGED_ATTENTION -> o proj -> +h -> rmsNorm -> SiLU(gate)*up -> down -> +h] -> final norm -> head.
    """
    bf = shape.weight_dtype == "bf16"
    B = len(token_ids)
    H, Hkv, hd = shape.num_heads, shape.num_kv_heads, shape.head_dim
    # HfDecoderGraph.kt:546: config.attentionScale?.toFloat() ?: 1f / sqrt(hd.toFloat()), widened
    scale = float(np.float32(shape.attention_scale)) if shape.attention_scale is not None \
        else float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    cos, sin = rope_tables(shape.rope_theta, hd, int(np.max(positions)) + 1)

    def proj(x, wt):
        """HfDecoderGraph.proj (:625-655): an int8 weight is (codes, scales); an unquantized one [in, out] values."""
        if isinstance(wt, tuple):
            return proj_int8(x, *wt, round_x_bf16=bf, threads=threads)
        return matmul_f32(snap_bf16(x) if bf else x, wt, threads=threads)

    def times(x, c):  # :702-703: MUL by the constant narrowed to f32
        return x if c == 1.0 else (x * np.float32(c)).astype(np.float32)

    h = embedding(w.embed, token_ids)
    if shape.embed_scale is not None:
        h = times(h, shape.embed_scale)
    for l, lw in enumerate(w.layers):
        hn = rmsnorm(h, lw["ln1"], shape.rms_eps)
        q = proj(hn, lw["q"]).reshape(B, H, hd)
        k = proj(hn, lw["k"]).reshape(B, Hkv, hd)
        v = proj(hn, lw["v"]).reshape(B, Hkv, hd)
        q, k = rope(q, positions, cos, sin), rope(k, positions, cos, sin)
        if shape.kv_dtype == "bf16":
            k, v = snap_bf16(k), snap_bf16(v)
        elif shape.kv_dtype == "e4m3":  # DxirInterpreter.kt:2241-2246: an f8e4m3fn cache stores each value clamped and rounded
            k, v = snap_e4m3(k), snap_e4m3(v)
        kv_cache_write_inplace(key_pools[l], k.reshape(B, -1), slot_mapping)
        kv_cache_write_inplace(value_pools[l], v.reshape(B, -1), slot_mapping)
        att = paged_attention(q, key_pools[l], value_pools[l], block_tables, seq_lens, scale, threads=threads)
        h = h + times(proj(att.reshape(B, H * hd), lw["o"]), shape.residual_multiplier)
        hn2 = rmsnorm(h, lw["ln2"], shape.rms_eps)
        g = proj(hn2, lw["gate"])
        u = proj(hn2, lw["up"])
        h = h + times(proj(swiglu(g, u), lw["down"]), shape.residual_multiplier)
    hf = rmsnorm(h, w.final_norm, shape.rms_eps)
    return times(proj(hf, w.head), shape.logit_multiplier)
