"""Pins the CPU oracle against the reference's own known answers (no GPU).

1. triton/examples/reference/reference_decode.json: five decode steps of
   maestro/.../ReferenceDecodeGraph.kt evaluated by the reference interpreter; the oracle
   must reproduce every logit bit for bit.
2. ir/src/commonTest/.../passes/PagedAttentionTest.kt: the hand-exact cases (2.0 / 1.5,
   4.5 / 2.5, +-10), the dense-twin sweeps and the refusals.
3. The quantizer formula of ir/src/jvmTest/.../HfMuseGlimmerTest.kt:452-494 and the identity
   "int8 graph == graph of dequantized weights" (:502-527).
"""
import json
import os

import numpy as np
import pytest

import oracle
from refdata import dense_twin, lcg_weights, pseudo

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


# --------------------------------------------------------------------------- reference_decode.json


def reference_decode_model():
    V, d, H, Hkv, hd = 11, 8, 4, 2, 2
    return dict(
        V=V, d=d, H=H, Hkv=Hkv, hd=hd, P=6, bs=2,
        embed=lcg_weights(1, V * d).reshape(V, d),
        q=lcg_weights(2, d * H * hd).reshape(d, H * hd),
        k=lcg_weights(3, d * Hkv * hd).reshape(d, Hkv * hd),
        v=lcg_weights(4, d * Hkv * hd).reshape(d, Hkv * hd),
        head=lcg_weights(5, H * hd * V).reshape(H * hd, V),
        scale=float(np.float32(1.0) / np.sqrt(np.float32(hd))),
    )


def reference_decode_step(m, kc, vc, step):
    """ReferenceDecodeGraph.kt:101-149: embed -> q/k/v MATMUL -> KV_CACHE_WRITE x2 -> PAGED_ATTENTION -> head."""
    i = step["inputs"]
    ids = np.array(i["tokenIds"]["data"], np.int32)
    tables = np.array(i["blockTables"]["data"], np.int32).reshape(i["blockTables"]["shape"])
    lens = np.array(i["seqLens"]["data"], np.int32)
    slots = np.array(i["slotMapping"]["data"], np.int32)
    B = ids.shape[0]
    h = oracle.embedding(m["embed"], ids)
    q = oracle.matmul_f32(h, m["q"]).reshape(B, m["H"], m["hd"])
    k = oracle.matmul_f32(h, m["k"])
    v = oracle.matmul_f32(h, m["v"])
    kc[...] = oracle.kv_cache_write(kc, k, slots)
    vc[...] = oracle.kv_cache_write(vc, v, slots)
    att = oracle.paged_attention(q, kc, vc, tables, lens, m["scale"])
    return oracle.matmul_f32(att.reshape(B, -1), m["head"])


def test_reference_decode_json_is_reproduced_bit_for_bit():
    with open(os.path.join(GOLDEN, "reference_decode.json")) as f:
        golden = json.load(f)
    m = reference_decode_model()
    kc = np.zeros((m["P"], m["bs"], m["Hkv"], m["hd"]), np.float32)
    vc = np.zeros_like(kc)
    assert len(golden["steps"]) == 5
    for n, step in enumerate(golden["steps"]):
        got = reference_decode_step(m, kc, vc, step).reshape(-1)
        want = np.array(step["outputs"]["logits"]["data"], dtype=np.float32)
        assert got.shape == want.shape
        assert np.array_equal(got, want), f"step {n}: worst |d| {np.abs(got - want).max()}"


# --------------------------------------------------------------------------- PagedAttentionTest.kt

R, H, HKV, D, BS, P, M = 2, 4, 2, 3, 2, 6, 3
CTX = M * BS
SCALE = 0.5


def _inputs(sq, sk, sv):
    q = pseudo(R * H * D, sq).reshape(R, H, D)
    k = pseudo(P * BS * HKV * D, sk).reshape(P, BS, HKV, D)
    v = pseudo(P * BS * HKV * D, sv).reshape(P, BS, HKV, D)
    return q, k, v


def _close(a, b, tol=1e-5):
    assert np.abs(a - b).max() <= tol, np.abs(a - b).max()


def test_identity_table_matches_dense():
    q, k, v = _inputs(7, 11, 13)
    table = np.arange(6, dtype=np.int32).reshape(R, M)
    lens = np.array([CTX, CTX])
    _close(dense_twin(q, k, v, table, lens, SCALE), oracle.paged_attention(q, k, v, table, lens, SCALE))


def test_permuted_table_and_ragged_lengths_match_dense():
    q, k, v = _inputs(17, 19, 23)
    table = np.array([4, 1, 5, 2, 0, 3], np.int32).reshape(R, M)
    lens = np.array([6, 3])
    _close(dense_twin(q, k, v, table, lens, SCALE), oracle.paged_attention(q, k, v, table, lens, SCALE))


def test_seq_len_sweep_matches_dense():
    q, k, v = _inputs(29, 31, 37)
    table = np.array([5, 3, 1, 0, 4, 2], np.int32).reshape(R, M)
    for len0 in range(1, CTX + 1):
        lens = np.array([len0, CTX - len0 + 1])
        _close(dense_twin(q, k, v, table, lens, SCALE), oracle.paged_attention(q, k, v, table, lens, SCALE))


def test_sliding_window_matches_dense_over_the_last_positions():
    q, k, v = _inputs(41, 43, 47)
    table = np.array([5, 3, 1, 0, 4, 2], np.int32).reshape(R, M)
    for w in range(1, CTX + 1):
        for len0 in range(1, CTX + 1):
            lens = np.array([len0, CTX - len0 + 1])
            _close(dense_twin(q, k, v, table, lens, SCALE, window=w),
                   oracle.paged_attention(q, k, v, table, lens, SCALE, sliding_window=w))


def test_window_changes_the_answer_only_when_shorter_than_the_row():
    q, k, v = _inputs(53, 59, 61)
    table = np.array([4, 1, 5, 2, 0, 3], np.int32).reshape(R, M)
    lens = np.array([5, 6])
    full = oracle.paged_attention(q, k, v, table, lens, SCALE)
    win = oracle.paged_attention(q, k, v, table, lens, SCALE, sliding_window=2)
    assert np.abs(full - win).max() > 1e-2
    _close(full, oracle.paged_attention(q, k, v, table, lens, SCALE, sliding_window=CTX))


def _live_rows(table, lens, fill):
    v = np.full((P, BS, HKV, D), 1000.0, np.float32)
    for s in range(R):
        for t in range(lens[s]):
            v[table[s, t // BS], t % BS] = fill(s, t)
    return v


def test_hand_exact_uniform_softmax_over_partially_filled_pages():
    """PagedAttentionTest.kt:301-333: zero keys, V rows 1,2,3..., dead slots poisoned with 1000."""
    q = np.ones((R, H, D), np.float32)
    k = np.zeros((P, BS, HKV, D), np.float32)
    table = np.array([2, 0, 4, 5, 3, 1], np.int32).reshape(R, M)
    lens = np.array([3, 2])
    v = _live_rows(table, lens, lambda s, t: t + 1)
    got = oracle.paged_attention(q, k, v, table, lens, SCALE)
    assert np.abs(got[0] - 2.0).max() <= 1e-5 and np.abs(got[1] - 1.5).max() <= 1e-5


def test_hand_exact_window_averages_the_last_two_rows():
    """PagedAttentionTest.kt:258-281: window 2 over lens 5 and 3 gives 4.5 and 2.5."""
    q = np.ones((R, H, D), np.float32)
    k = np.zeros((P, BS, HKV, D), np.float32)
    table = np.array([2, 0, 4, 5, 3, 1], np.int32).reshape(R, M)
    lens = np.array([5, 3])
    v = _live_rows(table, lens, lambda s, t: 1000.0 if t < lens[s] - 2 else t + 1)
    got = oracle.paged_attention(q, k, v, table, lens, SCALE, sliding_window=2)
    assert np.abs(got[0] - 4.5).max() <= 1e-5 and np.abs(got[1] - 2.5).max() <= 1e-5


def test_gqa_grouping_is_contiguous_per_kv_head():
    """PagedAttentionTest.kt:335-357."""
    q = np.ones((R, H, D), np.float32)
    k = np.zeros((P, BS, HKV, D), np.float32)
    v = np.empty((P, BS, HKV, D), np.float32)
    v[:, :, 0] = 10.0
    v[:, :, 1] = -10.0
    table = np.arange(6, dtype=np.int32).reshape(R, M)
    got = oracle.paged_attention(q, k, v, table, np.array([4, 4]), SCALE)
    for h in range(H):
        assert np.abs(got[:, h] - (10.0 if h // (H // HKV) == 0 else -10.0)).max() <= 1e-5


def test_rows_sharing_a_table_equal_rows_with_the_table_repeated():
    """PagedAttentionTest.kt:368-405: three rows per table, bit for bit, with and without a window."""
    rows, per = 6, 3
    q = pseudo(rows * H * D, 211).reshape(rows, H, D)
    k = pseudo(P * BS * HKV * D, 223).reshape(P, BS, HKV, D)
    v = pseudo(P * BS * HKV * D, 227).reshape(P, BS, HKV, D)
    tables = np.array([4, 1, 5, 2, 0, 3], np.int32).reshape(2, M)
    lens = np.array([4, 5, 6, 2, 3, 4])
    repeated = np.repeat(tables, per, axis=0)
    for w in (None, 2):
        shared = oracle.paged_attention(q, k, v, tables, lens, SCALE, sliding_window=w)
        per_row = oracle.paged_attention(q, k, v, repeated, lens, SCALE, sliding_window=w)
        assert np.array_equal(shared, per_row)
        swapped = np.array([2, 0, 3, 4, 1, 5], np.int32).reshape(2, M)
        assert not np.array_equal(shared, oracle.paged_attention(q, k, v, swapped, lens, SCALE, sliding_window=w))


def test_refusals():
    q, k, v = _inputs(3, 5, 5)
    ident = np.arange(6, dtype=np.int32).reshape(R, M)
    with pytest.raises(oracle.OracleRefusal):
        oracle.paged_attention(q, k, v, ident, np.array([2, 2]), SCALE, sliding_window=0)
    with pytest.raises(oracle.OracleRefusal):
        oracle.paged_attention(q, k, v, ident, np.array([CTX + 1, 2]), SCALE)
    with pytest.raises(oracle.OracleRefusal):
        oracle.paged_attention(q, k, v, np.array([0, 1, 9, 3, 4, 5], np.int32).reshape(R, M), np.array([6, 6]), SCALE)
    with pytest.raises(oracle.OracleRefusal):  # tables that do not divide the rows
        oracle.paged_attention(np.ones((3, H, D), np.float32), k, v, ident, np.array([1, 1, 1]), SCALE)


def test_an_empty_row_is_zero_and_lse_is_minus_inf():
    q, k, v = _inputs(3, 5, 7)
    ident = np.arange(6, dtype=np.int32).reshape(R, M)
    out, lse = oracle.paged_attention(q, k, v, ident, np.array([0, 3]), SCALE, return_lse=True)
    assert np.all(out[0] == 0) and np.all(np.isneginf(lse[0])) and np.all(np.isfinite(lse[1]))


def test_threads_do_not_change_a_bit():
    q, k, v = _inputs(71, 73, 79)
    table = np.array([4, 1, 5, 2, 0, 3], np.int32).reshape(R, M)
    lens = np.array([5, 6])
    assert np.array_equal(oracle.paged_attention(q, k, v, table, lens, SCALE, threads=1),
                          oracle.paged_attention(q, k, v, table, lens, SCALE, threads=4))
    qb, kb, vb = oracle.bf16_bits(q), oracle.bf16_bits(k), oracle.bf16_bits(v)
    a = oracle.paged_attention_bf16(qb, kb, vb, table, lens, SCALE, threads=3)
    b = oracle.paged_attention(oracle.bf16_widen(qb), oracle.bf16_widen(kb), oracle.bf16_widen(vb), table, lens, SCALE)
    assert np.array_equal(a, b)


# --------------------------------------------------------------------------- int8 quantizer and projection


def test_quantizer_is_the_formula():
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((24, 40)) * 0.02).astype(np.float32)
    w[3] = 0.0  # a zero row has scale 1
    w[5, 7] = 0.0125  # ties go to even under rint
    codes, scales = oracle.quantize_int8(w)
    assert codes.shape == (40, 24) and scales.shape == (24,) and codes.dtype == np.int8
    for o in range(24):
        mx = np.float32(np.abs(w[o]).max())
        s = np.float32(1.0) if mx == 0 else np.float32(mx / np.float32(127.0))
        assert scales[o] == s
        want = np.clip(np.rint((w[o] / s).astype(np.float64)), -127, 127).astype(np.int8)
        assert np.array_equal(codes[:, o], want)
    assert np.abs(codes).max() == 127 and codes.min() >= -127


def test_int8_projection_equals_the_dequantized_weight_projection():
    """HfMuseGlimmerTest.kt:502-527: (x @ codes) * scale against x @ (codes * scale), 4.7e-6 relative."""
    rng = np.random.default_rng(6)
    w = (rng.standard_normal((48, 64)) * 0.02).astype(np.float32)
    codes, scales = oracle.quantize_int8(w)
    x = rng.standard_normal((5, 64)).astype(np.float32)
    y = oracle.proj_int8(x, codes, scales, round_x_bf16=False)
    deq = codes.astype(np.float32) * scales[None, :]
    y2 = oracle.matmul_f32(x, deq)
    assert np.abs(y - y2).max() <= 4.7e-6 * max(1.0, np.abs(y2).max())
    # reversed scales (the reference's negative control, :537-543) must not agree
    y3 = oracle.proj_int8(x, codes, scales[::-1].copy(), round_x_bf16=False)
    assert np.abs(y3 - y2).max() > 1e-3 * np.abs(y2).max()


def test_matmul_order_is_p_ascending_f32_without_fma():
    rng = np.random.default_rng(7)
    a = rng.standard_normal((3, 37)).astype(np.float32)
    a[1, 4] = 0.0
    b = rng.standard_normal((37, 5)).astype(np.float32)
    got = oracle.matmul_f32(a, b)
    want = np.zeros((3, 5), np.float32)
    for i in range(3):
        for p in range(37):
            if a[i, p] == 0:
                continue
            want[i] = want[i] + (a[i, p] * b[p]).astype(np.float32)
    assert np.array_equal(got, want)
    assert np.array_equal(got, oracle.matmul_f32(a, b, threads=3))


def test_bf16_snap_is_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.005859375, 1.01171875, -3.3, 65504.0, 1e-40], np.float32)
    got = oracle.snap_bf16(x)
    import ml_dtypes

    assert np.array_equal(got, x.astype(ml_dtypes.bfloat16).astype(np.float32))


def test_decode_step_small_shapes_run_and_threads_agree():
    shape = oracle.DecoderShape(num_layers=2, d_model=32, num_heads=4, num_kv_heads=2, head_dim=8, ffn=48, vocab=64,
                                block_size=4)
    w = oracle.make_weights(shape, seed=0)
    P = 8
    kp = [np.zeros((P, 4, 2, 8), np.float32) for _ in range(2)]
    vp = [np.zeros((P, 4, 2, 8), np.float32) for _ in range(2)]
    kp2 = [a.copy() for a in kp]
    vp2 = [a.copy() for a in vp]
    ids = np.array([3, 9], np.int32)
    pos = np.array([0, 0], np.int32)
    tables = np.array([[1, 2], [3, 4]], np.int32)
    lens = np.array([1, 1], np.int32)
    slots = np.array([4, 12], np.int32)
    a = oracle.decode_step(shape, w, kp, vp, ids, pos, tables, lens, slots, threads=1)
    b = oracle.decode_step(shape, w, kp2, vp2, ids, pos, tables, lens, slots, threads=4)
    assert a.shape == (2, 64) and np.all(np.isfinite(a)) and np.array_equal(a, b)


def test_e4m3fn_pool_narrowing_is_xlas_convert():
    """An f8e4m3fn KV pool stores saturateToF8e4m3fn(v) (core/.../Fp8.kt:89-90): clamp to +-448, then the f32 ->
    f8e4m3fn convert (ties to even, subnormals in steps of 2^-9, NaN -> 0x7F).  The restatement is held to an
    independent implementation of the same convert (PyTorch's float8_e4m3fn cast) on every boundary and 200,000 draws,
    and the widening to all 256 codes."""
    import torch

    rng = np.random.default_rng(0)
    x = np.concatenate([
        (rng.standard_normal(200000) * 30).astype(np.float32), (rng.standard_normal(50000) * 0.02).astype(np.float32),
        np.array([0, -0.0, 448, 449, 463.9, 464, 465, 1e9, -1e9, 2 ** -9, 2 ** -10, 1.5 * 2 ** -9, 2.5 * 2 ** -9, 0.0146,
                  0.015625, np.inf, -np.inf, 17.0, 18.0, 19.0, 0.40625, 0.4375], np.float32)])
    mine = oracle.e4m3_bits(x)
    theirs = torch.from_numpy(np.clip(x, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mine, theirs)
    assert oracle.e4m3_bits(np.array([np.nan], np.float32))[0] == 0x7F
    codes = np.arange(256, dtype=np.uint8)
    want = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    got = oracle.e4m3_widen(codes)
    assert np.array_equal(np.isnan(got), np.isnan(want)) and np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])
    assert np.array_equal(oracle.snap_e4m3(np.array([17.0, 19.0, 500.0, -1e9], np.float32)), np.array([16.0, 20.0, 448.0, -448.0], np.float32))
