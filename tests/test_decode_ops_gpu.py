"""The decode step's small ops against the CPU oracle, through the C ABI (needs a B200)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from tlaloc_b200 import ops as o

    return o


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def test_embedding_rmsnorm_swiglu_argmax():
    rng = np.random.default_rng(0)
    table = oracle.snap_bf16(rng.standard_normal((50, 96)).astype(np.float32))
    ids = np.array([3, 49, 0, 7], np.int32)
    got = ops().embedding(dev(table, torch.bfloat16), dev(ids)).cpu().numpy()
    assert np.array_equal(got, oracle.embedding(table, ids))
    x = rng.standard_normal((5, 4096)).astype(np.float32) * 3
    gain = rng.standard_normal(4096).astype(np.float32)
    want = oracle.rmsnorm(x, gain, 1e-5)
    got = ops().rmsnorm(dev(x), dev(gain), 1e-5).cpu().numpy()
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    got_b = ops().rmsnorm(dev(x), dev(gain), 1e-5, out_dtype=torch.bfloat16).float().cpu().numpy()
    assert np.mean(got_b == oracle.snap_bf16(want)) > 0.99  # a last-ulp difference may flip a bf16 rounding
    assert np.abs(got_b - want).max() <= 8e-3 * np.abs(want).max()
    g, u = rng.standard_normal((3, 688)).astype(np.float32) * 4, rng.standard_normal((3, 688)).astype(np.float32)
    got = ops().swiglu(dev(g), dev(u)).cpu().numpy()
    want = oracle.swiglu(g, u)
    assert np.abs(got - want).max() <= 1e-6 * max(1.0, np.abs(want).max())
    gu = dev(np.concatenate([g, u], axis=1))
    got2 = ops().swiglu(gu[:, :688], gu[:, 688:]).cpu().numpy()
    assert np.array_equal(got, got2)
    logits = rng.standard_normal((6, 128256)).astype(np.float32)
    logits[1, 5] = logits[1, 90000] = 9.0  # a tie: the first index wins
    logits[2, :] = 0.0
    got = ops().argmax(dev(logits)).cpu().numpy()
    assert np.array_equal(got, oracle.argmax(logits)) and got[1] == 5 and got[2] == 0


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
def test_rope_and_kv_write(kv_dtype):
    rng = np.random.default_rng(1)
    T, H, Hkv, hd, P, bs = 5, 8, 2, 64, 12, 16
    qkv = rng.standard_normal((T, (H + 2 * Hkv) * hd)).astype(np.float32)
    q = qkv[:, :H * hd].reshape(T, H, hd)
    k = qkv[:, H * hd:(H + Hkv) * hd].reshape(T, Hkv, hd)
    v = qkv[:, (H + Hkv) * hd:].reshape(T, Hkv, hd)
    pos = np.array([0, 5, 199, 31, 7], np.int32)
    slots = np.array([3, -1, 100, 191, 64], np.int32)
    cos, sin = oracle.rope_tables(10000.0, hd, 200)
    kc0 = rng.standard_normal((P, bs, Hkv, hd)).astype(np.float32)
    vc0 = rng.standard_normal((P, bs, Hkv, hd)).astype(np.float32)
    if kv_dtype == torch.bfloat16:
        kc0, vc0 = oracle.snap_bf16(kc0), oracle.snap_bf16(vc0)
    want_q = oracle.rope(q, pos, cos, sin)
    want_k = oracle.rope(k, pos, cos, sin)
    want_v = v
    if kv_dtype == torch.bfloat16:
        want_k, want_v = oracle.snap_bf16(want_k), oracle.snap_bf16(want_v)
    want_kc = oracle.kv_cache_write(kc0, want_k.reshape(T, -1), slots)
    want_vc = oracle.kv_cache_write(vc0, want_v.reshape(T, -1), slots)
    dq = dev(qkv)
    tq = dq[:, :H * hd].view(T, H, hd)
    tk = dq[:, H * hd:(H + Hkv) * hd].view(T, Hkv, hd)
    tv = dq[:, (H + Hkv) * hd:].view(T, Hkv, hd)
    kc, vc = dev(kc0, kv_dtype), dev(vc0, kv_dtype)
    got_q = ops().rope_kv_write(tq, tk, tv, dev(pos), dev(cos), dev(sin), dev(slots), kc, vc)
    torch.cuda.synchronize()
    assert np.array_equal(got_q.cpu().numpy(), want_q)
    assert np.array_equal(kc.float().cpu().numpy(), want_kc) and np.array_equal(vc.float().cpu().numpy(), want_vc)
    # the standalone KV_CACHE_WRITE: negative slots are padding, slots past the pool are dropped
    pool = dev(kc0, kv_dtype)
    rows = rng.standard_normal((4, Hkv, hd)).astype(np.float32)
    sl = np.array([-1, 5, P * bs + 3, 0], np.int32)
    ops().kv_cache_write(pool, dev(rows), dev(sl))
    ref_rows = oracle.snap_bf16(rows) if kv_dtype == torch.bfloat16 else rows
    want = oracle.kv_cache_write(kc0, ref_rows.reshape(4, -1), np.array([-1, 5, -1, 0], np.int32))
    assert np.array_equal(pool.float().cpu().numpy(), want)


def test_parity_mode_rmsnorm_and_swiglu_are_bit_identical_to_the_oracle():
    """tlaloc_b200_set_order_faithful: RMSNorm sums its squares sequentially in f32 and SiLU runs in double, as the
    interpreter evaluates those nodes (the default kernels use a tree of fused multiply-adds and an f32 exponential)."""
    o = ops()
    rng = np.random.default_rng(21)
    before = o.set_order_faithful(True)
    try:
        for rows, n in [(4, 256), (3, 688), (2, 8192), (5, 37)]:
            x = (rng.standard_normal((rows, n)) * 3).astype(np.float32)
            gain = rng.uniform(0.5, 1.5, size=n).astype(np.float32)
            got = o.rmsnorm(dev(x), dev(gain), 1e-5)
            torch.cuda.synchronize()
            assert np.array_equal(got.cpu().numpy(), oracle.rmsnorm(x, gain, 1e-5))
            got = o.rmsnorm(dev(x), None, 1e-6, out_dtype=torch.bfloat16)
            assert np.array_equal(got.float().cpu().numpy(), oracle.snap_bf16(oracle.rmsnorm(x, None, 1e-6)))
        gu = (rng.standard_normal((6, 2 * 688)) * 4).astype(np.float32)
        t = dev(gu)
        got = o.swiglu(t[:, :688], t[:, 688:])
        torch.cuda.synchronize()
        want = oracle.swiglu(gu[:, :688], gu[:, 688:])
        # the exponential is the device library's double exp, the oracle's is the host's: equal except, at most, where
        # the double quotient sits on an f32 rounding boundary
        assert np.mean(got.cpu().numpy() == want) >= 0.9999 and np.abs(got.cpu().numpy() - want).max() <= 1e-6
    finally:
        o.set_order_faithful(before)
