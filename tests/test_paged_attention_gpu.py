"""Parity of the CUDA paged-attention path with the CPU oracle, through the C ABI (needs a B200).

Fixtures follow the reference's own tests: permuted block tables, ragged lengths with a partial last page,
poisoned dead slots, shared tables, a sliding window (ir/src/commonTest/.../PagedAttentionTest.kt,
runtime-pjrt/.../kptx/KptxPagedAttentionKernelTest.kt:59-76, PjrtFusedPagedAttentionTest.kt:106-150).
Tolerances: f32 pools max(1e-4, 1e-5*|y|max) (PjrtFusedPagedAttentionTest.kt:94-97); bf16 pools the same
against the oracle evaluated on the bf16-rounded values (the kernel keeps q and p to ~16 bits); the
build-wide floating-point bar is rel 1e-2 / abs 2e-3.
"""
import numpy as np
import pytest
import torch

import oracle
from refdata import dense_twin, pseudo

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops():
    from tlaloc_b200 import ops as o

    return o


def tol_of(want):
    return max(1e-4, 1e-5 * float(np.abs(want).max()))


def run(q, kc, vc, tables, lens, scale, *, q_dtype=torch.float32, kv_dtype=torch.float32, splits=None, **kw):
    o = ops()
    tq = torch.from_numpy(np.ascontiguousarray(q)).to(DEV).to(q_dtype)
    tk = torch.from_numpy(np.ascontiguousarray(kc)).to(DEV).to(kv_dtype)
    tv = torch.from_numpy(np.ascontiguousarray(vc)).to(DEV).to(kv_dtype)
    tt = torch.from_numpy(np.ascontiguousarray(tables, dtype=np.int32)).to(DEV)
    tl = torch.from_numpy(np.ascontiguousarray(lens, dtype=np.int32)).to(DEV)
    keep = kw.pop("keep", None)
    if keep is not None:
        keep = torch.from_numpy(np.ascontiguousarray(keep, dtype=np.int32)).to(DEV)
    scratch = None
    if splits is not None:
        R, H, D = q.shape
        scratch = torch.full((splits, R, H, D + 2), float("nan"), dtype=torch.float32, device=DEV)
    out = o.paged_attention(tq, tk, tv, tt, tl, scale=scale, keep=keep, scratch=scratch, **kw)
    torch.cuda.synchronize()
    if isinstance(out, tuple):
        return out[0].float().cpu().numpy(), out[1].cpu().numpy()
    return out.float().cpu().numpy()


def as_bf16(a):
    return oracle.snap_bf16(a)


# ------------------------------------------------------------------ the reference's tiny shape (generic kernel)

R, H, HKV, D, BS, P, M = 2, 4, 2, 3, 2, 6, 3
CTX = M * BS


def tiny(sq, sk, sv):
    return (pseudo(R * H * D, sq).reshape(R, H, D), pseudo(P * BS * HKV * D, sk).reshape(P, BS, HKV, D),
            pseudo(P * BS * HKV * D, sv).reshape(P, BS, HKV, D))


def test_tiny_shape_matches_oracle_and_dense_twin_over_len_and_window_sweeps():
    q, k, v = tiny(41, 43, 47)
    table = np.array([5, 3, 1, 0, 4, 2], np.int32).reshape(R, M)
    for w in [None] + list(range(1, CTX + 1)):
        for len0 in range(1, CTX + 1):
            lens = np.array([len0, CTX - len0 + 1])
            got = run(q, k, v, table, lens, 0.5, sliding_window=w)
            want = oracle.paged_attention(q, k, v, table, lens, 0.5, sliding_window=w)
            assert np.abs(got - want).max() <= 1e-5, (w, len0)
            assert np.abs(got - dense_twin(q, k, v, table, lens, 0.5, window=w)).max() <= 1e-5


def test_hand_exact_cases():
    q = np.ones((R, H, D), np.float32)
    k = np.zeros((P, BS, HKV, D), np.float32)
    table = np.array([2, 0, 4, 5, 3, 1], np.int32).reshape(R, M)

    def live(lens, fill):
        v = np.full((P, BS, HKV, D), 1000.0, np.float32)
        for s in range(R):
            for t in range(lens[s]):
                v[table[s, t // BS], t % BS] = fill(s, t)
        return v

    lens = np.array([3, 2])
    got = run(q, k, live(lens, lambda s, t: t + 1), table, lens, 0.5)
    assert np.abs(got[0] - 2.0).max() <= 1e-5 and np.abs(got[1] - 1.5).max() <= 1e-5
    lens = np.array([5, 3])
    got = run(q, k, live(lens, lambda s, t: 1000.0 if t < lens[s] - 2 else t + 1), table, lens, 0.5, sliding_window=2)
    assert np.abs(got[0] - 4.5).max() <= 1e-5 and np.abs(got[1] - 2.5).max() <= 1e-5
    v = np.empty((P, BS, HKV, D), np.float32)
    v[:, :, 0], v[:, :, 1] = 10.0, -10.0
    got = run(q, k, v, np.arange(6, dtype=np.int32).reshape(R, M), np.array([4, 4]), 0.5)
    for h in range(H):
        assert np.abs(got[:, h] - (10.0 if h // 2 == 0 else -10.0)).max() <= 1e-5


def test_rows_sharing_a_table_are_bit_equal_to_repeated_tables_and_empty_rows_are_zero():
    rows, per = 6, 3
    q = pseudo(rows * H * D, 211).reshape(rows, H, D)
    k = pseudo(P * BS * HKV * D, 223).reshape(P, BS, HKV, D)
    v = pseudo(P * BS * HKV * D, 227).reshape(P, BS, HKV, D)
    tables = np.array([4, 1, 5, 2, 0, 3], np.int32).reshape(2, M)
    lens = np.array([4, 5, 6, 2, 3, 4])
    for w in (None, 2):
        shared = run(q, k, v, tables, lens, 0.5, sliding_window=w)
        per_row = run(q, k, v, np.repeat(tables, per, axis=0), lens, 0.5, sliding_window=w)
        assert np.array_equal(shared, per_row)
        assert np.abs(shared - oracle.paged_attention(q, k, v, tables, lens, 0.5, sliding_window=w)).max() <= 1e-5
    out, lse = run(q[:2], k, v, np.arange(6, dtype=np.int32).reshape(2, M), np.array([0, 3]), 0.5, return_lse=True)
    _, want_lse = oracle.paged_attention(q[:2], k, v, np.arange(6, dtype=np.int32).reshape(2, M), np.array([0, 3]), 0.5,
                                         return_lse=True)
    assert np.all(out[0] == 0) and np.all(np.isneginf(lse[0])) and np.abs(lse[1] - want_lse[1]).max() <= 1e-5


def test_keep_mask_matches_oracle():
    q, k, v = tiny(61, 67, 71)
    table = np.array([4, 1, 5, 2, 0, 3], np.int32).reshape(R, M)
    lens = np.array([6, 5])
    keep = np.array([[1, 0, 1], [0, 1, 1]], np.int32)
    got = run(q, k, v, table, lens, 0.5, keep=keep)
    want = oracle.paged_attention(q, k, v, table, lens, 0.5, keep=keep)
    assert np.abs(got - want).max() <= 1e-5


# ------------------------------------------------------------------ the KPTX fixture (8 seqs, 8Q/2KV, D 64, block 16)


def kptx_fixture():
    S, Hq, Hk, Dh, bs, mb = 8, 8, 2, 64, 16, 8
    nb = S * mb
    table = np.array([(i * 37 + 11) % nb for i in range(S * mb)], np.int32).reshape(S, mb)
    lens = np.array([mb * bs, 1, 17, 64, 33, mb * bs - 1, 5, 100], np.int32)
    q = pseudo(S * Hq * Dh, 101).reshape(S, Hq, Dh)
    k = pseudo(nb * bs * Hk * Dh, 103).reshape(nb, bs, Hk, Dh)
    v = pseudo(nb * bs * Hk * Dh, 107).reshape(nb, bs, Hk, Dh)
    return q, k, v, table, lens


def test_kptx_fixture_f32_within_1e4_of_the_oracle():
    q, k, v, table, lens = kptx_fixture()
    want = oracle.paged_attention(q, k, v, table, lens, 0.125)
    got = run(q, k, v, table, lens, 0.125)
    assert np.abs(got - want).max() <= 1e-4


@pytest.mark.parametrize("q_dtype", [torch.bfloat16, torch.float32])
def test_kptx_fixture_bf16_pools_take_the_tensor_core_kernel(q_dtype):
    q, k, v, table, lens = kptx_fixture()
    kb, vb = as_bf16(k), as_bf16(v)
    qb = as_bf16(q) if q_dtype == torch.bfloat16 else q
    want = oracle.paged_attention(qb, kb, vb, table, lens, 0.125)
    got = run(qb, kb, vb, table, lens, 0.125, q_dtype=q_dtype, kv_dtype=torch.bfloat16)
    tol = 2e-3 if q_dtype == torch.bfloat16 else tol_of(want)  # a bf16 output is rounded to 8 bits
    assert np.abs(got - want).max() <= tol
    # dead slots poisoned: nothing at or past a row's length may reach the output
    kp, vp = kb.copy(), vb.copy()
    live = np.zeros(k.shape[:2], bool)
    for s in range(8):
        for t in range(lens[s]):
            live[table[s, t // 16], t % 16] = True
    kp[~live], vp[~live] = np.float32(1000.0), np.float32(1000.0)
    got2 = run(qb, kp, vp, table, lens, 0.125, q_dtype=q_dtype, kv_dtype=torch.bfloat16)
    assert np.array_equal(got, got2)


# ------------------------------------------------------------------ decode / verify shapes of the fused-kernel test


def rand_case(rng, rows, tables, heads, kv_heads, dim, bs, width, num_blocks, lens, poison=True):
    q = rng.standard_normal((rows, heads, dim)).astype(np.float32)
    k = rng.standard_normal((num_blocks, bs, kv_heads, dim)).astype(np.float32)
    v = rng.standard_normal((num_blocks, bs, kv_heads, dim)).astype(np.float32)
    tab = np.stack([rng.permutation(num_blocks)[:width] for _ in range(tables)]).astype(np.int32)
    return q, k, v, tab, np.asarray(lens, np.int32)


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
def test_decode_and_verify_shapes_across_slice_boundaries(kv_dtype):
    rng = np.random.default_rng(1)
    cases = [
        dict(rows=3, tables=3, heads=6, kv_heads=2, dim=16, bs=16, width=48, num_blocks=200, lens=[1, 300, 768]),
        dict(rows=8, tables=2, heads=8, kv_heads=2, dim=32, bs=16, width=40, num_blocks=120,
             lens=[500, 501, 502, 503, 30, 31, 32, 33]),
        dict(rows=4, tables=2, heads=24, kv_heads=4, dim=256, bs=16, width=32, num_blocks=80, lens=[400, 401, 64, 65]),
        dict(rows=10, tables=2, heads=16, kv_heads=2, dim=64, bs=16, width=64, num_blocks=140,
             lens=[990 + i if i < 5 else 700 + i for i in range(10)]),  # 40 queries per kv head: five passes of 8
    ]
    for c in cases:
        q, k, v, tab, lens = rand_case(rng, **c)
        if kv_dtype == torch.bfloat16:
            k, v = as_bf16(k), as_bf16(v)
        scale = 1.0 / np.sqrt(c["dim"])
        want = oracle.paged_attention(q, k, v, tab, lens, scale, threads=8)
        got = run(q, k, v, tab, lens, scale, kv_dtype=kv_dtype)
        assert np.abs(got - want).max() <= tol_of(want), c


# ------------------------------------------------------------------ the tensor-core kernel at Llama shapes

EDGE_LENS = [1, 15, 16, 17, 255, 256, 257, 511, 512, 513, 1000, 2049, 4096, 31, 768, 3000]


@pytest.mark.parametrize("heads,kv_heads,dim", [(32, 8, 128), (64, 8, 128), (32, 4, 64), (8, 8, 128)])
@pytest.mark.parametrize("q_dtype", [torch.bfloat16, torch.float32])
def test_llama_shapes_ragged_lengths_permuted_tables(heads, kv_heads, dim, q_dtype):
    rng = np.random.default_rng(heads * 1000 + dim)
    B, bs, width = len(EDGE_LENS), 16, 256
    nb = 700
    q, k, v, tab, lens = rand_case(rng, B, B, heads, kv_heads, dim, bs, width, nb, EDGE_LENS)
    k, v = as_bf16(k), as_bf16(v)
    if q_dtype == torch.bfloat16:
        q = as_bf16(q)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(dim)))
    want = oracle.paged_attention(q, k, v, tab, lens, scale, threads=8)
    got32 = run(q, k, v, tab, lens, scale, q_dtype=q_dtype, kv_dtype=torch.bfloat16)
    if q_dtype == torch.float32:
        assert np.abs(got32 - want).max() <= tol_of(want)
    else:  # bf16 out: half an ulp of bf16 on values up to a few units
        assert np.abs(got32 - want).max() <= 2e-3 + 4e-3 * np.abs(want).max()
    # the split count must not matter beyond rounding: 1 slice, the emitter's 256-position slices, the default
    for splits in (1, 3, 16):
        other = run(q, k, v, tab, lens, scale, q_dtype=q_dtype, kv_dtype=torch.bfloat16, splits=splits)
        assert np.abs(other - want).max() <= (tol_of(want) if q_dtype == torch.float32 else 2e-3 + 4e-3 * np.abs(want).max())


@pytest.mark.parametrize("bs", [8, 16, 32])
@pytest.mark.parametrize("dim", [64, 128])
def test_dead_slots_holding_nan_never_reach_the_output(bs, dim):
    """Slots at or past a row's length hold NaN in both pools (what an unwritten block may hold): the output is, bit
    for bit, that of clean pools.  Block sizes 16 and 32 take the TMA-fed kernel, which copies whole 16-position
    groups and must blank the V rows past the end itself; 8 takes the cp.async form, which never copies them."""
    rng = np.random.default_rng(100 + bs + dim)
    lens = [1, 5, 16, 17, 31, 33, 250, 1023, 1025, 700]
    B, width = len(lens), 1040 // bs + 1
    nb = B * width
    q = rng.standard_normal((B, 16, dim)).astype(np.float32)
    k = as_bf16(rng.standard_normal((nb, bs, 2, dim)).astype(np.float32))
    v = as_bf16(rng.standard_normal((nb, bs, 2, dim)).astype(np.float32))
    tab = rng.permutation(nb).reshape(B, width).astype(np.int32)  # every block belongs to one row
    lens = np.asarray(lens, np.int32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(dim)))
    want = oracle.paged_attention(q, k, v, tab, lens, scale, threads=8)
    clean = run(q, k, v, tab, lens, scale, kv_dtype=torch.bfloat16)
    assert np.abs(clean - want).max() <= tol_of(want)
    kp, vp = k.copy(), v.copy()
    live = np.zeros((nb, bs), bool)
    for r in range(B):
        for t in range(lens[r]):
            live[tab[r, t // bs], t % bs] = True
    kp[~live], vp[~live] = np.float32("nan"), np.float32("nan")
    got = run(q, kp, vp, tab, lens, scale, kv_dtype=torch.bfloat16)
    assert np.isfinite(got).all() and np.array_equal(got, clean)
    from tlaloc_b200 import _native as N

    assert N.lib().tlaloc_b200_device_status() == 0  # no wait for a tile ran out


def test_tensor_core_kernel_window_shared_tables_and_lse():
    rng = np.random.default_rng(9)
    heads, kv_heads, dim, bs, width, nb = 16, 4, 128, 16, 128, 300
    # two verify rows per table (8 queries per kv head), causal lengths
    lens = [700, 701, 45, 46, 2000, 2001, 16, 17]
    q, k, v, tab, lens = rand_case(rng, 8, 4, heads, kv_heads, dim, bs, width, nb, lens)
    k, v = as_bf16(k), as_bf16(v)
    scale = dim ** -0.5
    for w in (None, 1, 100, 640):
        want = oracle.paged_attention(q, k, v, tab, lens, scale, sliding_window=w, threads=8)
        got = run(q, k, v, tab, lens, scale, kv_dtype=torch.bfloat16, sliding_window=w)
        assert np.abs(got - want).max() <= tol_of(want), w
        rep = run(q, k, v, np.repeat(tab, 2, axis=0), lens, scale, kv_dtype=torch.bfloat16, sliding_window=w)
        assert np.abs(rep - want).max() <= tol_of(want), w
    want, want_lse = oracle.paged_attention(q, k, v, tab, lens, scale, return_lse=True, threads=8)
    got, lse = run(q, k, v, tab, lens, scale, kv_dtype=torch.bfloat16, return_lse=True)
    assert np.abs(got - want).max() <= tol_of(want) and np.abs(lse - want_lse).max() <= 1e-4


def test_block_permutation_leaves_the_output_bit_identical():
    """Physical placement must not matter: relabel the pool's blocks and the tables together."""
    rng = np.random.default_rng(11)
    heads, kv_heads, dim, bs, width, nb = 32, 8, 128, 16, 64, 400
    q, k, v, tab, lens = rand_case(rng, 6, 6, heads, kv_heads, dim, bs, width, nb, [1000, 17, 512, 513, 64, 999])
    k, v, q = as_bf16(k), as_bf16(v), as_bf16(q)
    a = run(q, k, v, tab, lens, dim ** -0.5, q_dtype=torch.bfloat16, kv_dtype=torch.bfloat16)
    perm = rng.permutation(nb)
    inv = np.empty(nb, np.int64)
    inv[perm] = np.arange(nb)
    b = run(q, k[perm], v[perm], inv[tab].astype(np.int32), lens, dim ** -0.5, q_dtype=torch.bfloat16, kv_dtype=torch.bfloat16)
    assert np.array_equal(a, b)


def test_operator_config_full_size_against_the_oracle():
    """The paged-attention operator configuration: bf16 Q [32, 32, 128], 8 KV heads, block 16, 4096 physical
    blocks, permuted (aliasing) tables, lengths uniform in [512, 8192], seed 1."""
    rng = np.random.default_rng(1)
    B, Hq, Hk, Dh, bs, nb, width = 32, 32, 8, 128, 16, 4096, 512
    lens = rng.integers(512, 8193, size=B).astype(np.int32)
    q = as_bf16(rng.standard_normal((B, Hq, Dh)).astype(np.float32))
    kbits = oracle.bf16_bits(rng.standard_normal((nb, bs, Hk, Dh)).astype(np.float32))
    vbits = oracle.bf16_bits(rng.standard_normal((nb, bs, Hk, Dh)).astype(np.float32))
    tab = np.stack([rng.permutation(nb)[:width] for _ in range(B)]).astype(np.int32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(Dh)))
    want = oracle.paged_attention_bf16(oracle.bf16_bits(q), kbits, vbits, tab, lens, scale, threads=oracle.host_threads())
    o = ops()
    tk = torch.from_numpy(kbits.view(np.int16)).to(DEV).view(torch.bfloat16)
    tv = torch.from_numpy(vbits.view(np.int16)).to(DEV).view(torch.bfloat16)
    tq = torch.from_numpy(q).to(DEV).to(torch.bfloat16)
    out = o.paged_attention(tq, tk, tv, torch.from_numpy(tab).to(DEV), torch.from_numpy(lens).to(DEV), scale=scale,
                            out=torch.empty((B, Hq, Dh), dtype=torch.float32, device=DEV))
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    err = np.abs(got - want)
    assert err.max() <= 2e-3 and np.all(err <= 2e-3 + 1e-2 * np.abs(want))
    assert err.max() <= tol_of(want)  # and in fact at the f32 kernels' own bar


def test_one_kv_head_per_rank_shape_against_the_oracle_on_sampled_rows():
    """What one of eight tensor-parallel ranks runs in the 70B-shape step: 8 query heads on 1 KV head, batch 128,
    lengths uniform in [1024, 16384], nothing shared between sequences.  The oracle walks a sample of rows (their
    pages gathered into a small pool of their own)."""
    rng = np.random.default_rng(70)
    B, Hq, Hk, Dh, bs = 128, 8, 1, 128, 16
    lens = rng.integers(1024, 16385, size=B).astype(np.int32)
    lens[:4] = [1024, 16384, 4097, 8191]
    need = (lens + bs - 1) // bs
    nb, width = int(need.sum()) + 1, 1024
    perm = 1 + rng.permutation(nb - 1)
    tab = np.zeros((B, width), np.int32)
    o = 0
    for i in range(B):
        tab[i, :need[i]] = perm[o:o + need[i]]
        o += int(need[i])
    g = torch.Generator(device=DEV)
    g.manual_seed(70)
    tk = torch.randn((nb, bs, Hk, Dh), device=DEV, generator=g).to(torch.bfloat16)
    tv = torch.randn((nb, bs, Hk, Dh), device=DEV, generator=g).to(torch.bfloat16)
    tq = torch.randn((B, Hq, Dh), device=DEV, generator=g).to(torch.bfloat16)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(Dh)))
    out = ops().paged_attention(tq, tk, tv, torch.from_numpy(tab).to(DEV), torch.from_numpy(lens).to(DEV), scale=scale,
                                out=torch.empty((B, Hq, Dh), dtype=torch.float32, device=DEV))
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    rows = [0, 1, 2, 3, 64, 127]
    for r in rows:
        pages = torch.from_numpy(tab[r, :need[r]].astype(np.int64)).to(DEV)
        k_r = tk[pages].float().cpu().numpy()
        v_r = tv[pages].float().cpu().numpy()
        want = oracle.paged_attention(tq[r:r + 1].float().cpu().numpy(), k_r, v_r,
                                      np.arange(need[r], dtype=np.int32)[None, :], lens[r:r + 1], scale,
                                      threads=oracle.host_threads())
        err = np.abs(got[r:r + 1] - want)
        assert err.max() <= tol_of(want), (r, float(err.max()))


def test_long_contexts_with_empty_tables_between_and_a_window_on_the_tensor_core_kernel():
    """48 tables x 8 KV heads at up to 16384 positions (four 4096-position slices each), tables of length 0 and 1 in
    between, and a sliding window that moves the first live position off zero.  Pool blocks are shared between tables
    (512 physical blocks) to keep the case small; the oracle walks sampled rows."""
    rng = np.random.default_rng(48)
    B, Hq, Hk, Dh, bs, nb, width = 48, 16, 8, 128, 16, 512, 1024
    lens = rng.integers(15000, 16385, size=B).astype(np.int32)
    lens[[3, 4, 20, 47]] = 0
    lens[[0, 7, 30]] = [16384, 1, 8193]
    q = as_bf16(rng.standard_normal((B, Hq, Dh)).astype(np.float32))
    k = as_bf16(rng.standard_normal((nb, bs, Hk, Dh)).astype(np.float32))
    v = as_bf16(rng.standard_normal((nb, bs, Hk, Dh)).astype(np.float32))
    tab = rng.integers(0, nb, size=(B, width)).astype(np.int32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(Dh)))
    rows = [0, 2, 3, 7, 19, 20, 21, 30, 46, 47]
    for w in (None, 5000):
        got = run(q, k, v, tab, lens, scale, q_dtype=torch.bfloat16, kv_dtype=torch.bfloat16, sliding_window=w,
                  out=torch.empty((B, Hq, Dh), dtype=torch.float32, device=DEV))
        want = oracle.paged_attention(q[rows], k, v, tab[rows], lens[rows], scale, sliding_window=w, threads=oracle.host_threads())
        assert np.abs(got[rows] - want).max() <= tol_of(want), w
        assert not got[[3, 4, 20, 47]].any()  # a row of length 0 is all zeros


def test_pools_off_a_16_byte_boundary_take_the_generic_kernel():
    """A pool that starts 2 bytes into an allocation must not reach the tensor-core kernel's 16-byte copies."""
    rng = np.random.default_rng(13)
    q, k, v, tab, lens = rand_case(rng, 4, 4, 8, 2, 64, 16, 8, 40, [100, 17, 128, 64])
    q, k, v = as_bf16(q), as_bf16(k), as_bf16(v)
    want = oracle.paged_attention(q, k, v, tab, lens, 0.125)
    o = ops()
    bufs = []
    for a in (k, v):
        buf = torch.zeros((a.size + 1,), dtype=torch.bfloat16, device=DEV)
        view = buf[1:].view(*a.shape)
        view.copy_(torch.from_numpy(a).to(DEV))
        assert view.data_ptr() % 16 == 2
        bufs.append(view)
    out = o.paged_attention(torch.from_numpy(q).to(DEV).to(torch.bfloat16), bufs[0], bufs[1], torch.from_numpy(tab).to(DEV),
                            torch.from_numpy(lens.astype(np.int32)).to(DEV), scale=0.125,
                            out=torch.empty(q.shape, dtype=torch.float32, device=DEV))
    torch.cuda.synchronize()
    assert np.abs(out.cpu().numpy() - want).max() <= tol_of(want)
    with pytest.raises(ValueError, match="PAGED_ATTENTION out"):
        o.paged_attention(torch.from_numpy(q).to(DEV), bufs[0], bufs[1], torch.from_numpy(tab).to(DEV),
                          torch.from_numpy(lens.astype(np.int32)).to(DEV), scale=0.125,
                          out=torch.empty((4, 8, 32), dtype=torch.float32, device=DEV))


def test_parity_mode_walks_like_the_interpreter():
    """tlaloc_b200_set_order_faithful: double accumulators, ascending positions, one narrowing; equals the oracle to the
    last bits on f32 and bf16 pools, windows, keep masks, shared tables and empty rows."""
    o = ops()
    rng = np.random.default_rng(14)
    before = o.set_order_faithful(True)
    try:
        q, k, v = tiny(41, 43, 47)
        table = np.array([5, 3, 1, 0, 4, 2], np.int32).reshape(R, M)
        for w in (None, 1, 3):
            for len0 in range(0, CTX + 1):
                lens = np.array([len0, CTX - len0])
                got, lse = run(q, k, v, table, lens, 0.5, sliding_window=w, return_lse=True)
                want, wlse = oracle.paged_attention(q, k, v, table, lens, 0.5, sliding_window=w, return_lse=True)
                assert np.abs(got - want).max() <= 1e-7 and np.array_equal(np.isneginf(lse), np.isneginf(wlse))
        q, k, v, tab, lens = rand_case(rng, 6, 3, 8, 2, 64, 16, 20, 70, [300, 17, 1, 64, 0, 255])
        keep = (rng.random((6, 10)) < 0.7).astype(np.int32)
        for kw in ({}, {"sliding_window": 40}, {"keep": keep}):
            got = run(q, k, v, tab, lens, 0.125, **kw)
            want = oracle.paged_attention(q, k, v, tab, lens, 0.125, **kw)
            assert np.abs(got - want).max() <= 2e-7 * max(1.0, float(np.abs(want).max())), kw
        qb, kb, vb = as_bf16(q), as_bf16(k), as_bf16(v)
        got = run(qb, kb, vb, tab, lens, 0.125, q_dtype=torch.bfloat16, kv_dtype=torch.bfloat16)
        want = oracle.paged_attention(qb, kb, vb, tab, lens, 0.125)
        assert np.abs(got - as_bf16(want)).max() <= 1e-7  # out takes the query's dtype: the same values, snapped once
    finally:
        o.set_order_faithful(before)


def test_refusals_reach_the_caller():
    o = ops()
    from tlaloc_b200._native import KernelError

    q = torch.zeros((2, 4, 8), device=DEV)
    k = torch.zeros((4, 2, 2, 8), device=DEV)
    t = torch.zeros((2, 2), dtype=torch.int32, device=DEV)
    l = torch.ones((2,), dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError, match="sliding_window"):
        o.paged_attention(q, k, k, t, l, scale=0.5, sliding_window=0)
    with pytest.raises(KernelError, match="too few"):
        o.paged_attention(torch.zeros((2, 4, 128), device=DEV, dtype=torch.bfloat16),
                          torch.zeros((4, 16, 2, 128), device=DEV, dtype=torch.bfloat16),
                          torch.zeros((4, 16, 2, 128), device=DEV, dtype=torch.bfloat16),
                          torch.zeros((2, 2000), dtype=torch.int32, device=DEV), l, scale=0.5,
                          scratch=torch.empty((1, 2, 4, 130), device=DEV))
    with pytest.raises(ValueError, match="no CPU path"):
        o.paged_attention(q.cpu(), k.cpu(), k.cpu(), t.cpu(), l.cpu(), scale=0.5)
