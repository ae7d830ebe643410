"""The typed-FFI handlers end to end on a B200: INITIALIZE, then EXECUTE on a stream handed over through
XLA_FFI_Stream_Get, against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

import ffi_frames as F
import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_paged_attention_int8_gemm_and_kv_write_through_call_frames():
    from tlaloc_b200 import _native as N

    lib = N.lib()
    stream = torch.cuda.Stream(device=DEV)
    xla = F.FakeXla(stream=stream.cuda_stream)
    rng = np.random.default_rng(0)
    t = lambda a, dt=None: (torch.from_numpy(np.ascontiguousarray(a)).to(DEV) if dt is None else torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dt))
    for name in ("tlaloc_paged_attention", "tlaloc_int8_gemm", "tlaloc_kv_cache_write"):
        assert F.handler(lib, name)(C.byref(xla.frame(F.INITIALIZE))) is None
    # --- paged attention, the emitter's scratch sizing S = ceil(M*bs / 256)
    R, H, Hkv, D, bs, nb, M = 4, 8, 2, 128, 16, 80, 40
    q = rng.standard_normal((R, H, D)).astype(np.float32)
    k = oracle.snap_bf16(rng.standard_normal((nb, bs, Hkv, D)).astype(np.float32))
    v = oracle.snap_bf16(rng.standard_normal((nb, bs, Hkv, D)).astype(np.float32))
    tab = np.stack([rng.permutation(nb)[:M] for _ in range(R)]).astype(np.int32)
    lens = np.array([1, 300, 640, 17], np.int32)
    scale = D ** -0.5
    S = (M * bs + 255) // 256
    tq, tk, tv, tt, tl = t(q), t(k, torch.bfloat16), t(v, torch.bfloat16), t(tab), t(lens)
    out = torch.zeros((R, H, D), device=DEV)
    scratch = torch.empty((S, R, H, D + 2), device=DEV)
    lse = torch.empty((R, H), device=DEV)
    torch.cuda.synchronize()
    a = [xla.buffer(F.F32, tq.data_ptr(), q.shape), xla.buffer(F.BF16, tk.data_ptr(), k.shape), xla.buffer(F.BF16, tv.data_ptr(), v.shape),
         xla.buffer(F.S32, tt.data_ptr(), tab.shape), xla.buffer(F.S32, tl.data_ptr(), lens.shape)]
    r = [xla.buffer(F.F32, out.data_ptr(), q.shape), xla.buffer(F.F32, scratch.data_ptr(), scratch.shape), xla.buffer(F.F32, lse.data_ptr(), (R, H))]
    attrs = {"scale": (F.F32, C.c_float(scale)), "prefill_f16": (F.S32, C.c_int32(1))}
    assert F.handler(lib, "tlaloc_paged_attention")(C.byref(xla.frame(F.EXECUTE, a, r, attrs))) is None, xla.errors
    stream.synchronize()
    want, want_lse = oracle.paged_attention(q, k, v, tab, lens, float(np.float32(scale)), return_lse=True)
    assert np.abs(out.cpu().numpy() - want).max() <= 1e-4 and np.abs(lse.cpu().numpy() - want_lse).max() <= 1e-4
    # --- int8 projection with a residual, f32 activations (cast to bf16 through the scratch result)
    m, kk, n = 5, 512, 1024
    x = rng.standard_normal((m, kk)).astype(np.float32)
    codes = rng.integers(-127, 128, size=(kk, n), dtype=np.int8)
    scales = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    res = rng.standard_normal((m, n)).astype(np.float32)
    tx, tw, ts, tr = t(x), t(codes), t(scales), t(res)
    y = torch.zeros((m, n), device=DEV)
    sc = torch.empty((m * kk,), device=DEV)
    torch.cuda.synchronize()
    a = [xla.buffer(F.F32, tx.data_ptr(), x.shape), xla.buffer(F.S8, tw.data_ptr(), codes.shape), xla.buffer(F.F32, ts.data_ptr(), (n,)),
         xla.buffer(F.F32, tr.data_ptr(), res.shape)]
    r = [xla.buffer(F.F32, y.data_ptr(), (m, n)), xla.buffer(F.F32, sc.data_ptr(), (m * kk,))]
    assert F.handler(lib, "tlaloc_int8_gemm")(C.byref(xla.frame(F.EXECUTE, a, r))) is None, xla.errors
    stream.synchronize()
    wanty = oracle.proj_int8(x, codes, scales, round_x_bf16=True) + res
    assert np.abs(y.cpu().numpy() - wanty).max() <= 1e-4 * max(1.0, np.abs(wanty).max())
    # --- the same call with 40 integer-valued rows and the i8_mma attribute: the int8 tensor-core kernel, exact sums
    m2 = 40
    x2 = rng.integers(-8, 9, size=(m2, kk)).astype(np.float32)
    tx2, y2 = t(x2), torch.zeros((m2, n), device=DEV)
    sc2 = torch.empty((m2 * kk,), device=DEV)  # 4 bytes per element: more than the two int8 planes and the row steps need
    torch.cuda.synchronize()
    before = lib.tlaloc_b200_launch_count()
    a = [xla.buffer(F.F32, tx2.data_ptr(), x2.shape), xla.buffer(F.S8, tw.data_ptr(), codes.shape), xla.buffer(F.F32, ts.data_ptr(), (n,))]
    r = [xla.buffer(F.F32, y2.data_ptr(), (m2, n)), xla.buffer(F.F32, sc2.data_ptr(), (m2 * kk,))]
    assert F.handler(lib, "tlaloc_int8_gemm")(C.byref(xla.frame(F.EXECUTE, a, r, {"i8_mma": (F.S32, C.c_int32(1))}))) is None, xla.errors
    stream.synchronize()
    assert lib.tlaloc_b200_launch_count() - before == 2  # the row quantizer and the projection
    want2 = (x2.astype(np.float64) @ codes.astype(np.float64)).astype(np.float32) * scales[None, :]
    assert np.array_equal(y2.cpu().numpy(), want2)
    # --- KV write into a distinct result buffer: the pool is copied, then the rows land; negative slot = padding
    pool = rng.standard_normal((6, 16, 2, 64)).astype(np.float32)
    rows = rng.standard_normal((3, 2, 64)).astype(np.float32)
    slots = np.array([5, -1, 95], np.int32)
    tp, tro, tsl = t(pool), t(rows), t(slots)
    outp = torch.zeros_like(tp)
    torch.cuda.synchronize()
    a = [xla.buffer(F.F32, tp.data_ptr(), pool.shape), xla.buffer(F.F32, tro.data_ptr(), rows.shape), xla.buffer(F.S32, tsl.data_ptr(), (3,))]
    assert F.handler(lib, "tlaloc_kv_cache_write")(C.byref(xla.frame(F.EXECUTE, a, [xla.buffer(F.F32, outp.data_ptr(), pool.shape)]))) is None
    stream.synchronize()
    assert np.array_equal(outp.cpu().numpy(), oracle.kv_cache_write(pool, rows.reshape(3, -1), slots))
    assert xla.errors == []


def test_paged_attention_handler_takes_e4m3fn_pools():
    """An artifact exported with f8e4m3fn KV pools hands the handler buffers of XLA_FFI_DataType_F8E4M3FN (20)."""
    from tlaloc_b200 import _native as N

    lib = N.lib()
    stream = torch.cuda.Stream(device=DEV)
    xla = F.FakeXla(stream=stream.cuda_stream)
    rng = np.random.default_rng(2)
    R, H, Hkv, D, bs, nb, M = 3, 8, 2, 128, 16, 40, 20
    q = rng.standard_normal((R, H, D)).astype(np.float32)
    k = oracle.snap_e4m3((rng.standard_normal((nb, bs, Hkv, D)) * 2).astype(np.float32))
    v = oracle.snap_e4m3((rng.standard_normal((nb, bs, Hkv, D)) * 2).astype(np.float32))
    tab = np.stack([rng.permutation(nb)[:M] for _ in range(R)]).astype(np.int32)
    lens = np.array([1, 300, 17], np.int32)
    scale = D ** -0.5
    S = (M * bs + 255) // 256
    tq = torch.from_numpy(q).to(DEV)
    tk = torch.from_numpy(oracle.e4m3_bits(k)).to(DEV)
    tv = torch.from_numpy(oracle.e4m3_bits(v)).to(DEV)
    tt, tl = torch.from_numpy(tab).to(DEV), torch.from_numpy(lens).to(DEV)
    out = torch.zeros((R, H, D), device=DEV)
    scratch = torch.empty((S, R, H, D + 2), device=DEV)
    torch.cuda.synchronize()
    F8 = 20
    a = [xla.buffer(F.F32, tq.data_ptr(), q.shape), xla.buffer(F8, tk.data_ptr(), k.shape), xla.buffer(F8, tv.data_ptr(), v.shape),
         xla.buffer(F.S32, tt.data_ptr(), tab.shape), xla.buffer(F.S32, tl.data_ptr(), lens.shape)]
    r = [xla.buffer(F.F32, out.data_ptr(), q.shape), xla.buffer(F.F32, scratch.data_ptr(), scratch.shape)]
    h = F.handler(lib, "tlaloc_paged_attention")
    assert h(C.byref(xla.frame(F.INITIALIZE))) is None
    assert h(C.byref(xla.frame(F.EXECUTE, a, r, {"scale": (F.F32, C.c_float(scale))}))) is None, xla.errors
    stream.synchronize()
    want = oracle.paged_attention(q, k, v, tab, lens, float(np.float32(scale)))
    assert np.abs(out.cpu().numpy() - want).max() <= 1e-4
