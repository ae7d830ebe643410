"""This library's paged attention against the REFERENCE's own CUDA kernel on the same GPU.

oracle/build_ref.sh compiles triton/kernels/paged_attention.cu from the reference checkout for sm_100a into
oracle/_ref/ (where the checkout is mounted; the built library then travels with the tree).  Its typed-FFI handler is
driven with the same hand-built call frames as this library's (tests/ffi_frames.py), on the operand kinds it accepts:
an f32 query with f32 or bf16 pools (triton/kernels/paged_attention.cu:1378,1429-1441).  Bar: 1e-4, the tolerance of
the reference's own kernel test (runtime-pjrt/.../kptx/KptxPagedAttentionKernelTest.kt:96-102)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import ffi_frames as F
import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libtlaloc_ref_kernels.so")


def ref_handler():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libtlaloc_ref_kernels.so has not been built (oracle/build_ref.sh needs the reference checkout)")
    lib = C.CDLL(REF_LIB)
    lib.tlaloc_ref_paged_attention_handler.restype = C.c_void_p
    return F.HANDLER(lib.tlaloc_ref_paged_attention_handler())


def both(q, k, v, tab, lens, scale, kv_dtype):
    """(this library's out, the reference kernel's out) for an f32 query, through call frames on one stream."""
    from tlaloc_b200 import _native as N

    ours, theirs = F.handler(N.lib(), "tlaloc_paged_attention"), ref_handler()
    stream = torch.cuda.Stream(device=DEV)
    xla = F.FakeXla(stream=stream.cuda_stream)
    t = lambda a, dt=None: (torch.from_numpy(np.ascontiguousarray(a)).to(DEV) if dt is None else torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dt))
    R, H, D = q.shape
    S = (tab.shape[1] * k.shape[1] + 255) // 256  # the emitter's scratch sizing
    tq, tk, tv, tt, tl = t(q), t(k, kv_dtype), t(v, kv_dtype), t(tab), t(lens)
    kvt = F.F32 if kv_dtype == torch.float32 else F.BF16
    outs = []
    for h in (ours, theirs):
        assert h(C.byref(xla.frame(F.INITIALIZE))) is None, xla.errors
        out = torch.zeros((R, H, D), device=DEV)
        scratch = torch.zeros((S, R, H, D + 2), device=DEV)
        torch.cuda.synchronize()
        a = [xla.buffer(F.F32, tq.data_ptr(), q.shape), xla.buffer(kvt, tk.data_ptr(), k.shape), xla.buffer(kvt, tv.data_ptr(), v.shape),
             xla.buffer(F.S32, tt.data_ptr(), tab.shape), xla.buffer(F.S32, tl.data_ptr(), lens.shape)]
        r = [xla.buffer(F.F32, out.data_ptr(), q.shape), xla.buffer(F.F32, scratch.data_ptr(), scratch.shape)]
        assert h(C.byref(xla.frame(F.EXECUTE, a, r, {"scale": (F.F32, C.c_float(scale))}))) is None, xla.errors
        stream.synchronize()
        outs.append(out.cpu().numpy())
    return outs


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
def test_the_reference_kernels_own_fixture(kv_dtype):
    """KptxPagedAttentionKernelTest.kt:59-76: 8 sequences, 8 query / 2 KV heads, D 64, block 16, 64 blocks, table entry
    (i * 37 + 11) % 64, lengths [128, 1, 17, 64, 33, 127, 5, 100]."""
    rng = np.random.default_rng(101)
    R, H, Hkv, D, bs, nb, M = 8, 8, 2, 64, 16, 64, 8
    q = rng.standard_normal((R, H, D)).astype(np.float32)
    k = oracle.snap_bf16(rng.standard_normal((nb, bs, Hkv, D)).astype(np.float32))
    v = oracle.snap_bf16(rng.standard_normal((nb, bs, Hkv, D)).astype(np.float32))
    tab = ((np.arange(R * M) * 37 + 11) % nb).astype(np.int32).reshape(R, M)
    lens = np.array([128, 1, 17, 64, 33, 127, 5, 100], np.int32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(D)))
    got, ref = both(q, k, v, tab, lens, scale, kv_dtype)
    want = oracle.paged_attention(q, k, v, tab, lens, scale)
    assert np.abs(got - ref).max() <= 1e-4, float(np.abs(got - ref).max())
    assert np.abs(ref - want).max() <= 1e-4 and np.abs(got - want).max() <= 1e-4


def test_the_operator_configuration_shape():
    """32 sequences, 32 query / 8 KV heads of 128, block 16, 4096 blocks, permuted tables, lengths U[512, 8192], bf16 pools
    (an f32 query: the reference handler takes no other)."""
    rng = np.random.default_rng(1)
    B, H, Hkv, D, bs, nb, width = 32, 32, 8, 128, 16, 4096, 512
    lens = rng.integers(512, 8193, size=B).astype(np.int32)
    q = rng.standard_normal((B, H, D)).astype(np.float32)
    g = torch.Generator(device=DEV)
    g.manual_seed(1)
    k = torch.randn((nb, bs, Hkv, D), device=DEV, generator=g).to(torch.bfloat16).float().cpu().numpy()
    v = torch.randn((nb, bs, Hkv, D), device=DEV, generator=g).to(torch.bfloat16).float().cpu().numpy()
    tab = np.stack([rng.permutation(nb)[:width] for _ in range(B)]).astype(np.int32)
    got, ref = both(q, k, v, tab, lens, float(D ** -0.5), torch.bfloat16)
    assert np.abs(got - ref).max() <= 1e-4, float(np.abs(got - ref).max())


def test_same_gpu_timing_of_both_kernels_on_the_operator_configuration(capsys):
    """Both handlers on the operator configuration with nothing shared between sequences (every (sequence, 16
    positions) its own block: all K/V bytes come from HBM), f32 query, bf16 pools, 20 calls each after 3 warm-ups, CUDA
    events on the handlers' stream.  Prints the two times (run with -s to see them); asserts only that both ran and
    agree."""
    rng = np.random.default_rng(1)
    B, H, Hkv, D, bs, width = 32, 32, 8, 128, 16, 512
    lens = rng.integers(512, 8193, size=B).astype(np.int32)
    need = (lens + bs - 1) // bs
    nb = int(need.sum()) + 1
    perm = 1 + rng.permutation(nb - 1)
    tab = np.zeros((B, width), np.int32)
    o = 0
    for i in range(B):
        tab[i, :need[i]] = perm[o:o + need[i]]
        o += int(need[i])
    from tlaloc_b200 import _native as N

    g = torch.Generator(device=DEV)
    g.manual_seed(1)
    tk = torch.randn((nb, bs, Hkv, D), device=DEV, generator=g).to(torch.bfloat16)
    tv = torch.randn((nb, bs, Hkv, D), device=DEV, generator=g).to(torch.bfloat16)
    tq = torch.randn((B, H, D), device=DEV, generator=g)
    tt, tl = torch.from_numpy(tab).to(DEV), torch.from_numpy(lens).to(DEV)
    S = (width * bs + 255) // 256
    stream = torch.cuda.Stream(device=DEV)
    xla = F.FakeXla(stream=stream.cuda_stream)
    scale = float(D ** -0.5)
    times, outs = {}, {}
    for name, h in (("this library", F.handler(N.lib(), "tlaloc_paged_attention")), ("reference kernel", ref_handler())):
        assert h(C.byref(xla.frame(F.INITIALIZE))) is None, xla.errors
        out = torch.zeros((B, H, D), device=DEV)
        scratch = torch.zeros((S, B, H, D + 2), device=DEV)
        a = [xla.buffer(F.F32, tq.data_ptr(), tq.shape), xla.buffer(F.BF16, tk.data_ptr(), tk.shape), xla.buffer(F.BF16, tv.data_ptr(), tv.shape),
             xla.buffer(F.S32, tt.data_ptr(), tab.shape), xla.buffer(F.S32, tl.data_ptr(), lens.shape)]
        r = [xla.buffer(F.F32, out.data_ptr(), tq.shape), xla.buffer(F.F32, scratch.data_ptr(), scratch.shape)]
        frame = xla.frame(F.EXECUTE, a, r, {"scale": (F.F32, C.c_float(scale))})
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            for _ in range(3):
                assert h(C.byref(frame)) is None, xla.errors
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(20):
                assert h(C.byref(frame)) is None, xla.errors
            e1.record(stream)
        stream.synchronize()
        times[name] = e0.elapsed_time(e1) / 20 * 1e3
        outs[name] = out.cpu().numpy()
    byts = 2 * int(lens.sum()) * Hkv * D * 2 + B * H * D * 8
    with capsys.disabled():
        for name, us in times.items():
            print(f"\n{name}: {us:.1f} us per call, {byts / us / 1e3:.0f} GB/s on the live K/V bytes (f32 query, bf16 pools, nothing shared)")
    assert np.abs(outs["this library"] - outs["reference kernel"]).max() <= 1e-4
