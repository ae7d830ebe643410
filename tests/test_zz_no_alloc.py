"""The allocation-free paged-attention entry point (needs a B200).  Collected last on purpose: if it fails, a run
that stops at the first failure has already run every other test.

Some callers of this library hold device pointers but cannot allocate: a handler inside a CUDA graph capture, a
program whose custom call has no scratch result, a JVM or plugin binding without an allocator.  For them
`tlaloc_b200_paged_attention_static` keeps the split records in an array inside the library.  It must give what
`tlaloc_b200_paged_attention` gives with a caller-owned scratch, call after call, although the array is shared
and keeps whatever the previous call left in it.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, lens, B, H, Hkv, D, bs, width, nb, kv_dtype):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    q = torch.randn((B, H, D), device=DEV, generator=g)
    k = torch.randn((nb, bs, Hkv, D), device=DEV, generator=g).to(kv_dtype)
    v = torch.randn((nb, bs, Hkv, D), device=DEV, generator=g).to(kv_dtype)
    rng = np.random.default_rng(seed)
    tab = torch.from_numpy(np.stack([rng.permutation(nb)[:width] for _ in range(B)]).astype(np.int32)).to(DEV)
    return q, k, v, tab, torch.tensor(lens, dtype=torch.int32, device=DEV)


def _both(q, k, v, tab, lens, scale):
    from tlaloc_b200 import _native as N
    from tlaloc_b200 import ops

    lib = N.lib()
    B, H, D = q.shape
    nb, bs, Hkv, _ = k.shape
    want = ops.paged_attention(q, k, v, tab, lens, scale=scale)  # the existing entry point, caller-owned scratch
    got = torch.full_like(q, float("nan"))
    dt = N.F32 if k.dtype == torch.float32 else N.BF16
    N.check(lib.tlaloc_b200_paged_attention_static(
        q.data_ptr(), N.F32, k.data_ptr(), v.data_ptr(), dt, tab.data_ptr(), lens.data_ptr(), None, 0, got.data_ptr(),
        N.F32, None, B, H, D, nb, bs, Hkv, tab.shape[1], tab.shape[0], scale, 0, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return got.cpu().numpy(), want.cpu().numpy()


@pytest.mark.parametrize("kv_dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_matches_the_caller_scratch_entry_point_on_two_calls_in_a_row(kv_dtype):
    # first call: long rows, many slices in use; second call: short rows, so most of what the first call left in
    # the array is stale and must not be read
    first = _case(1, [2000, 17, 1024, 513, 4096, 300], 6, 16, 4, 128, 16, 256, 600, kv_dtype)
    second = _case(2, [5, 300, 1, 64, 100, 257], 6, 16, 4, 128, 16, 256, 600, kv_dtype)
    for case in (first, second, first):
        got, want = _both(*case, 128 ** -0.5)
        # the parity tests' bar for f32 outputs: max(1e-4, 1e-5 * largest |y|)
        assert np.abs(got - want).max() <= max(1e-4, 1e-5 * np.abs(want).max())


def test_sizes_beyond_the_built_in_array_are_refused_with_both_sizes_named():
    from tlaloc_b200 import _native as N

    lib = N.lib()
    cap = lib.tlaloc_b200_paged_attention_static_scratch_bytes()
    assert cap == 16 << 20
    one = 256  # never dereferenced: the refusal comes before any launch
    # 512 rows x 64 heads x (128 + 2) floats is 17 MB for a single slice: more than the array holds
    rc = lib.tlaloc_b200_paged_attention_static(one, N.F32, one, one, N.BF16, one, one, None, 0, one, N.F32, None, 512, 64,
                                                128, 100, 16, 8, 64, 512, 0.1, 0, None)
    msg = lib.tlaloc_b200_last_error().decode()
    assert rc == N.INVALID_ARGUMENT and str(cap) in msg and "bytes of split records" in msg
