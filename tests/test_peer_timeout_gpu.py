"""The bounded waits of the tensor-parallel sum, made to run out on ONE GPU without faulting anything: a "world" of
two whose buffers are both ordinary local allocations, in which only rank 0 ever launches.  Rank 1's flag never
arrives, so each wait gives up after the limit the caller put in state[3]; the kernel then finishes, leaves
1 + 16 * phase + rank in state[2], and later launches skip their waits.  All memory is local and every wait is
bounded: nothing here can hang or fault the device."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_peer_that_never_arrives_times_out_and_leaves_the_context_usable():
    from tlaloc_b200 import _native as N
    from tlaloc_b200 import ops

    dev = torch.device("cuda", 0)
    lib = N.lib()
    count = 4096
    flag_offset = 4 * count
    # two "ranks", both in local memory: [count f32 values][2 * world flag words, zero]
    bufs = [torch.zeros((count + 64,), dtype=torch.float32, device=dev) for _ in range(2)]
    bufs[0][:count] = 1.0
    bufs[1][:count] = 2.0
    bases = (ctypes.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    state = torch.zeros((4,), dtype=torch.int32, device=dev)
    state[3] = 3000  # each wait gives up after 3 ms
    stream = torch.cuda.current_stream(dev).cuda_stream
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    N.check(lib.tlaloc_b200_peer_allreduce_f32(bases, 0, flag_offset, state.data_ptr(), 0, 2, count, stream))
    torch.cuda.synchronize(dev)
    first = time.perf_counter() - t0
    st = state.cpu().tolist()
    assert st[2] == 1 + 16 * 0 + 1, st        # the arrive phase gave up on rank 1
    assert st[0] == 1 and st[1] == 0, st      # the launch still completed and reset its CTA counter
    assert 0.002 < first < 2.0, first         # two waits of 3 ms, not the default 20 s
    # rank 0 still reduced its own half from both buffers and wrote it to both
    assert torch.all(bufs[0][:count // 2] == 3.0) and torch.all(bufs[1][:count // 2] == 3.0)
    # a later launch does not wait at all
    t0 = time.perf_counter()
    N.check(lib.tlaloc_b200_peer_allreduce_f32(bases, 0, flag_offset, state.data_ptr(), 0, 2, count, stream))
    torch.cuda.synchronize(dev)
    second = time.perf_counter() - t0
    st = state.cpu().tolist()
    assert st[0] == 2 and st[2] == 2, st
    assert second < 0.002 or second < first / 2, (first, second)
    # the context is alive: another operator of the library runs and is right
    x = torch.randn((8, 256), device=dev)
    got = ops.rmsnorm(x, None, 1e-5)
    want = x * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + 1e-5)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)
    assert lib.tlaloc_b200_device_status() == 0
