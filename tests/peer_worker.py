"""Child process of tests/test_tp_gpu.py: one rank of the peer-memory sum (csrc/peer_allreduce.cu), checked against
the sum of the ranks' inputs added in rank order, eagerly and replayed from a CUDA graph."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def rank_input(shape, rank, round_):
    rng = np.random.default_rng(1000 * round_ + rank)
    return (rng.standard_normal(shape) * 10.0 ** rng.integers(-3, 4)).astype(np.float32)


def main():
    from tlaloc_b200 import ops
    from tlaloc_b200.peer import PeerBuffers

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    torch.distributed.init_process_group("nccl", device_id=dev)
    shapes = [(4, 256), (128, 8192), (3, 4), (1, 131076)]  # the last: slices that do not divide evenly into 16-byte units
    peer = PeerBuffers(shapes, rank=rank, world=world, group=torch.distributed.group.WORLD, device=dev, norm_shape=shapes[1])

    def expected(shape, round_):
        acc = rank_input(shape, 0, round_)
        for q in range(1, world):
            acc = acc + rank_input(shape, q, round_)  # f32 adds in rank order, as the kernel does
        return acc

    round_ = 0
    for _ in range(3):
        for i, shape in enumerate(shapes):
            round_ += 1
            peer.tensors[i].copy_(torch.from_numpy(rank_input(shape, rank, round_)))
            out = peer.all_reduce_(i)
            assert np.array_equal(out.cpu().numpy(), expected(shape, round_)), (i, round_)
    # the sum with the RMSNorm folded in: exact sums again, and the normalised rows (bf16) on every rank within one
    # bf16 step of RMSNorm computed from those sums in double
    assert peer.can_fuse_norm(1) and not peer.can_fuse_norm(0)
    gain = torch.from_numpy(np.random.default_rng(77).uniform(0.5, 1.5, size=shapes[1][1]).astype(np.float32)).to(dev)
    for use_gain in (True, False):
        round_ += 1
        peer.tensors[1].copy_(torch.from_numpy(rank_input(shapes[1], rank, round_)))
        out, normed = peer.all_reduce_norm_(1, gain if use_gain else None, 1e-5)
        want = expected(shapes[1], round_)
        assert np.array_equal(out.cpu().numpy(), want), round_
        w64 = want.astype(np.float64)
        ref = w64 / np.sqrt((w64 * w64).mean(axis=1, keepdims=True) + 1e-5)
        if use_gain:
            ref = ref * gain.cpu().numpy().astype(np.float64)[None, :]
        got = normed.float().cpu().numpy().astype(np.float64)
        assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-6), float(np.abs(got - ref).max())
    # the same launches captured in a CUDA graph and replayed: 20 sums back to back on the two big buffers
    src = [torch.empty(s, device=dev) for s in shapes]
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for i in (0, 1):
            peer.tensors[i].copy_(src[i])
            peer.all_reduce_(i)
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    torch.distributed.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(10):
            for i in (0, 1):
                peer.tensors[i].copy_(src[i])
                peer.all_reduce_(i)
    for rep in range(3):
        round_ += 1
        for i in (0, 1):
            src[i].copy_(torch.from_numpy(rank_input(shapes[i], rank, round_)))
        graph.replay()
        for i in (0, 1):
            assert np.array_equal(peer.tensors[i].cpu().numpy(), expected(shapes[i], round_)), (i, rep)
    assert peer.status() == 0
    calls = 3 * len(shapes) + 2 + 2 + 3 * 20
    assert int(peer.state[0].item()) == calls
    # The residual stream distributed by rows: tensor 1 holds bare partials; each rank adds its own rows of the residual
    # stream (rank 0's partial first, then the residual, then the other partials, as the kernel does), keeps the sums
    # locally and every rank receives only the normalised bf16 rows.
    if peer.can_fuse_norm(1):
        rows_, cols_ = shapes[1]
        lo, hi = rows_ * rank // world, rows_ * (rank + 1) // world
        gain_r = torch.from_numpy(np.random.default_rng(5).uniform(0.5, 1.5, size=cols_).astype(np.float32)).to(dev)
        for rep in range(2):
            round_ += 1
            res_all = rank_input(shapes[1], 77, round_)
            own = torch.from_numpy(res_all[lo:hi].copy()).to(dev)
            peer.tensors[1].copy_(torch.from_numpy(rank_input(shapes[1], rank, round_)))
            normed_all = peer.reduce_norm_rows_(1, own, gain_r, 1e-5)
            torch.cuda.synchronize(dev)
            torch.distributed.barrier()
            acc = rank_input(shapes[1], 0, round_) + res_all
            for q in range(1, world):
                acc = acc + rank_input(shapes[1], q, round_)
            assert np.array_equal(own.cpu().numpy(), acc[lo:hi]), rep
            w64 = acc.astype(np.float64)
            ref = w64 / np.sqrt((w64 * w64).mean(axis=1, keepdims=True) + 1e-5) * gain_r.cpu().numpy().astype(np.float64)[None, :]
            got = normed_all.float().cpu().numpy().astype(np.float64)
            assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-6), float(np.abs(got - ref).max())
            torch.distributed.barrier()
        calls += 2
        assert peer.status() == 0 and int(peer.state[0].item()) == calls
        # The same exchange handing over the int8 tensor-core projection's planes instead of bf16 rows: the region holds,
        # bit for bit, what that projection's own quantizer makes of the bf16 rows of the run above with the same inputs.
        round_ += 1
        res_all = rank_input(shapes[1], 77, round_)
        mine = torch.from_numpy(rank_input(shapes[1], rank, round_)).to(dev)
        own = torch.from_numpy(res_all[lo:hi].copy()).to(dev)
        peer.tensors[1].copy_(mine)
        rows_bf16 = peer.reduce_norm_rows_(1, own, gain_r, 1e-5).clone()
        torch.cuda.synchronize(dev)
        torch.distributed.barrier()
        sums = own.clone()
        want_planes = torch.zeros((ops.int8_gemm_scratch_bytes(rows_, cols_, 0) + 3) // 4, device=dev)
        codes = torch.zeros((cols_, 256), dtype=torch.int8, device=dev)
        ops.int8_gemm(rows_bf16, codes, None, scratch=want_planes, i8_mma=True)  # runs the quantizer on the bf16 rows
        own = torch.from_numpy(res_all[lo:hi].copy()).to(dev)
        peer.tensors[1].copy_(mine)
        got_planes = peer.reduce_norm_rows_(1, own, gain_r, 1e-5, planes=True)
        torch.cuda.synchronize(dev)
        torch.distributed.barrier()
        used = (2 * rows_ * cols_ + 4 * rows_) // 4
        assert torch.equal(own, sums)
        assert torch.equal(got_planes[:used].view(torch.int32), want_planes[:used].view(torch.int32))
        # ... and the projection reads them from the peer block
        wq = torch.from_numpy(np.random.default_rng(9).integers(-127, 128, size=(cols_, 256)).astype(np.int8)).to(dev)
        y_quant = ops.int8_gemm(rows_bf16, wq, None, scratch=want_planes, i8_mma=True)
        y_peer = ops.int8_gemm(rows_bf16, wq, None, scratch=got_planes, i8_mma=True, x_planes=True)
        torch.cuda.synchronize(dev)
        assert torch.equal(y_quant, y_peer)
        torch.distributed.barrier()
        calls += 2
        assert peer.status() == 0 and int(peer.state[0].item()) == calls
    # The one-barrier form: out = residual + the ranks' partials in rank order, kept locally, with the RMSNorm.  Two
    # partial buffers in turn (tensors 1 and a twin), eagerly and from a CUDA graph.
    twin = PeerBuffers([shapes[1], shapes[1]], rank=rank, world=world, group=torch.distributed.group.WORLD, device=dev)
    res = torch.empty(shapes[1], device=dev)
    out = torch.empty(shapes[1], device=dev)
    normed = torch.empty(shapes[1], device=dev, dtype=torch.bfloat16)

    def check_one_shot(round_, which, use_res, gain_t):
        want = expected(shapes[1], round_)
        if use_res:
            r = rank_input(shapes[1], 99, round_)
            acc = r + rank_input(shapes[1], 0, round_)  # residual first, then the partials in rank order
            for q in range(1, world):
                acc = acc + rank_input(shapes[1], q, round_)
            want = acc
        assert np.array_equal(out.cpu().numpy(), want), (round_, which, use_res)
        w64 = want.astype(np.float64)
        ref = w64 / np.sqrt((w64 * w64).mean(axis=1, keepdims=True) + 1e-5)
        if gain_t is not None:
            ref = ref * gain_t.cpu().numpy().astype(np.float64)[None, :]
        got = normed.float().cpu().numpy().astype(np.float64)
        assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-6), float(np.abs(got - ref).max())

    for rep in range(4):
        round_ += 1
        which, use_res = rep % 2, rep >= 1
        twin.tensors[which].copy_(torch.from_numpy(rank_input(shapes[1], rank, round_)))
        if use_res:
            res.copy_(torch.from_numpy(rank_input(shapes[1], 99, round_)))
        planes = torch.zeros((ops.int8_gemm_scratch_bytes(shapes[1][0], shapes[1][1], 0) + 3) // 4, device=dev) if rep == 3 else None
        twin.sum_rows_(which, res if use_res else None, out, gain if rep != 2 else None, 1e-5, norm_out=normed, planes=planes)
        check_one_shot(round_, which, use_res, gain if rep != 2 else None)
        if planes is not None:
            # the planes the kernel left for the int8 tensor-core projection are what that projection's own quantizer
            # writes for the same bf16 rows (it is launched by a projection call without x_planes)
            rows_, cols_ = shapes[1]
            other = torch.zeros_like(planes)
            codes = torch.zeros((cols_, 256), dtype=torch.int8, device=dev)
            ops.int8_gemm(normed, codes, None, scratch=other, i8_mma=True)
            torch.cuda.synchronize(dev)
            used = (2 * rows_ * cols_ + 4 * rows_) // 4
            assert torch.equal(planes[:used].view(torch.int32), other[:used].view(torch.int32))
    # in place on the residual stream, replayed from a graph: h += sum(partial 0); h += sum(partial 1); ten times
    hbuf = torch.zeros(shapes[1], device=dev)
    srcs = [torch.empty(shapes[1], device=dev) for _ in range(2)]
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for i in (0, 1):
            twin.tensors[i].copy_(srcs[i])
            twin.sum_rows_(i, hbuf, hbuf, gain, 1e-5, norm_out=normed)
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    torch.distributed.barrier()
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2):
        for _ in range(10):
            for i in (0, 1):
                twin.tensors[i].copy_(srcs[i])
                twin.sum_rows_(i, hbuf, hbuf, gain, 1e-5, norm_out=normed)
    round_ += 1
    parts = [rank_input(shapes[1], q, round_) * np.float32(2.0 ** -6) for q in range(world)]
    srcs[0].copy_(torch.from_numpy(parts[rank]))
    srcs[1].copy_(torch.from_numpy(parts[rank] * np.float32(0.5)))
    hbuf.zero_()
    g2.replay()
    want = np.zeros(shapes[1], np.float32)
    for _ in range(10):
        for scale_ in (np.float32(1.0), np.float32(0.5)):
            for q in range(world):
                want = want + parts[q] * scale_
    assert np.array_equal(hbuf.cpu().numpy(), want)
    assert twin.status() == 0 and int(twin.state[0].item()) == 4 + 2 + 20
    torch.distributed.barrier()
    torch.cuda.synchronize(dev)
    if rank == 0:
        print("peer sum ok", flush=True)
    sys.stdout.flush()
    os._exit(0)  # no process-group teardown over a live CUDA graph


if __name__ == "__main__":
    main()
