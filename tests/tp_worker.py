"""Child process of tests/test_tp_gpu.py: one rank of a tensor-parallel tiny decoder (NCCL), checked against the oracle on rank 0."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    import oracle
    from tlaloc_b200 import decoder as D
    from tlaloc_b200 import sharding

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    torch.distributed.init_process_group("nccl", device_id=dev)
    # TP_WORKER_BATCH=32 (with an FFN width whose per-rank half tiles in blocks of 128) puts the layers' projections on the
    # int8 tensor-core form, SwiGLU in the gate|up epilogue and, with the row-distributed exchange, the exchange's planes
    big = int(os.environ.get("TP_WORKER_BATCH", "4")) > 16
    dims = dict(D.TINY, ffn=512) if big else dict(D.TINY)
    shape = oracle.DecoderShape(num_layers=dims["num_layers"], d_model=dims["d_model"], num_heads=dims["num_heads"],
                                num_kv_heads=dims["num_kv_heads"], head_dim=dims["head_dim"], ffn=dims["ffn"], vocab=dims["vocab"],
                                kv_dtype="bf16", head_quant=True)
    w = oracle.make_weights(shape, seed=0)
    cfg = D.DecoderConfig(**dims, kv_dtype=torch.bfloat16, head_quant=True, max_positions=256)
    B, bs, M = int(os.environ.get("TP_WORKER_BATCH", "4")), 16, 6
    rng = np.random.default_rng(1)
    tables = (1 + rng.permutation(B * M)).reshape(B, M).astype(np.int32)
    dec = D.Decoder(cfg, B, 1 + B * M, M, device=dev, rank=rank, world=world, group=torch.distributed.group.WORLD)
    dec.load_host_weights(w)
    if big and os.environ.get("TLALOC_B200_TP_REDUCE") == "peer2":
        assert dec.i8_mma and dec.rows_residual and dec.rows_planes and dec.fuse_swiglu
    kp = [np.zeros((1 + B * M, bs, 2, 64), np.float32) for _ in range(2)]
    vp = [np.zeros_like(a) for a in kp]
    ids = rng.integers(0, 1024, size=B).astype(np.int32)
    worst, swaps = 0.0, 0
    for step in range(40):
        pos = np.full(B, step, np.int32)
        lens = pos + 1
        slots = sharding.slot_mapping(tables, pos, bs)
        dec.set_inputs(ids, pos, tables, lens, slots)
        if step == 8:
            dec.capture()  # the rest of the run replays the CUDA graph, all-reduces included
        nxt = dec.step().cpu().numpy()
        want = oracle.decode_step(shape, w, kp, vp, ids, pos, tables, lens, slots, threads=8)
        want_tok = oracle.argmax(want).astype(np.int32)
        vp_rank = shape.vocab // world
        got = dec.logits.cpu().numpy()
        err = np.abs(got - want[:, rank * vp_rank:(rank + 1) * vp_rank])
        assert np.all(err <= 2e-3 + 1e-2 * np.abs(want).max(axis=1, keepdims=True)), (step, float(err.max()))
        worst = max(worst, float(err.max()))
        for i in np.nonzero(nxt != want_tok)[0]:
            gap = float(want[i, want_tok[i]] - want[i, nxt[i]])
            assert gap <= (2.0 * float(err[i].max()) if big else 2 * 5e-3), (step, i, gap)  # only a near-tie may swap
            swaps += 1
        ids = want_tok
    assert swaps <= max(2, int(0.015 * 40 * B))
    assert dec.exchange_status() == 0
    torch.distributed.barrier()
    torch.cuda.synchronize(dev)
    if rank == 0:
        print(f"TP{world} ok: worst logit |d| {worst:.2e}, near-tie swaps {swaps}", flush=True)
    # No destroy_process_group(): it blocks while a CUDA graph still holds the captured collectives.
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
