"""The tensor-parallel partition on CPU: two gloo ranks each run their shard of a decode step with the oracle's
primitives, all-reduce the o_proj / down_proj partial sums, merge their greedy candidates, and must reproduce the
unsharded step (same f32 sums up to the order of one addition per all-reduce)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from tlaloc_b200 import sharding

SHAPE = dict(num_layers=2, d_model=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn=96, vocab=128, block_size=4,
             head_quant=True)


def _inputs():
    rng = np.random.default_rng(3)
    B, bs, M = 3, 4, 4
    tables = (1 + rng.permutation(B * M)).reshape(B, M).astype(np.int32)
    lens0 = np.array([5, 1, 9])
    return B, bs, tables, lens0, rng.integers(0, 128, size=(4, B)).astype(np.int32)


def _tp_step(shape, w, rank, world, kp, vp, ids, pos, tables, lens, slots):
    """One decode step on this rank's shard; mirrors tlaloc_b200.decoder.Decoder._run_step with NumPy + gloo."""
    H, Hkv, hd, f = shape.num_heads // world, shape.num_kv_heads // world, shape.head_dim, shape.ffn // world
    B = len(ids)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    cos, sin = oracle.rope_tables(shape.rope_theta, hd, int(pos.max()) + 1)

    def all_reduce(x):
        t = torch.from_numpy(np.ascontiguousarray(x))
        dist.all_reduce(t)
        return t.numpy()

    h = oracle.embedding(w.embed, ids)
    for l, lw in enumerate(w.layers):
        s = sharding.shard_layer(lw, shape.num_heads, shape.num_kv_heads, hd, shape.ffn, rank, world)
        hn = oracle.rmsnorm(h, s["ln1"], shape.rms_eps)
        qkv = oracle.proj_int8(hn, *s["qkv"])
        q = oracle.rope(qkv[:, :H * hd].reshape(B, H, hd), pos, cos, sin)
        k = oracle.rope(qkv[:, H * hd:(H + Hkv) * hd].reshape(B, Hkv, hd), pos, cos, sin)
        v = qkv[:, (H + Hkv) * hd:].reshape(B, Hkv, hd)
        oracle.kv_cache_write_inplace(kp[l], k.reshape(B, -1), slots)
        oracle.kv_cache_write_inplace(vp[l], v.reshape(B, -1), slots)
        att = oracle.paged_attention(q, kp[l], vp[l], tables, lens, scale)
        part = oracle.proj_int8(att.reshape(B, -1), *s["o"])
        h = all_reduce(part + h if rank == 0 else part)  # the residual enters the sum once
        hn2 = oracle.rmsnorm(h, s["ln2"], shape.rms_eps)
        gu = oracle.proj_int8(hn2, *s["gate_up"])
        part = oracle.proj_int8(oracle.swiglu(gu[:, :f], gu[:, f:]), *s["down"])
        h = all_reduce(part + h if rank == 0 else part)
    hf = oracle.rmsnorm(h, w.final_norm, shape.rms_eps)
    logits = oracle.proj_int8(hf, *sharding.shard_head(w.head, shape.vocab, rank, world))
    best = oracle.argmax(logits).astype(np.int32)
    vals = [torch.empty(B) for _ in range(world)]
    ids_l = [torch.empty(B, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(vals, torch.from_numpy(logits[np.arange(B), best].copy()))
    dist.all_gather(ids_l, torch.from_numpy(best))
    tok = sharding.merge_greedy(torch.stack(vals).numpy(), torch.stack(ids_l).numpy(), shape.vocab // world)
    full = [torch.empty(logits.shape) for _ in range(world)]
    dist.all_gather(full, torch.from_numpy(logits))
    return np.concatenate([t.numpy() for t in full], axis=1), tok


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shape = oracle.DecoderShape(**SHAPE)
        w = oracle.make_weights(shape, seed=1)
        B, bs, tables, lens0, id_steps = _inputs()
        Hkv = shape.num_kv_heads // world
        kp = [np.zeros((1 + B * 4, bs, Hkv, shape.head_dim), np.float32) for _ in range(shape.num_layers)]
        vp = [np.zeros_like(a) for a in kp]
        out = []
        for step, ids in enumerate(id_steps):
            pos = (lens0 - 1 + step).astype(np.int32)
            out.append(_tp_step(shape, w, rank, world, kp, vp, ids, pos, tables, (pos + 1).astype(np.int32),
                                sharding.slot_mapping(tables, pos, bs)))
        if rank == 0:
            q.put(out)
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_step_matches_the_unsharded_oracle():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    shape = oracle.DecoderShape(**SHAPE)
    w = oracle.make_weights(shape, seed=1)
    B, bs, tables, lens0, id_steps = _inputs()
    kp = [np.zeros((1 + B * 4, bs, shape.num_kv_heads, shape.head_dim), np.float32) for _ in range(shape.num_layers)]
    vp = [np.zeros_like(a) for a in kp]
    # Steps where every activation rounds to bf16 the same way on both sides agree to f32 rounding; an all-reduce
    # changes one addition's order, which now and then flips a bf16 rounding of an activation (a few 1e-3 on a logit).
    for step, ids in enumerate(id_steps):
        pos = (lens0 - 1 + step).astype(np.int32)
        want = oracle.decode_step(shape, w, kp, vp, ids, pos, tables, (pos + 1).astype(np.int32),
                                  sharding.slot_mapping(tables, pos, bs))
        logits, tok = got[step]
        assert np.abs(logits - want).max() <= 2e-3 + 1e-2 * np.abs(want).max()
        assert np.array_equal(tok, oracle.argmax(logits))  # the merge is the first-maximum rule over the full row


def test_sharding_helpers():
    shape = oracle.DecoderShape(**SHAPE)
    w = oracle.make_weights(shape, seed=2)
    parts = [sharding.shard_layer(w.layers[0], 4, 2, 16, 96, r, 2) for r in range(2)]
    assert parts[0]["qkv"][0].shape == (64, (2 + 2) * 16) and parts[0]["o"][0].shape == (32, 64)
    assert np.array_equal(np.concatenate([parts[0]["o"][0], parts[1]["o"][0]], axis=0), w.layers[0]["o"][0])
    assert np.array_equal(parts[1]["qkv"][0][:, :32], w.layers[0]["q"][0][:, 32:])
    assert np.array_equal(parts[1]["gate_up"][1][48:], w.layers[0]["up"][1][48:])
    with pytest.raises(ValueError):
        sharding.check_world(4, 2, 96, 128, 3)
    vals = np.array([[1.0, 5.0, 2.0], [1.0, 4.0, 3.0]], np.float32)
    ids = np.array([[7, 1, 2], [0, 9, 5]], np.int32)
    assert sharding.merge_greedy(vals, ids, 64).tolist() == [7, 1, 64 + 5]  # a tie goes to the lower rank (lower ids)
    tables = np.array([[3, 9], [4, 1]], np.int32)
    assert sharding.slot_mapping(tables, np.array([5, 2]), 4).tolist() == [9 * 4 + 1, 4 * 4 + 2]


def test_interleaved_gate_up_layout():
    """Blocks of 256 columns: 128 gate columns, then the same 128 up columns (the layout the fused SwiGLU epilogue reads)."""
    import numpy as np

    from tlaloc_b200 import sharding

    k, f = 6, 384
    gate = (np.arange(k * f, dtype=np.int32).reshape(k, f) % 100).astype(np.int8), np.arange(f, dtype=np.float32)
    up = (-(np.arange(k * f, dtype=np.int32).reshape(k, f) % 100)).astype(np.int8), -np.arange(f, dtype=np.float32) - 1
    codes, scales = sharding.interleave_gate_up(gate, up)
    assert codes.shape == (k, 2 * f) and scales.shape == (2 * f,)
    for t in range(f // 128):
        assert np.array_equal(codes[:, 256 * t:256 * t + 128], gate[0][:, 128 * t:128 * (t + 1)])
        assert np.array_equal(codes[:, 256 * t + 128:256 * (t + 1)], up[0][:, 128 * t:128 * (t + 1)])
        assert np.array_equal(scales[256 * t:256 * t + 128], gate[1][128 * t:128 * (t + 1)])
        assert np.array_equal(scales[256 * t + 128:256 * (t + 1)], up[1][128 * t:128 * (t + 1)])
    import pytest
    with pytest.raises(ValueError):
        sharding.interleave_gate_up((gate[0][:, :100], gate[1][:100]), (up[0][:, :100], up[1][:100]))
    lw = {n: (np.zeros((256, 256), np.int8), np.zeros(256, np.float32)) for n in ("q", "k", "v", "o")}
    lw.update(gate=(np.ones((256, 512), np.int8), np.ones(512, np.float32)), up=(np.full((256, 512), 2, np.int8), np.full(512, 2, np.float32)),
              down=(np.zeros((512, 256), np.int8), np.zeros(256, np.float32)), ln1=np.ones(256, np.float32), ln2=np.ones(256, np.float32))
    s = sharding.shard_layer(lw, 4, 4, 64, 512, rank=1, world=2, fuse_swiglu=True)
    assert s["gate_up"][0].shape == (256, 512) and np.all(s["gate_up"][0][:, :128] == 1) and np.all(s["gate_up"][0][:, 128:256] == 2)
