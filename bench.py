"""Benchmark of the decode hot path: decode tokens/s of a Llama-3-shape int8-weight decoder with a paged bf16 KV
cache, on N B200s of one box (tensor parallel), plus the HBM roofline of its dominant kernel and a CPU baseline.

    python bench.py --gpus 1 --steps 20 --warmup 3                                  # this arm (CUDA kernels)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference --gpus 1 --steps 3 --warmup 1                  # the CPU restatement of the reference

One JSON line on stdout (rank 0).  A step is one decode step: one new token for every sequence of the batch.
`value` times K CUDA-graph replays with every input resident in HBM; `e2e` times K steps through
`Decoder.set_inputs` / `Decoder.step` from pinned host buffers, the host->device copy of the step's inputs and the
device->host read of the next tokens inside the timed region.  Data is synthetic: random-init weights of the named
shape, random K/V, context lengths drawn as the configuration states.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (config kwargs, batch, context range, workload string)
    "llama70b": (dict(num_layers=80, d_model=8192, num_heads=64, num_kv_heads=8, head_dim=128, ffn=28672, vocab=128256),
                 128, (1024, 16384), "llama3-70b-shape decode, int8 per-channel weights, bf16 paged KV block 16, "
                                     "batch 128, contexts U[1024,16384], tensor parallel over the GPUs"),
    "llama8b": (dict(num_layers=32, d_model=4096, num_heads=32, num_kv_heads=8, head_dim=128, ffn=14336, vocab=128256),
                64, (128, 4096), "llama3-8b-shape decode, int8 per-channel weights, bf16 paged KV block 16, batch 64, "
                                 "contexts U[128,4096]"),
}
METRIC, UNIT = "decode_tokens_per_s", "tokens/s"


def peaks() -> tuple[float, str]:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], 0.0, set()
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx = max(mx, float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_tables(rng, batch, lens, block_size, num_blocks, max_blocks, steps_ahead):
    """Block tables over `num_blocks` physical blocks (block 0 is the padding page).  Each sequence's past blocks
    are a random draw of the shared pool (sequences alias each other's blocks when the pool is smaller than the
    logical total); the blocks its new tokens land in are its own."""
    tail_first = 1
    tails_per_seq = (steps_ahead + block_size - 1) // block_size + 2
    shared_lo = tail_first + batch * tails_per_seq
    if shared_lo + 16 > num_blocks:
        raise ValueError("the KV pool is too small for this batch")
    tables = np.zeros((batch, max_blocks), np.int32)
    shared = np.arange(shared_lo, num_blocks)
    for i in range(batch):
        full = int(lens[i]) // block_size  # whole blocks of the prompt
        take = rng.choice(shared, size=full, replace=full > len(shared)) if full else np.zeros(0, np.int64)
        tables[i, :full] = take
        own = tail_first + i * tails_per_seq + np.arange(tails_per_seq)
        tables[i, full:full + tails_per_seq] = own
    return tables


def run_ours(args) -> dict:
    import torch

    from tlaloc_b200 import _native
    from tlaloc_b200 import decoder as D
    from tlaloc_b200 import ops, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch N>1 with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
        group = torch.distributed.group.WORLD

    cfg_kw, batch, (lo, hi), wl_name = WORKLOADS[args.workload]
    if args.layers:
        cfg_kw = dict(cfg_kw, num_layers=args.layers)
    K, W = args.steps, args.warmup
    bs = 16
    rng = np.random.default_rng(5)
    lens0 = rng.integers(lo, hi + 1, size=batch).astype(np.int64)
    steps_ahead = 2 * (K + W) + 8
    max_blocks = (hi + steps_ahead + bs - 1) // bs + 1
    cfg = D.DecoderConfig(**cfg_kw, kv_dtype=torch.bfloat16, head_quant=True, max_positions=max_blocks * bs)

    # Size the KV pool: all logical blocks when they fit beside the weights, else what the memory budget allows
    # (then block tables alias physical blocks across sequences; logical bytes are what the step reads).
    hk = cfg.num_kv_heads // world
    block_bytes = 2 * bs * hk * cfg.head_dim * 2 * cfg.num_layers  # K and V, all layers
    logical_blocks = int(np.sum((lens0 + bs - 1) // bs)) + batch * 4 + 64
    free, total = torch.cuda.mem_get_info(dev)
    per_layer_w = cfg.d_model * (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim + cfg.num_heads * cfg.head_dim * cfg.d_model \
        + 3 * cfg.d_model * cfg.ffn
    weight_bytes = (per_layer_w * cfg.num_layers + cfg.vocab * cfg.d_model) // world + 2 * cfg.vocab * cfg.d_model
    budget = min(free - weight_bytes - (12 << 30), int(0.42 * total))
    num_blocks = int(min(logical_blocks, budget // block_bytes))
    aliased = num_blocks < logical_blocks
    tables = make_tables(rng, batch, lens0, bs, num_blocks, max_blocks, steps_ahead)

    dec = D.Decoder(cfg, batch, num_blocks, max_blocks, device=dev, rank=rank, world=world, group=group)
    dec.init_random_weights(seed=0)
    g = torch.Generator(device=dev)
    g.manual_seed(100 + rank)
    for l in range(cfg.num_layers):  # random K/V, N(0,1), filled layer by layer to bound the f32 temporaries
        for pool in (dec.key_pools[l], dec.value_pools[l]):
            flat = pool.view(-1)
            step = 1 << 28
            for o in range(0, flat.numel(), step):
                n = min(step, flat.numel() - o)
                flat[o:o + n] = torch.randn((n,), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)

    def host_inputs(step_no: int):
        pos = lens0 + step_no
        return (rng_ids[step_no % len(rng_ids)], pos.astype(np.int32), tables, (pos + 1).astype(np.int32),
                sharding.slot_mapping(tables, pos, bs))

    rng_ids = [np.random.default_rng(7 + i).integers(0, cfg.vocab, size=batch).astype(np.int32) for i in range(8)]
    pinned = [torch.empty(s, dtype=torch.int32).pin_memory() for s in ((batch,), (batch,), (batch, max_blocks), (batch,), (batch,))]

    def stage(step_no: int):
        for dst, src in zip(pinned, host_inputs(step_no)):
            dst.copy_(torch.from_numpy(np.ascontiguousarray(src, dtype=np.int32)))
        return pinned

    dec.set_inputs(*stage(0))
    torch.cuda.synchronize(dev)
    if world > 1:  # the ranks enter their first exchange together (its waits are bounded)
        torch.distributed.barrier(group=group)
    before = _native.lib().tlaloc_b200_launch_count()
    dec.capture()
    launches_per_step = (_native.lib().tlaloc_b200_launch_count() - before) // 2  # one eager warm-up + one captured

    def barrier():
        if world > 1:
            torch.distributed.barrier(group=group)
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=group)
        return float(t.item())

    # ---- value: K graph replays, inputs resident -------------------------------------------------------------
    for _ in range(W):
        dec.step()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        a.record()
        for _ in range(K):
            dec.step()
        b.record()
        barrier()
    ms_total = max_over_ranks(a.elapsed_time(b))
    ms_step = ms_total / K
    value = batch * K / (ms_total / 1e3)

    # ---- e2e: host buffers in, next tokens out, every step ---------------------------------------------------
    out_host = torch.empty((batch,), dtype=torch.int32).pin_memory()
    for s in range(W):
        dec.set_inputs(*stage(s))
        out_host.copy_(dec.step(), non_blocking=True)
    barrier()
    t0 = time.perf_counter()
    a.record()
    for s in range(K):
        dec.set_inputs(*stage(W + s))
        out_host.copy_(dec.step(), non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()  # the caller reads the tokens before building the next step
    b.record()
    barrier()
    e2e_ms = max_over_ranks(a.elapsed_time(b))
    h2d = int(sum(p.numel() * 4 for p in pinned))
    e2e = {"value": batch * K / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": batch * 4}

    # ---- roofline of the dominant kernel: paged attention (slice + combine), timed alone ---------------------------
    # Timed on a pool of its own in which no two sequences share a block (one layer's worth, a few GB, far larger
    # than L2), so the bytes it is credited with are bytes that come from HBM; the same launches over the step's own
    # pools (which alias blocks when the logical KV does not fit the GPU) are reported beside it.
    lens_now = (lens0 + 1).astype(np.int64)
    att_bytes = 2 * int(lens_now.sum()) * hk * cfg.head_dim * 2 + 2 * batch * (cfg.num_heads // world) * cfg.head_dim * 3
    reps = 20
    dec.set_inputs(*stage(0))
    torch.cuda.synchronize(dev)

    def time_attention(kpools, vpools, tables_dev):
        def att(l):
            ops.paged_attention(dec.q_rot, kpools[l % len(kpools)], vpools[l % len(vpools)], tables_dev, dec.seq_lens,
                                scale=cfg.scale, out=dec.att, scratch=dec.att_scratch)
        for l in range(3):
            att(l)
        torch.cuda.synchronize(dev)
        a.record()
        for l in range(reps):
            att(l)
        b.record()
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b) / reps

    in_step_ms = time_attention(dec.key_pools, dec.value_pools, dec.block_tables)
    need = np.asarray((lens_now + bs - 1) // bs, np.int64)
    own_blocks = int(need.sum()) + 1
    perm = 1 + np.random.default_rng(11).permutation(own_blocks - 1)
    own_tables = np.zeros((batch, max_blocks), np.int32)
    o = 0
    for i in range(batch):
        own_tables[i, :need[i]] = perm[o:o + need[i]]
        o += int(need[i])
    roof_k = torch.empty((own_blocks, bs, hk, cfg.head_dim), dtype=torch.bfloat16, device=dev)
    roof_v = torch.empty_like(roof_k)
    for pool in (roof_k, roof_v):
        flat = pool.view(-1)
        for o in range(0, flat.numel(), 1 << 28):
            n = min(1 << 28, flat.numel() - o)
            flat[o:o + n] = torch.randn((n,), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    att_ms = time_attention([roof_k], [roof_v], torch.from_numpy(own_tables).to(dev))
    del roof_k, roof_v
    peak, peak_kind = peaks()
    achieved = att_bytes / (att_ms / 1e3) / 1e9
    traffic = None
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            per_pos = json.load(f).get("paged_attention_dram_bytes_per_position_per_kv_head")
            if per_pos:
                traffic = float(per_pos) * int(lens_now.sum()) * hk
    except Exception:
        pass
    roofline = {"kernel": "PaSliceMma+PaCombine", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind, "bytes_per_launch": att_bytes,
                "ms_per_launch": att_ms, "pool": "one block per (sequence, 16 positions): nothing shared",
                "in_step_pools": {"ms_per_launch": in_step_ms, "logical_gbs": att_bytes / (in_step_ms / 1e3) / 1e9,
                                  "aliased": bool(aliased)}}
    sb = dec.step_bytes(lens_now)
    step_gbs = (sb["weights"] + sb["kv"]) / (ms_step / 1e3) / 1e9

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 weights x bf16, f32 accumulate; bf16 KV",
        "data": "synthetic",
        "config": {"workload": wl_name, "global_batch": batch, "layers": cfg.num_layers, "parallelism": f"tp{world}",
                   "mean_context": float(lens_now.mean()), "kv_blocks_per_layer": num_blocks,
                   "kv_blocks_logical": logical_blocks, "kv_aliased": bool(aliased),
                   "l2": "inputs larger than L2 (weights and KV pools are tens of GB)", "head": "int8 (headQuant)"},
        "e2e": e2e, "gpu_launches": int(launches_per_step * K), "launches_per_step": int(launches_per_step),
        "clocks": clocks.summary(), "roofline": roofline,
        "step_hbm": {"weights_bytes": sb["weights"], "kv_bytes": sb["kv"], "achieved_gbs": step_gbs, "frac": step_gbs / peak},
    }
    if world > 1:
        line["config"]["rank_sum"] = "peer-memory kernel" if dec.peer is not None else "nccl"
        line["exchange_status"] = dec.exchange_status()  # 0: no bounded wait of the exchange kernel ever gave up
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(cfg_kw, batch, lens_now, seconds=args.cpu_seconds)
    if world > 1:
        # Print first, then leave without tearing the communicator down: destroying a process group whose
        # collectives live inside a CUDA graph blocks, and the process is about to exit anyway.
        if rank == 0:
            print(json.dumps(line), flush=True)
        torch.cuda.synchronize(dev)
        torch.distributed.barrier(group=group)
        sys.stdout.flush()
        os._exit(0)
    return line


def _time_graph(torch, fn, reps, warm=3):
    """Best and median device time (ms) of one CUDA-graph replay of fn()."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[0], ts[len(ts) // 2]


def run_operator(args) -> dict:
    """The two operators alone (single GPU): the paged-attention decode operator (bf16 Q [32, 32, 128], 8 KV heads,
    block 16, 4096 physical blocks, permuted tables, lengths U[512, 8192], seed 1) or the int8 projection sweep
    (N x K in {4096x4096, 14336x4096, 4096x14336, 128256x4096}, M in {1, 8, 32, 128, 256}).  HBM GB/s on algorithmic bytes."""
    import torch

    from tlaloc_b200 import ops
    from tlaloc_b200.attrs import parse_paged_attention

    dev = torch.device("cuda", 0)
    peak, peak_kind = peaks()
    if args.workload == "paged_attn":
        rng = np.random.default_rng(1)
        B, H, Hkv, D, bs, nb, width = 32, 32, 8, 128, 16, 4096, 512
        lens = rng.integers(512, 8193, size=B).astype(np.int32)
        logical = 2 * int(lens.sum()) * Hkv * D * 2 + 2 * B * H * D * 2
        g = torch.Generator(device=dev)
        g.manual_seed(1)
        out = {}
        for name in ("as_configured", "no_shared_blocks"):
            if name == "as_configured":
                P = nb
                tab = np.stack([rng.permutation(nb)[:width] for _ in range(B)]).astype(np.int32)
            else:
                need = (lens + bs - 1) // bs
                P = int(need.sum()) + 1
                perm = 1 + rng.permutation(P - 1)
                tab = np.zeros((B, width), np.int32)
                o = 0
                for i in range(B):
                    tab[i, :need[i]] = perm[o:o + need[i]]
                    o += int(need[i])
            k = torch.randn((P, bs, Hkv, D), device=dev, generator=g).to(torch.bfloat16)
            v = torch.randn((P, bs, Hkv, D), device=dev, generator=g).to(torch.bfloat16)
            q = torch.randn((B, H, D), device=dev, generator=g).to(torch.bfloat16)
            tt, tl = torch.from_numpy(tab).to(dev), torch.from_numpy(lens).to(dev)
            o_t = torch.empty((B, H, D), dtype=torch.bfloat16, device=dev)
            scratch = ops.paged_attention_scratch(parse_paged_attention(q, k, v, tt, tl, scale=D ** -0.5), dev)
            best, med = _time_graph(torch, lambda: ops.paged_attention(q, k, v, tt, tl, scale=D ** -0.5, out=o_t, scratch=scratch),
                                    max(args.steps, 20))
            out[name] = {"us": med * 1e3, "gbs": logical / med / 1e6, "best_gbs": logical / best / 1e6, "physical_blocks": P}
            del k, v
        head = out["no_shared_blocks"]
        return {"metric": "paged_attention_hbm_gbs", "value": head["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": max(args.steps, 20),
                "warmup": 3, "higher_is_better": True, "data": "synthetic", "dtype": "bf16 KV and Q, f32 accumulate",
                "config": {"workload": "paged-attention decode operator alone", "algorithmic_bytes": logical, "cases": out},
                "roofline": {"kernel": "PaSliceMma+PaCombine", "bound": "hbm", "achieved": head["gbs"], "peak": peak,
                             "unit": "GB/s", "frac": head["gbs"] / peak, "peak_kind": peak_kind, "traffic": None}}
    rows = []
    shapes, ms = [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)], (1, 8, 32, 128, 256)
    if args.only:  # one shape "NxKxM", for profiler captures
        n, k, m = (int(v) for v in args.only.lower().split("x"))
        shapes, ms = [(n, k)], (m,)
    for (n, k) in shapes:
        nbuf = max(4, int(400e6 // (k * n)) + 1)  # distinct weight buffers, > 3x L2 in total, visited round robin
        ws = [torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev) for _ in range(nbuf)]
        sc = torch.rand((n,), device=dev) * 0.019 + 0.001
        for m in ms:
            x = torch.randn((m, k), device=dev).to(torch.bfloat16)
            y = torch.empty((m, n), dtype=torch.float32, device=dev)

            def fn():
                for w in ws:
                    ops.int8_gemm(x, w, sc, out=y, weights_const=True)
            best, med = _time_graph(torch, fn, 10)
            byts = k * n + 4 * n + 2 * m * k + 4 * m * n
            rows.append({"N": n, "K": k, "M": m, "us": med / nbuf * 1e3, "gbs": byts / (med / nbuf) / 1e6,
                         "tflops": 2.0 * m * n * k / (med / nbuf) / 1e9})
        del ws
    big = ([r for r in rows if r["N"] == 128256 and r["M"] == 8] or rows)[0]
    return {"metric": "int8_projection_hbm_gbs", "value": big["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": 10, "warmup": 3,
            "higher_is_better": True, "data": "synthetic", "dtype": "int8 weights x bf16, f32 accumulate",
            "config": {"workload": "int8 weight-only projection sweep", "rows": rows},
            "roofline": {"kernel": "Int8GemvKernel", "bound": "hbm", "achieved": big["gbs"], "peak": peak, "unit": "GB/s",
                         "frac": big["gbs"] / peak, "peak_kind": peak_kind, "traffic": None}}


def cpu_sample(cfg_kw, lens, b_sample, threads):
    """One layer of the decode step for `b_sample` sequences through the CPU restatement: the int8 projections and the
    paged attention (the two hot ops), all host threads.  Returns seconds."""
    import oracle

    d, H, Hkv, hd, ffn = cfg_kw["d_model"], cfg_kw["num_heads"], cfg_kw["num_kv_heads"], cfg_kw["head_dim"], cfg_kw["ffn"]
    rng = np.random.default_rng(0)
    lens = np.asarray(lens[:b_sample], np.int32)
    bs = 16
    nblk = int(np.sum((lens + bs - 1) // bs)) + 1
    kbits = rng.integers(0, 1 << 16, size=(nblk, bs, Hkv, hd), dtype=np.uint16) & np.uint16(0xBFFF)
    vbits = rng.integers(0, 1 << 16, size=(nblk, bs, Hkv, hd), dtype=np.uint16) & np.uint16(0xBFFF)
    tab = np.zeros((b_sample, int(lens.max() + bs - 1) // bs), np.int32)
    o = 1
    for i in range(b_sample):
        n = (lens[i] + bs - 1) // bs
        tab[i, :n] = np.arange(o, o + n)
        o += n
    tab = np.minimum(tab, nblk - 1)
    q = oracle.bf16_bits(rng.standard_normal((b_sample, H, hd)).astype(np.float32))
    x = rng.standard_normal((b_sample, d)).astype(np.float32)

    def w(k, n):  # tiled random codes: generating hundreds of MB of random bytes would dominate the sample
        base = rng.integers(-127, 128, size=(k, min(n, 1024)), dtype=np.int8)
        return np.ascontiguousarray(np.tile(base, (1, (n + base.shape[1] - 1) // base.shape[1]))[:, :n])

    ws = {"qkv": w(d, (H + 2 * Hkv) * hd), "o": w(H * hd, d), "gu": w(d, 2 * ffn), "down": w(ffn, d)}
    sc = {k: np.full(v.shape[1], 0.01, np.float32) for k, v in ws.items()}
    t0 = time.perf_counter()
    oracle.proj_int8(x, ws["qkv"], sc["qkv"], threads=threads)
    oracle.paged_attention_bf16(q, kbits, vbits, tab, lens, hd ** -0.5, threads=threads)
    oracle.proj_int8(rng.standard_normal((b_sample, H * hd)).astype(np.float32), ws["o"], sc["o"], threads=threads)
    oracle.proj_int8(x, ws["gu"], sc["gu"], threads=threads)
    oracle.proj_int8(rng.standard_normal((b_sample, ffn)).astype(np.float32), ws["down"], sc["down"], threads=threads)
    return time.perf_counter() - t0


def cpu_baseline(cfg_kw, batch, lens, seconds=15.0) -> dict:
    """About `seconds` of CPU work: the largest batch slice whose one-layer sample stays under a third of the budget,
    then as many one-layer samples as fit (each layer of the step does the same work)."""
    import oracle

    threads = oracle.host_threads()
    b = 1
    t = cpu_sample(cfg_kw, lens, b, threads)
    while t < seconds / 3 and b * 2 <= batch:
        b *= 2
        t = cpu_sample(cfg_kw, lens, b, threads)
    times = [t]
    while sum(times) + t < seconds and len(times) < cfg_kw["num_layers"]:
        times.append(cpu_sample(cfg_kw, lens, b, threads))
    per_layer = float(np.mean(times))
    step_s = per_layer * cfg_kw["num_layers"] * (batch / b)
    return {"value": batch / step_s, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{len(times)} of {cfg_kw['num_layers']} layers (int8 projections + paged attention) for {b} of {batch} "
                      f"sequences: {sum(times):.1f} s on {threads} threads, {per_layer:.2f} s per layer; scaled by layers x batch/{b}"}


def run_reference(args) -> dict:
    """The reference's CPU path for this step cannot run here (its interpreter is Kotlin/JVM; no JVM in the image),
    so this arm times the C restatement of that interpreter (oracle/) on all host threads, a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    import oracle

    cfg_kw, batch, (lo, hi), wl_name = WORKLOADS[args.workload]
    rng = np.random.default_rng(5)
    lens = (rng.integers(lo, hi + 1, size=batch) + 1).astype(np.int64)
    threads = oracle.host_threads()
    b = min(16, batch)  # a step's sample: one layer for 16 sequences (about half a second on 16 threads)
    times = []
    for i in range(args.warmup + args.steps):
        t = cpu_sample(cfg_kw, lens, b, threads)
        if i >= args.warmup:
            times.append(t)
    t = float(np.mean(times))
    step_s = t * cfg_kw["num_layers"] * (batch / b)
    value = batch / step_s
    sample = (f"each step: one of {cfg_kw['num_layers']} layers for {b} of {batch} sequences ({t:.2f} s on {threads} threads), "
              f"scaled by layers x batch/{b}")
    return {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 accumulate on the host (f64 in the attention walk)", "data": "synthetic",
            "config": {"workload": wl_name, "global_batch": batch, "layers": cfg_kw["num_layers"], "parallelism": "host cores"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama70b", choices=sorted(WORKLOADS) + ["paged_attn", "int8_proj"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only; not a bench value)")
    ap.add_argument("--only", default="", help="int8_proj: a single shape NxKxM")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload in ("paged_attn", "int8_proj"):
        line = run_operator(args)
    else:
        line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
