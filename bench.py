"""Benchmark of the decode hot path: decode tokens/s of a Llama-3-shape int8-weight decoder with a paged bf16 KV
cache, on N B200s of one box (tensor parallel), plus the HBM roofline of its kernels and a CPU baseline.

    python bench.py --gpus 1 --steps 20 --warmup 3                                  # this arm (CUDA kernels)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference --gpus 1 --steps 3 --warmup 1                  # the CPU restatement of the reference
    python bench.py --workload llama8b | paged_attn | int8_proj | peer_sum          # one configuration / operator alone
    python bench.py --timeline                                                      # per-kernel times inside one step

One JSON line on stdout (rank 0).  A step is one decode step: one new token for every sequence of the batch.
`value` times K CUDA-graph replays with every input resident in HBM; `e2e` times K steps through
`Decoder.set_inputs` / `Decoder.step` from pinned host buffers, the host->device copy of the step's inputs and the
device->host read of the next tokens inside the timed region.  Data is synthetic: random-init weights of the named
shape, random K/V, context lengths drawn as the configuration states.

The default line (70B shape) also carries, at one GPU: `roofline_projection` (the step's four int8 projections timed
alone at the step's batch), `operators` (the paged-attention operator configuration and the int8 projection sweep) and
`llama8b` (the 8B-shape configuration, the one that fits a single GPU without sharing KV pages).  At two or more GPUs
it first checks the tensor-parallel path (`tp_parity`: the sum over ranks bit for bit, a small sharded decoder against
the CPU oracle) and exits non-zero if that fails.
"""
from __future__ import annotations

import argparse
import gc
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
BS = 16  # KV block size


def peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p["bf16_tflops_sustained"]), "kind": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


def host_cores() -> int:
    """Host threads this process may use: its affinity mask (not $OMP_NUM_THREADS, which a launcher may pin to 1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


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


def fill_normal_bf16(torch, pool, gen):
    """N(0, 1) into a (possibly huge) bf16 or e4m3fn tensor, piece by piece to bound the f32 temporaries."""
    flat = pool.view(-1)
    step = 1 << 28
    for o in range(0, flat.numel(), step):
        n = min(step, flat.numel() - o)
        flat[o:o + n].copy_(torch.randn((n,), device=pool.device, generator=gen, dtype=torch.float32).to(pool.dtype))


def kv_torch_dtype(torch, kv: str):
    return {"bf16": torch.bfloat16, "e4m3": torch.float8_e4m3fn}[kv]


def workload_config(wl_name, batch, layers, world, extra=None) -> dict:
    """The `config` object both arms print (same keys, so the two lines can be matched)."""
    cfg = {"workload": wl_name, "global_batch": batch, "layers": layers, "parallelism": f"tp{world}"}
    cfg.update(extra or {})
    return cfg


class StepBench:
    """One decoder of a named workload on this rank with synthetic weights, pools and inputs, and its timings."""

    def __init__(self, torch, workload, K, W, *, dev, rank=0, world=1, group=None, layers=0, kv="bf16"):
        from tlaloc_b200 import _native
        from tlaloc_b200 import decoder as D
        from tlaloc_b200 import sharding

        self.torch, self.dev, self.rank, self.world, self.group, self.K, self.W = torch, dev, rank, world, group, K, W
        cfg_kw, batch, (lo, hi), self.wl_name = WORKLOADS[workload]
        if layers:
            cfg_kw = dict(cfg_kw, num_layers=layers)
        self.cfg_kw, self.batch = cfg_kw, batch
        rng = np.random.default_rng(5)
        self.lens0 = rng.integers(lo, hi + 1, size=batch).astype(np.int64)
        steps_ahead = 2 * (K + W) + 8
        self.max_blocks = (hi + steps_ahead + BS - 1) // BS + 1
        self.kv, self.kv_bytes = kv, (2 if kv == "bf16" else 1)
        cfg = self.cfg = D.DecoderConfig(**cfg_kw, kv_dtype=kv_torch_dtype(torch, kv), head_quant=True, max_positions=self.max_blocks * BS)
        # Size the KV pool: all logical blocks when they fit beside the weights, else what the memory budget allows
        # (then block tables alias physical blocks across sequences; logical bytes are what the step reads).
        self.hk = cfg.num_kv_heads // world
        block_bytes = 2 * BS * self.hk * cfg.head_dim * self.kv_bytes * cfg.num_layers  # K and V, all layers
        self.logical_blocks = int(np.sum((self.lens0 + BS - 1) // BS)) + batch * 4 + 64
        free, total = torch.cuda.mem_get_info(dev)
        per_layer_w = cfg.d_model * (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim + cfg.num_heads * cfg.head_dim * cfg.d_model \
            + 3 * cfg.d_model * cfg.ffn
        weight_bytes = (per_layer_w * cfg.num_layers + cfg.vocab * cfg.d_model) // world + 2 * cfg.vocab * cfg.d_model
        budget = min(free - weight_bytes - (12 << 30), int(0.42 * total))
        self.num_blocks = int(min(self.logical_blocks, budget // block_bytes))
        self.aliased = self.num_blocks < self.logical_blocks
        self.tables = make_tables(rng, batch, self.lens0, BS, self.num_blocks, self.max_blocks, steps_ahead)
        self.dec = D.Decoder(cfg, batch, self.num_blocks, self.max_blocks, device=dev, rank=rank, world=world, group=group)
        self.dec.init_random_weights(seed=0)
        self.gen = torch.Generator(device=dev)
        self.gen.manual_seed(100 + rank)
        for l in range(cfg.num_layers):  # random K/V, N(0,1)
            fill_normal_bf16(torch, self.dec.key_pools[l], self.gen)
            fill_normal_bf16(torch, self.dec.value_pools[l], self.gen)
        self.rng_ids = [np.random.default_rng(7 + i).integers(0, cfg.vocab, size=batch).astype(np.int32) for i in range(8)]
        self.pinned = [torch.empty(s, dtype=torch.int32).pin_memory()
                       for s in ((batch,), (batch,), (batch, self.max_blocks), (batch,), (batch,))]
        self._sharding, self._native = sharding, _native
        self.dec.set_inputs(*self.stage(0))
        torch.cuda.synchronize(dev)
        if world > 1:  # the ranks enter their first exchange together (its waits are bounded)
            torch.distributed.barrier(group=group)
        before = _native.lib().tlaloc_b200_launch_count()
        self.dec.capture()
        self.launches_per_step = (_native.lib().tlaloc_b200_launch_count() - before) // 2  # one eager warm-up + one captured

    def host_inputs(self, step_no: int):
        pos = self.lens0 + step_no
        return (self.rng_ids[step_no % len(self.rng_ids)], pos.astype(np.int32), self.tables, (pos + 1).astype(np.int32),
                self._sharding.slot_mapping(self.tables, pos, BS))

    def stage(self, step_no: int):
        torch = self.torch
        for dst, src in zip(self.pinned, self.host_inputs(step_no)):
            dst.copy_(torch.from_numpy(np.ascontiguousarray(src, dtype=np.int32)))
        return self.pinned

    def barrier(self):
        if self.world > 1:
            self.torch.distributed.barrier(group=self.group)
        self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, ms: float) -> float:
        if self.world == 1:
            return ms
        torch = self.torch
        t = torch.tensor([ms], dtype=torch.float64, device=self.dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=self.group)
        return float(t.item())

    def time_value(self, local_gpu: int):
        """K graph replays, inputs resident: (tokens/s, ms per step, clock summary)."""
        torch, dec, K = self.torch, self.dec, self.K
        for _ in range(self.W):
            dec.step()
        self.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_gpu) as clocks:
            a.record()
            for _ in range(K):
                dec.step()
            b.record()
            self.barrier()
        ms_total = self.max_over_ranks(a.elapsed_time(b))
        return self.batch * K / (ms_total / 1e3), ms_total / K, clocks.summary()

    def time_with_bf16_projections(self, local_gpu: int) -> dict:
        """The same K replays with the layers' projections on the bf16 form of the tensor-core kernel (f32
        accumulation of exact bf16 products) instead of the int8 form; the step graph is captured again for it and
        once more afterwards."""
        dec = self.dec
        if not dec.i8_mma:
            return {"note": "this batch size does not use the int8 form"}
        planes = dec.norm_planes
        dec.i8_mma, dec.norm_planes = False, False
        dec.capture()
        value, ms_step, _ = self.time_value(local_gpu)
        dec.i8_mma, dec.norm_planes = True, planes
        dec.capture()
        return {"value": value, "unit": UNIT, "ms_per_step": ms_step}

    def int8_form_check(self) -> dict:
        """What the int8 form of the projection does to this step's own numbers: layer 0's q|k|v, o and down
        projections on the activations the step left behind, in both forms, against a double-precision product."""
        from tlaloc_b200 import ops

        torch, dec = self.torch, self.dec
        lw = dec.layers[0]
        B = self.batch
        rows = {}
        for name, x in (("qkv", dec.hn), ("o", dec.att.view(B, -1)), ("down", dec.act)):
            codes, scales = lw[name]
            ref = torch.empty((B, codes.shape[1]), dtype=torch.float64, device=self.dev)
            xd = x.double()
            for c0 in range(0, codes.shape[1], 4096):  # column blocks keep the double copy of the codes small
                ref[:, c0:c0 + 4096] = (xd @ codes[:, c0:c0 + 4096].double()) * scales[c0:c0 + 4096].double()
            rms = float(ref.pow(2).mean().sqrt())
            out = {"output_rms": rms}
            for form, flag in (("int8", True), ("bf16", False)):
                y = ops.int8_gemm(x, codes, scales, i8_mma=flag).double()
                err = (y - ref).abs()
                out[form] = {"rms_err_over_output_rms": float(err.pow(2).mean().sqrt()) / max(rms, 1e-30), "max_abs_err": float(err.max()),
                             "beyond_rel_1e-2_abs_2e-3": int((err > 2e-3 + 1e-2 * ref.abs()).sum())}
            rows[name] = out
        return {"rows": rows, "what": "layer 0 projections of this step, each form against an f64 product of the same bf16 "
                                      "activations and int8 codes; the int8 form carries a row as 16-bit fixed point"}

    def time_e2e(self) -> dict:
        """Host buffers in, next tokens out, every step."""
        torch, dec, K, W = self.torch, self.dec, self.K, self.W
        out_host = torch.empty((self.batch,), dtype=torch.int32).pin_memory()
        for s in range(W):
            dec.set_inputs(*self.stage(s))
            out_host.copy_(dec.step(), non_blocking=True)
        self.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for s in range(K):
            dec.set_inputs(*self.stage(W + s))
            out_host.copy_(dec.step(), non_blocking=True)
            torch.cuda.current_stream(self.dev).synchronize()  # the caller reads the tokens before building the next step
        b.record()
        self.barrier()
        e2e_ms = self.max_over_ranks(a.elapsed_time(b))
        h2d = int(sum(p.numel() * 4 for p in self.pinned))
        return {"value": self.batch * K / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": self.batch * 4}

    def attention_roofline(self, pk) -> dict:
        """Paged attention (slice + combine) timed alone with CUDA events.  Timed on a pool of its own in which no two
        sequences share a block (one layer's worth, a few GB, far larger than L2), so the bytes it is credited with are
        bytes that come from HBM; the same launches over the step's own pools (which alias blocks when the logical KV
        does not fit the GPU) are reported beside it."""
        from tlaloc_b200 import ops

        torch, dec, cfg, dev, batch, hk = self.torch, self.dec, self.cfg, self.dev, self.batch, self.hk
        lens_now = (self.lens0 + 1).astype(np.int64)
        att_bytes = 2 * int(lens_now.sum()) * hk * cfg.head_dim * self.kv_bytes + 2 * batch * (cfg.num_heads // self.world) * cfg.head_dim * 3
        reps = 20
        dec.set_inputs(*self.stage(0))
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

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
        need = np.asarray((lens_now + BS - 1) // BS, np.int64)
        own_blocks = int(need.sum()) + 1
        perm = 1 + np.random.default_rng(11).permutation(own_blocks - 1)
        own_tables = np.zeros((batch, self.max_blocks), np.int32)
        o = 0
        for i in range(batch):
            own_tables[i, :need[i]] = perm[o:o + need[i]]
            o += int(need[i])
        roof_k = torch.empty((own_blocks, BS, hk, cfg.head_dim), dtype=cfg.kv_dtype, device=dev)
        roof_v = torch.empty_like(roof_k)
        fill_normal_bf16(torch, roof_k, self.gen)
        fill_normal_bf16(torch, roof_v, self.gen)
        att_ms = time_attention([roof_k], [roof_v], torch.from_numpy(own_tables).to(dev))
        del roof_k, roof_v
        achieved = att_bytes / (att_ms / 1e3) / 1e9
        traffic = None
        try:
            with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
                per_pos = json.load(f).get("paged_attention_dram_bytes_per_position_per_kv_head")
                if per_pos and self.kv == "bf16":
                    traffic = float(per_pos) * int(lens_now.sum()) * hk
        except Exception:
            pass
        return {"kernel": ("PaSliceTma" if self.kv == "bf16" else "PaSliceTmaF8") + "+PaCombine", "bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "traffic": traffic, "peak_kind": pk["kind"], "bytes_per_launch": att_bytes,
                "ms_per_launch": att_ms, "pool": "one block per (sequence, 16 positions): nothing shared",
                "in_step_pools": {"ms_per_launch": in_step_ms, "logical_gbs": att_bytes / (in_step_ms / 1e3) / 1e9,
                                  "aliased": bool(self.aliased)}}

    def projection_roofline(self, pk) -> dict:
        """The step's four int8 projections at the step's batch, each timed alone with CUDA events over the layers' own
        weights (every launch streams a different layer's weights: far more than L2 in total).  floor = the slower of
        algorithmic bytes / measured HBM rate and flops / measured sustained bf16 rate."""
        from tlaloc_b200 import ops

        torch, dec, dev, B = self.torch, self.dec, self.dev, self.batch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        L = len(dec.layers)
        hq, hd = dec.hq, self.cfg.head_dim
        how = dict(weights_const=True, scratch=dec.proj_scratch, i8_mma=dec.i8_mma)  # as the step launches them
        xp = bool(dec.norm_planes)  # q|k|v and gate|up find their input's planes already written by the RMSNorm kernel
        calls = {
            "qkv": lambda lw: ops.int8_gemm(dec.hn, *lw["qkv"], out=dec.qkv, x_planes=xp, **how),
            "o": lambda lw: ops.int8_gemm(dec.att.view(B, hq * hd), *lw["o"], residual=dec.h, out=dec.h2, **how),
            "gate_up": lambda lw: dec.gate_up_proj(lw, x_planes=xp),
            "down": lambda lw: ops.int8_gemm(dec.act, *lw["down"], residual=dec.h2, out=dec.h, **how),
        }
        rows, t_sum, f_sum = [], 0.0, 0.0
        for name, fn in calls.items():
            k, n = dec.layers[0][name][0].shape
            for l in range(min(3, L)):
                fn(dec.layers[l])
            torch.cuda.synchronize(dev)
            a.record()
            for l in range(L):
                fn(dec.layers[l])
            b.record()
            torch.cuda.synchronize(dev)
            us = a.elapsed_time(b) / L * 1e3
            out_bytes = 2 * B * (n // 2) if (name == "gate_up" and dec.fuse_swiglu) else 4 * B * n  # SwiGLU folded in: bf16 [B, F]
            byts = k * n + 4 * n + 2 * B * k + out_bytes
            flops = 2.0 * B * k * n
            floor_us = max(byts / pk["hbm_gbs"] / 1e3, flops / pk["bf16_tflops_sustained"] / 1e6)
            rows.append({"proj": name, "K": int(k), "N": int(n), "M": B, "us": us, "gbs": byts / us / 1e3,
                         "tflops": flops / us / 1e6, "floor_us": floor_us, "frac_of_floor": floor_us / us})
            t_sum += us
            f_sum += floor_us
        kernel = "QuantizeRowsI8Kernel + Int8GemmI8Kernel" if dec.i8_mma else "Int8GemmTcKernel" if B >= 17 else "Int8GemvKernel"
        return {"kernel": kernel, "bound": "hbm | tensor (the slower floor)",
                "rows": rows, "us_per_layer": t_sum, "floor_us_per_layer": f_sum, "frac": f_sum / t_sum,
                "peak_kind": pk["kind"], "hbm_gbs": pk["hbm_gbs"], "bf16_tflops_sustained": pk["bf16_tflops_sustained"]}

    def timeline(self) -> dict:
        """Durations per kernel inside ONE graph replay of the step (CUPTI kernel records through torch.profiler)."""
        import collections

        from torch.profiler import ProfilerActivity, profile

        torch, dec = self.torch, self.dec
        for _ in range(3):
            dec.step()
        torch.cuda.synchronize(self.dev)
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            dec.step()
            torch.cuda.synchronize(self.dev)
        ks = sorted((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                    if e.device_type == torch.autograd.DeviceType.CUDA and e.time_range is not None
                    and "Memcpy" not in e.name and "Memset" not in e.name)
        # Kernels of one step overlap (a kernel launched with programmatic serialization starts while its predecessor
        # drains and waits inside), so a record's own duration counts that wait.  "exclusive" time is what the kernel adds
        # to the step: from the later of its start and the previous kernel's end, to its own end.
        tot = collections.defaultdict(lambda: [0, 0.0, 0.0])
        prev_end = None
        n_proj = 0
        for (s, e, name) in ks:
            key = name.split("<")[0].split("::")[-1][:48]
            if key in ("Int8GemmTcKernel", "Int8GemvKernel"):  # a layer launches them in this order; the head comes last
                key += ":" + (("qkv", "o", "gate_up", "down")[n_proj % 4] if n_proj < 4 * dec.cfg.num_layers else "head")
                n_proj += 1
            tot[key][0] += 1
            tot[key][1] += e - s
            tot[key][2] += max(0.0, e - (s if prev_end is None else max(s, prev_end)))
            prev_end = e if prev_end is None else max(prev_end, e)
        span = (ks[-1][1] - ks[0][0]) if ks else 0.0
        excl = sum(v[2] for v in tot.values())
        return {"step_span_ms": span / 1e3, "sum_of_exclusive_ms": excl / 1e3,
                "kernels": [{"name": k, "launches": v[0], "exclusive_ms": v[2] / 1e3, "exclusive_us_each": v[2] / v[0],
                             "share": v[2] / max(excl, 1e-9), "duration_us_each": v[1] / v[0]}
                            for k, v in sorted(tot.items(), key=lambda kv: -kv[1][2])]}

    def close(self):
        self.dec = None
        gc.collect()
        self.torch.cuda.empty_cache()


def tp_parity(torch, dev, rank, world, group) -> dict:
    """The tensor-parallel path checked on the N ranks of this run, before anything is timed:
    (1) the sum over ranks on a [128, 8192] f32 buffer (the step's own shape), bit for bit against the f32 sum in rank
        order, plain and with the RMSNorm folded in (normalised rows within one bf16 step of the norm of those sums);
    (2) two decode steps of a small decoder that shards `world` ways (2 layers, d 512, 8 Q / 8 KV heads of 64, FFN
        1024, vocab 2048) against the CPU oracle's unsharded step: logits within rel 1e-2 / abs 2e-3, greedy tokens equal."""
    import oracle
    from tlaloc_b200 import decoder as D
    from tlaloc_b200 import sharding
    from tlaloc_b200.peer import PeerBuffers

    shape = (128, 8192)

    def rank_input(q, round_):
        r = np.random.default_rng(1000 * round_ + q)
        return (r.standard_normal(shape) * 10.0 ** r.integers(-2, 3)).astype(np.float32)

    def expected(round_):
        acc = rank_input(0, round_)
        for q in range(1, world):
            acc = acc + rank_input(q, round_)  # f32 adds in rank order, as the kernel adds
        return acc

    peer = PeerBuffers([shape], rank=rank, world=world, group=group, device=dev, norm_shape=shape)
    sum_exact, norm_ok = True, True
    for round_ in (1, 2):
        peer.tensors[0].copy_(torch.from_numpy(rank_input(rank, round_)))
        out = peer.all_reduce_(0)
        sum_exact &= bool(np.array_equal(out.cpu().numpy(), expected(round_)))
    if peer.can_fuse_norm(0):
        gain = torch.from_numpy(np.random.default_rng(77).uniform(0.5, 1.5, size=shape[1]).astype(np.float32)).to(dev)
        peer.tensors[0].copy_(torch.from_numpy(rank_input(rank, 3)))
        out, normed = peer.all_reduce_norm_(0, gain, 1e-5)
        want = expected(3)
        sum_exact &= bool(np.array_equal(out.cpu().numpy(), want))
        w64 = want.astype(np.float64)
        ref = w64 / np.sqrt((w64 * w64).mean(axis=1, keepdims=True) + 1e-5) * gain.cpu().numpy().astype(np.float64)[None, :]
        norm_ok = bool(np.all(np.abs(normed.float().cpu().numpy() - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-6))
    if peer.can_sum_rows(0):  # the one-barrier form the decode step uses: residual + partials in rank order, kept locally
        res_h = rank_input(99, 4)
        peer.tensors[0].copy_(torch.from_numpy(rank_input(rank, 4)))
        res = torch.from_numpy(res_h).to(dev)
        out = torch.empty(shape, dtype=torch.float32, device=dev)
        normed = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        gain = torch.from_numpy(np.random.default_rng(77).uniform(0.5, 1.5, size=shape[1]).astype(np.float32)).to(dev)
        peer.sum_rows_(0, res, out, gain, 1e-5, norm_out=normed)
        want = res_h + rank_input(0, 4)
        for q in range(1, world):
            want = want + rank_input(q, 4)
        sum_exact &= bool(np.array_equal(out.cpu().numpy(), want))
        w64 = want.astype(np.float64)
        ref = w64 / np.sqrt((w64 * w64).mean(axis=1, keepdims=True) + 1e-5) * gain.cpu().numpy().astype(np.float64)[None, :]
        norm_ok &= bool(np.all(np.abs(normed.float().cpu().numpy() - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-6))
        torch.distributed.barrier(group=group)  # every rank has read every partial before the buffers go away
    status = peer.status()
    peer.close()

    small = dict(num_layers=2, d_model=512, num_heads=8, num_kv_heads=8, head_dim=64, ffn=1024, vocab=2048)
    oshape = oracle.DecoderShape(**small, kv_dtype="bf16", head_quant=True)
    w = oracle.make_weights(oshape, seed=3)
    cfg = D.DecoderConfig(**small, kv_dtype=torch.bfloat16, head_quant=True, max_positions=64)
    B, M = 8, 3
    rng = np.random.default_rng(9)
    tables = (1 + rng.permutation(B * M)).reshape(B, M).astype(np.int32)
    dec = D.Decoder(cfg, B, 1 + B * M, M, device=dev, rank=rank, world=world, group=group)
    dec.load_host_weights(w)
    kp = [np.zeros((1 + B * M, BS, 8, 64), np.float32) for _ in range(2)]
    vp = [np.zeros_like(a) for a in kp]
    ids = rng.integers(0, 2048, size=B).astype(np.int32)
    vp_rank = small["vocab"] // world
    max_err, tokens_equal, logits_ok = 0.0, True, True
    for step in range(2):
        pos = np.full(B, step, np.int32)
        slots = sharding.slot_mapping(tables, pos, BS)
        dec.set_inputs(ids, pos, tables, pos + 1, slots)
        nxt = dec.step().cpu().numpy()
        want = oracle.decode_step(oshape, w, kp, vp, ids, pos, tables, pos + 1, slots)
        err = np.abs(dec.logits.cpu().numpy() - want[:, rank * vp_rank:(rank + 1) * vp_rank])
        logits_ok &= bool(np.all(err <= 2e-3 + 1e-2 * np.abs(want).max(axis=1, keepdims=True)))
        max_err = max(max_err, float(err.max()))
        ids = oracle.argmax(want).astype(np.int32)
        tokens_equal &= bool(np.array_equal(nxt, ids))
    status = status or dec.exchange_status()
    flags = torch.tensor([float(sum_exact), float(norm_ok), float(logits_ok), float(tokens_equal), -max_err, -float(status)],
                         dtype=torch.float64, device=dev)
    torch.distributed.all_reduce(flags, op=torch.distributed.ReduceOp.MIN, group=group)
    f = flags.cpu().tolist()
    dec = None
    gc.collect()
    torch.cuda.empty_cache()
    return {"n": world, "sum_exact": bool(f[0]), "norm_within_one_bf16_step": bool(f[1]), "logits_within_tolerance": bool(f[2]),
            "tokens_equal": bool(f[3]), "max_logit_err": -f[4], "exchange_status": int(-f[5]),
            "checked": "peer-memory sum [128, 8192] f32 on all ranks, bit for bit; 2 decode steps of a 2-layer d512 8Q/8KV "
                       "decoder against the CPU oracle (rel 1e-2 / abs 2e-3)"}


def run_ours(args) -> dict:
    import torch

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
    parity = None
    if world > 1:
        # NCCL carries only the handle exchange, barriers and the per-step gather of (best logit, id) pairs; the sums
        # over ranks are the library's own peer-memory kernels, so NCCL's NVLink multicast buffers are not set up
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.distributed.init_process_group("nccl", device_id=dev)
        group = torch.distributed.group.WORLD
        parity = tp_parity(torch, dev, rank, world, group)
        ok = parity["sum_exact"] and parity["norm_within_one_bf16_step"] and parity["logits_within_tolerance"] \
            and parity["tokens_equal"] and parity["exchange_status"] == 0
        if not ok:
            if rank == 0:
                print(json.dumps({"tp_parity": parity, "error": "tensor-parallel parity check failed"}), flush=True)
            torch.cuda.synchronize(dev)
            os._exit(3)

    pk = peaks()
    sb = StepBench(torch, args.workload, args.steps, args.warmup, dev=dev, rank=rank, world=world, group=group, layers=args.layers,
                   kv=args.kv)
    cfg, batch, dec = sb.cfg, sb.batch, sb.dec
    if args.timeline:
        return {"timeline": sb.timeline(), "config": workload_config(sb.wl_name, batch, cfg.num_layers, world)}
    value, ms_step, clocks = sb.time_value(local)
    e2e = sb.time_e2e()
    roofline = sb.attention_roofline(pk)
    lens_now = (sb.lens0 + 1).astype(np.int64)
    stb = dec.step_bytes(lens_now)
    step_gbs = (stb["weights"] + stb["kv"]) / (ms_step / 1e3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": (f"int8 weights x bf16 activations ({'rows as 16-bit fixed point on the int8 tensor-core form, int32 accumulate' if dec.i8_mma else 'f32 accumulate'}"
                  f"; head and attention f32 accumulate); {'bf16' if args.kv == 'bf16' else 'f8e4m3fn'} KV"), "data": "synthetic",
        "config": workload_config(sb.wl_name, batch, cfg.num_layers, world, {
            "mean_context": float(lens_now.mean()), "kv_blocks_per_layer": sb.num_blocks,
            "kv_blocks_logical": sb.logical_blocks, "kv_aliased": bool(sb.aliased),
            "l2": "inputs larger than L2 (weights and KV pools are tens of GB)", "head": "int8 (headQuant)", "kv": args.kv}),
        "e2e": e2e, "gpu_launches": int(sb.launches_per_step * args.steps), "launches_per_step": int(sb.launches_per_step),
        "clocks": clocks, "roofline": roofline,
        "step_hbm": {"weights_bytes": stb["weights"], "kv_bytes": stb["kv"], "achieved_gbs": step_gbs, "frac": step_gbs / pk["hbm_gbs"]},
    }
    if world > 1:
        line["config"]["rank_sum"] = ("peer-memory kernel, one barrier (every rank sums all partials)" if dec.one_shot
                                      else "peer-memory kernel, residual stream distributed by rows (reduce-scatter of the partials, "
                                           + ("all-gather of the normalised rows as the next projection's int8 planes)"
                                              if getattr(dec, "rows_planes", False) else "all-gather of the bf16 normalised rows)")
                                      if getattr(dec, "rows_residual", False)
                                      else "peer-memory kernel, reduce-scatter + all-gather" if dec.peer is not None else "nccl")
        line["exchange_status"] = dec.exchange_status()  # 0: no bounded wait of the exchange kernel ever gave up
        line["tp_parity"] = parity
    if world == 1 and not args.lean:
        line["roofline_projection"] = sb.projection_roofline(pk)
        line["int8_form_check"] = sb.int8_form_check()
        line["with_bf16_projections"] = sb.time_with_bf16_projections(local)
    if world > 1:
        # Print first, then leave without tearing the communicator down: destroying a process group whose
        # collectives live inside a CUDA graph blocks, and the process is about to exit anyway.
        if rank == 0:
            print(json.dumps(line), flush=True)
        torch.cuda.synchronize(dev)
        torch.distributed.barrier(group=group)
        sys.stdout.flush()
        os._exit(0)
    sb.close()
    del sb, dec
    if not args.lean and args.workload == "llama70b":
        line["operators"] = {"paged_attention": operator_paged_attention(torch, dev, pk, reps=20),
                             "paged_attention_e4m3_kv": operator_paged_attention(torch, dev, pk, reps=20, kv="e4m3"),
                             "int8_projection": operator_int8_projection(torch, dev, pk, only="")}
        line["llama8b"] = llama8b_block(torch, dev, local, pk)
    if rank == 0 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(WORKLOADS[args.workload][0] if not args.layers else dict(WORKLOADS[args.workload][0], num_layers=args.layers),
                                            batch, lens_now, seconds=args.cpu_seconds)
    return line


def llama8b_block(torch, dev, local, pk) -> dict:
    """The 8B-shape configuration (batch 64, contexts U[128, 4096]): fits one GPU with every KV page its own."""
    sb = StepBench(torch, "llama8b", 10, 3, dev=dev)
    value, ms_step, clocks = sb.time_value(local)
    e2e = sb.time_e2e()
    lens_now = (sb.lens0 + 1).astype(np.int64)
    stb = sb.dec.step_bytes(lens_now)
    gbs = (stb["weights"] + stb["kv"]) / (ms_step / 1e3) / 1e9
    out = {"workload": sb.wl_name, "value": value, "unit": UNIT, "ms_per_step": ms_step, "steps": 10, "warmup": 3,
           "e2e": e2e["value"], "kv_aliased": bool(sb.aliased), "launches_per_step": int(sb.launches_per_step),
           "step_hbm": {"weights_bytes": stb["weights"], "kv_bytes": stb["kv"], "achieved_gbs": gbs, "frac": gbs / pk["hbm_gbs"]},
           "clocks": clocks}
    sb.close()
    return out


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


def operator_paged_attention(torch, dev, pk, reps=20, kv="bf16") -> dict:
    """The paged-attention decode operator alone: bf16 Q [32, 32, 128], 8 KV heads, block 16, 4096 physical blocks,
    permuted tables, lengths U[512, 8192], seed 1; as configured (tables alias blocks: 8704 logical > 4096 physical)
    and with a block of its own for every (sequence, 16 positions).  HBM GB/s on algorithmic bytes."""
    from tlaloc_b200 import ops
    from tlaloc_b200.attrs import parse_paged_attention

    rng = np.random.default_rng(1)
    B, H, Hkv, D, nb, width = 32, 32, 8, 128, 4096, 512
    lens = rng.integers(512, 8193, size=B).astype(np.int32)
    kvb = 2 if kv == "bf16" else 1
    logical = 2 * int(lens.sum()) * Hkv * D * kvb + 2 * B * H * D * 2
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    out = {}
    for name in ("as_configured", "no_shared_blocks"):
        if name == "as_configured":
            P = nb
            tab = np.stack([rng.permutation(nb)[:width] for _ in range(B)]).astype(np.int32)
        else:
            need = (lens + BS - 1) // BS
            P = int(need.sum()) + 1
            perm = 1 + rng.permutation(P - 1)
            tab = np.zeros((B, width), np.int32)
            o = 0
            for i in range(B):
                tab[i, :need[i]] = perm[o:o + need[i]]
                o += int(need[i])
        k = torch.randn((P, BS, Hkv, D), device=dev, generator=g).to(kv_torch_dtype(torch, kv))
        v = torch.randn((P, BS, Hkv, D), device=dev, generator=g).to(kv_torch_dtype(torch, kv))
        q = torch.randn((B, H, D), device=dev, generator=g).to(torch.bfloat16)
        tt, tl = torch.from_numpy(tab).to(dev), torch.from_numpy(lens).to(dev)
        o_t = torch.empty((B, H, D), dtype=torch.bfloat16, device=dev)
        scratch = ops.paged_attention_scratch(parse_paged_attention(q, k, v, tt, tl, scale=D ** -0.5), dev)
        best, med = _time_graph(torch, lambda: ops.paged_attention(q, k, v, tt, tl, scale=D ** -0.5, out=o_t, scratch=scratch), reps)
        out[name] = {"us": med * 1e3, "gbs": logical / med / 1e6, "best_gbs": logical / best / 1e6, "physical_blocks": P,
                     "frac": logical / med / 1e6 / pk["hbm_gbs"]}
        del k, v
    out["algorithmic_bytes"] = logical
    out["kv"] = kv
    return out


def operator_int8_projection(torch, dev, pk, only="") -> dict:
    """The int8 projection sweep: N x K in {4096x4096, 14336x4096, 4096x14336, 128256x4096}, M in {1, 8, 32, 128, 256};
    M <= 128 against the HBM rate, M = 256 (a dense contraction) against the measured bf16 burst rate."""
    from tlaloc_b200 import ops

    rows = []
    shapes, ms = [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)], (1, 8, 32, 128, 256)
    forms = {32: ("bf16", "int8"), 128: ("bf16", "int8")}  # the tensor-core kernel's two forms where both apply
    if only:  # one shape "NxKxM" or "NxKxMxi8", for profiler captures
        parts = only.lower().split("x")
        n, k, m = (int(v) for v in parts[:3])
        shapes, ms = [(n, k)], (m,)
        forms = {m: ("int8",) if parts[3:] == ["i8"] else ("bf16",)}
    for (n, k) in shapes:
        nbuf = max(4, int(400e6 // (k * n)) + 1)  # distinct weight buffers, > 3x L2 in total, visited round robin
        ws = [torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev) for _ in range(nbuf)]
        sc = torch.rand((n,), device=dev) * 0.019 + 0.001
        for m in ms:
            x = torch.randn((m, k), device=dev).to(torch.bfloat16)
            y = torch.empty((m, n), dtype=torch.float32, device=dev)
            scr = torch.empty((ops.int8_gemm_scratch_bytes(m, k, n) + 3) // 4, dtype=torch.float32, device=dev)
            for form in forms.get(m, ("",)):
                i8 = form == "int8"

                def fn():
                    for w in ws:
                        ops.int8_gemm(x, w, sc, out=y, weights_const=True, scratch=scr, i8_mma=i8)
                best, med = _time_graph(torch, fn, 10)
                byts = k * n + 4 * n + 2 * m * k + 4 * m * n
                us = med / nbuf * 1e3
                row = {"N": n, "K": k, "M": m, "us": us, "gbs": byts / us / 1e3, "tflops": 2.0 * m * n * k / us / 1e6}
                if form:
                    row["tensor_core_form"] = form
                row["frac_hbm"] = row["gbs"] / pk["hbm_gbs"]
                if m >= 256:
                    row["frac_tensor"] = row["tflops"] / pk["bf16_tflops"]
                rows.append(row)
        del ws
    return {"rows": rows, "hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "peak_kind": pk["kind"]}


def run_operator(args) -> dict:
    """The two operators alone (single GPU)."""
    import torch

    dev = torch.device("cuda", 0)
    pk = peaks()
    if args.workload == "paged_attn":
        out = operator_paged_attention(torch, dev, pk, reps=max(args.steps, 20), kv=args.kv)
        head = out["no_shared_blocks"]
        return {"metric": "paged_attention_hbm_gbs", "value": head["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": max(args.steps, 20),
                "warmup": 3, "higher_is_better": True, "data": "synthetic", "dtype": "bf16 KV and Q, f32 accumulate",
                "config": {"workload": "paged-attention decode operator alone", "algorithmic_bytes": out["algorithmic_bytes"], "cases": out},
                "roofline": {"kernel": ("PaSliceTma" if args.kv == "bf16" else "PaSliceTmaF8") + "+PaCombine", "bound": "hbm", "achieved": head["gbs"], "peak": pk["hbm_gbs"],
                             "unit": "GB/s", "frac": head["gbs"] / pk["hbm_gbs"], "peak_kind": pk["kind"], "traffic": None}}
    out = operator_int8_projection(torch, dev, pk, only=args.only)
    rows = out["rows"]
    big = ([r for r in rows if r["N"] == 128256 and r["M"] == 8] or rows)[0]
    return {"metric": "int8_projection_hbm_gbs", "value": big["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": 10, "warmup": 3,
            "higher_is_better": True, "data": "synthetic", "dtype": "int8 weights x bf16, f32 accumulate",
            "config": {"workload": "int8 weight-only projection sweep", "rows": rows},
            "roofline": {"kernel": "Int8GemvKernel", "bound": "hbm", "achieved": big["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": big["gbs"] / pk["hbm_gbs"], "peak_kind": pk["kind"], "traffic": None}}


def run_peer_sum(args) -> dict:
    """The sum over ranks alone (N >= 2): the library's peer-memory kernel, the same with the RMSNorm folded in, and
    NCCL's all-reduce, each captured 50 times into one CUDA graph; microseconds per sum, max over ranks."""
    import torch

    from tlaloc_b200.peer import PeerBuffers

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2 or world != args.gpus:
        raise SystemExit("--workload peer_sum needs torch.distributed.run with --gpus N >= 2 ranks")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # NCCL's all-reduce is timed as plain ring/tree; no multicast buffers
    torch.distributed.init_process_group("nccl", device_id=dev)
    group = torch.distributed.group.WORLD
    shapes = [(128, 8192), (8, 8192), (64, 4096)]
    n = 50
    rows, keep = [], []
    for shp in shapes:
        peer = PeerBuffers([shp], rank=rank, world=world, group=group, device=dev, norm_shape=shp)
        priv = torch.randn(shp, device=dev)
        gain = torch.ones((shp[1],), device=dev)

        def timed(fn):
            s = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(s):
                for _ in range(3):
                    fn()
            torch.cuda.synchronize(dev)
            torch.distributed.barrier(group=group)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(n):
                    fn()
            keep.append(g)
            g.replay()
            torch.cuda.synchronize(dev)
            torch.distributed.barrier(group=group)
            torch.cuda.synchronize(dev)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            g.replay()
            b.record()
            torch.cuda.synchronize(dev)
            t = torch.tensor([a.elapsed_time(b) * 1e3 / (2 * n)], dtype=torch.float64, device=dev)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=group)
            return float(t.item())

        row = {"shape": list(shp), "bytes": 4 * shp[0] * shp[1], "peer_us": timed(lambda: peer.all_reduce_(0))}
        if peer.can_fuse_norm(0):
            row["peer_with_rmsnorm_us"] = timed(lambda: peer.all_reduce_norm_(0, gain, 1e-5))
            own = torch.zeros((shp[0] // world, shp[1]), device=dev)
            row["rows_residual_with_rmsnorm_us"] = timed(lambda: peer.reduce_norm_rows_(0, own, gain, 1e-5))
            row["rows_residual_with_rmsnorm_planes_us"] = timed(lambda: peer.reduce_norm_rows_(0, own, gain, 1e-5, planes=True))
        if peer.can_sum_rows(0):
            two = PeerBuffers([shp, shp], rank=rank, world=world, group=group, device=dev)
            hbuf = torch.zeros(shp, device=dev)
            hn = torch.empty(shp, device=dev, dtype=torch.bfloat16)
            turn = [0]

            def one_barrier():
                two.sum_rows_(turn[0] & 1, hbuf, hbuf, gain, 1e-5, norm_out=hn)
                turn[0] += 1
            row["one_barrier_with_residual_and_rmsnorm_us"] = timed(one_barrier)
            row["exchange_status_one_barrier"] = two.status()
        row["nccl_us"] = timed(lambda: torch.distributed.all_reduce(priv, group=group))
        row["exchange_status"] = peer.status()
        rows.append(row)
    line = {"metric": "tensor_parallel_sum_us", "value": rows[0]["peer_us"], "unit": "us", "n_gpus": world, "steps": 2 * n, "warmup": 3,
            "higher_is_better": False, "data": "synthetic", "dtype": "f32",
            "config": {"workload": "sum over ranks of an f32 matrix, in place, peer-memory kernel vs NCCL, 50 per CUDA graph", "rows": rows}}
    if rank == 0:
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize(dev)
    torch.distributed.barrier(group=group)
    sys.stdout.flush()
    os._exit(0)


def cpu_sample(cfg_kw, lens, b_sample, threads):
    """One layer of the decode step for `b_sample` sequences through the CPU restatement: the int8 projections and the
    paged attention (the two hot ops), all host threads.  Returns seconds."""
    import oracle

    d, H, Hkv, hd, ffn = cfg_kw["d_model"], cfg_kw["num_heads"], cfg_kw["num_kv_heads"], cfg_kw["head_dim"], cfg_kw["ffn"]
    rng = np.random.default_rng(0)
    lens = np.asarray(lens[:b_sample], np.int32)
    nblk = int(np.sum((lens + BS - 1) // BS)) + 1
    kbits = rng.integers(0, 1 << 16, size=(nblk, BS, Hkv, hd), dtype=np.uint16) & np.uint16(0xBFFF)
    vbits = rng.integers(0, 1 << 16, size=(nblk, BS, Hkv, hd), dtype=np.uint16) & np.uint16(0xBFFF)
    tab = np.zeros((b_sample, int(lens.max() + BS - 1) // BS), np.int32)
    o = 1
    for i in range(b_sample):
        n = (lens[i] + BS - 1) // BS
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
    threads = host_cores()
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
    so this arm times the C restatement of that interpreter (oracle/) on all the host threads this process may use.
    A timed step is a bounded SAMPLE of one decode step: one of the step's layers for 16 of its sequences; `value`
    is the sample's share of a step's tokens (16 / layers) over the sample's time, `ms_per_step` the sample's time."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    cfg_kw, batch, (lo, hi), wl_name = WORKLOADS[args.workload]
    if args.layers:
        cfg_kw = dict(cfg_kw, num_layers=args.layers)
    rng = np.random.default_rng(5)
    lens = (rng.integers(lo, hi + 1, size=batch) + 1).astype(np.int64)
    threads = host_cores()
    b = min(16, batch)
    times = []
    for i in range(args.warmup + args.steps):
        t = cpu_sample(cfg_kw, lens, b, threads)
        if i >= args.warmup:
            times.append(t)
    t = float(np.mean(times))
    tokens_per_sample = b / cfg_kw["num_layers"]  # b sequences through 1 of L layers = b / L of a token each... summed
    value = tokens_per_sample / t
    sample = (f"each timed step is a SAMPLE of one decode step: one of {cfg_kw['num_layers']} layers (int8 projections + paged "
              f"attention) for {b} of {batch} sequences = {tokens_per_sample:.3f} tokens' worth of work in {t:.2f} s on {threads} "
              f"threads; a whole step would take {t * cfg_kw['num_layers'] * batch / b:.0f} s (scaled x layers x batch/{b})")
    return {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3, "tokens_per_timed_step": tokens_per_sample,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 accumulate on the host (f64 in the attention walk)", "data": "synthetic",
            "config": workload_config(wl_name, batch, cfg_kw["num_layers"], args.gpus,
                                      {"sampled": f"1 layer x {b} sequences per timed step, scaled x layers x batch/{b}",
                                       "runs_on": f"{threads} host threads"}),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama70b", choices=sorted(WORKLOADS) + ["paged_attn", "int8_proj", "peer_sum"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only; not a bench value)")
    ap.add_argument("--only", default="", help="int8_proj: a single shape NxKxM")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--lean", action="store_true", help="skip the projection roofline, the operator sweeps and the 8B-shape block")
    ap.add_argument("--timeline", action="store_true", help="per-kernel durations inside one graph replay of the step")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "e4m3"],
                    help="KV pool dtype: bf16 (the benchmark configuration) or e4m3 (f8e4m3fn pools, half the bytes; reported beside it)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        line = run_reference(args)
    elif args.workload in ("paged_attn", "int8_proj"):
        line = run_operator(args)
    elif args.workload == "peer_sum":
        line = run_peer_sum(args)
    else:
        line = run_ours(args)
    if line:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
