"""The Llama-style decode step on one B200, or tensor-parallel over the B200s of one box.

What the step computes is the reference's decode graph (ir/.../inference/HfDecoderGraph.kt: embed :904-909;
per layer rmsNorm :663-699 -> q/k/v proj :1183-1213 -> rope :792-818 -> KV_CACHE_WRITE x2 :1230-1231 ->
PAGED_ATTENTION :1233-1253 -> o proj + residual :1266-1273 -> rmsNorm -> SiLU(gate)*up :979-988 -> down proj +
residual :1002-1009; then the final norm and head :2121-2128; greedy next token = first maximum).  Every
operator is one call through the C ABI of libtlaloc_kernels.so; PyTorch only owns device memory, the stream, the
CUDA graph and (for tensor parallelism) the NCCL communicator.  There is no CPU path.

Per layer the step launches: rmsnorm, fused q|k|v projection, rope + KV write, attention slice + combine,
o projection (+ residual), rmsnorm, fused gate|up projection, swiglu, down projection (+ residual); with
tensor parallelism a sum over the ranks follows the o and down projections: one kernel per rank that reduce-scatters
by peer loads and all-gathers by peer stores over NVLink (peer.py, csrc/peer_allreduce.cu).  The whole step is
captured once into a CUDA graph and replayed.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np
import torch

from . import ops, sharding
from .peer import PeerBuffers


@dataclass
class DecoderConfig:
    num_layers: int
    d_model: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    block_size: int = 16
    kv_dtype: torch.dtype = torch.bfloat16
    head_quant: bool = True
    max_positions: int = 8192

    @property
    def scale(self) -> float:
        # HfDecoderGraph.kt:546: 1f / sqrt(hd.toFloat()), widened
        return float(np.float32(1.0) / np.sqrt(np.float32(self.head_dim)))


LLAMA3_8B = dict(num_layers=32, d_model=4096, num_heads=32, num_kv_heads=8, head_dim=128, ffn=14336, vocab=128256)
LLAMA3_70B = dict(num_layers=80, d_model=8192, num_heads=64, num_kv_heads=8, head_dim=128, ffn=28672, vocab=128256)
TINY = dict(num_layers=2, d_model=256, num_heads=4, num_kv_heads=2, head_dim=64, ffn=688, vocab=1024)


def rope_tables(theta: float, head_dim: int, positions: int):
    """HfDecoderGraph.ropeTables (:436-462): computed in double, narrowed to f32, both halves equal."""
    half = head_dim // 2
    inv = np.power(float(theta), -2.0 * np.arange(half, dtype=np.float64) / head_dim)
    ang = np.arange(positions, dtype=np.float64)[:, None] * inv[None, :]
    cos = np.concatenate([np.cos(ang), np.cos(ang)], axis=1).astype(np.float32)
    sin = np.concatenate([np.sin(ang), np.sin(ang)], axis=1).astype(np.float32)
    return cos, sin


class Decoder:
    """Weights, KV pools and step buffers of one rank; `step()` runs one decode step for `batch` sequences."""

    def __init__(self, cfg: DecoderConfig, batch: int, num_blocks: int, max_blocks_per_seq: int, *, device="cuda:0",
                 rank: int = 0, world: int = 1, group=None, exact: bool = False):
        """`exact`: every operator runs in the library's parity mode (the reference interpreter's own evaluation
        order: order-faithful projections, double-precision attention walk, sequential RMSNorm sums, SiLU in
        double).  Slow; its logits equal the CPU oracle's to the last bits and its greedy tokens are the oracle's."""
        if not torch.cuda.is_available():
            raise RuntimeError("tlaloc_b200.Decoder needs a CUDA device: there is no CPU path")
        sharding.check_world(cfg.num_heads, cfg.num_kv_heads, cfg.ffn, cfg.vocab, world)
        self.cfg, self.batch, self.device, self.rank, self.world, self.group = cfg, batch, torch.device(device), rank, world, group
        self.exact = bool(exact)
        # SwiGLU in the gate|up projection's epilogue: batches the tensor-core kernels take (17 rows and more) and FFN
        # widths that tile in blocks of 128 per rank; $TLALOC_B200_FUSE_SWIGLU=0 keeps the separate kernel
        self.fuse_swiglu = (not exact and batch >= 17 and (cfg.ffn // world) % 128 == 0
                            and os.environ.get("TLALOC_B200_FUSE_SWIGLU", "1") != "0")
        self.hq, self.hk, self.f = cfg.num_heads // world, cfg.num_kv_heads // world, cfg.ffn // world
        self.num_blocks, self.max_blocks = num_blocks, max_blocks_per_seq
        dev, B, d, hd = self.device, batch, cfg.d_model, cfg.head_dim
        ops.init()
        self.layers: list[dict] = []
        self.embed = self.final_norm = self.head = None
        self.key_pools = [torch.zeros((num_blocks, cfg.block_size, self.hk, hd), dtype=cfg.kv_dtype, device=dev)
                          for _ in range(cfg.num_layers)]
        self.value_pools = [torch.zeros_like(p) for p in self.key_pools]
        cos, sin = rope_tables(cfg.rope_theta, hd, cfg.max_positions)
        self.cos, self.sin = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
        i32 = dict(dtype=torch.int32, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        # step inputs (static addresses: the CUDA graph reads them)
        self.token_ids = torch.zeros((B,), **i32)
        self.positions = torch.zeros((B,), **i32)
        self.block_tables = torch.zeros((B, max_blocks_per_seq), **i32)
        self.seq_lens = torch.ones((B,), **i32)
        self.slot_mapping = torch.full((B,), -1, **i32)
        # step buffers
        nqkv = (self.hq + 2 * self.hk) * hd
        # Tensor parallelism, the sum over ranks after o_proj and down_proj.  $TLALOC_B200_TP_REDUCE:
        #   "peer" (default)  the library's peer-memory kernels: at 2 ranks the one-barrier kernel ("peer1"), at more the
        #                     two-phase one ("peer2");
        #   "peer1"           the one-barrier kernel: the projections write their partial results into two alternating
        #                     peer-mapped buffers, and every rank builds residual + sum (and the next RMSNorm) locally
        #                     from all ranks' partials.  Every rank reads (world - 1) whole buffers, so its traffic
        #                     grows with the world size: 4 MiB at 2 ranks, 28 MiB at 8;
        #   "peer2"           the two-phase in-place kernel (reduce-scatter + all-gather over the residual buffers,
        #                     2 (world - 1) / world buffers of traffic per rank whatever the world size);
        #   "nccl"            NCCL's all-reduce on private buffers.
        self.peer, self.one_shot = None, False
        mode = os.environ.get("TLALOC_B200_TP_REDUCE", "peer") if world > 1 else "none"
        if mode == "peer":
            mode = "peer1" if world <= 2 else "peer2"
        if mode in ("peer1", "peer2"):
            self.peer = PeerBuffers([(B, d), (B, d)], rank=rank, world=world, group=group, device=dev, norm_shape=(B, d))
            self.one_shot = mode == "peer1" and self.peer.can_sum_rows(0)
        if self.peer is not None and not self.one_shot:
            self.h, self.h2 = self.peer.tensors  # summed in place
        else:
            self.h = torch.empty((B, d), **f32)
            self.h2 = torch.empty((B, d), **f32)
        # RMSNorm output; with the two-phase peer sum it lives in the peer block and the exchange kernel fills it
        self.fuse_norm = (self.peer is not None and not self.one_shot and self.peer.can_fuse_norm(0)
                          and os.environ.get("TLALOC_B200_TP_FUSE_NORM", "1") != "0")
        self.hn = self.peer.norm_out if self.fuse_norm else torch.empty((B, d), **bf)
        # With the norm folded into the exchange, the f32 residual stream need not travel at all: each rank keeps its
        # own rows of it, the projections hand over bare partial sums, and only the normalised bf16 rows are gathered
        # ($TLALOC_B200_TP_ROWS=0: every rank keeps the whole stream, summed in place).
        self.rows_residual = self.fuse_norm and os.environ.get("TLALOC_B200_TP_ROWS", "1") != "0"
        if self.rows_residual:
            self.row_lo, self.row_hi = B * rank // world, B * (rank + 1) // world
            self.h_rows = torch.empty((self.row_hi - self.row_lo, d), **f32)
        self.qkv = torch.empty((B, nqkv), **f32)
        self.q_rot = torch.empty((B, self.hq, hd), **f32)
        self.att = torch.empty((B, self.hq, hd), **bf)
        self.gu = torch.empty((B, 2 * self.f), **f32)
        self.act = torch.empty((B, self.f), **bf)
        # Batches of 17 to 128 rows run the layers' projections on the int8 tensor-core kernel (the activations as
        # 16-bit fixed point per row; $TLALOC_B200_GEMM_I8=0 keeps the bf16 one).  Their int8 planes live in a scratch
        # that the projections share: the projections of a step run one at a time.
        self.i8_mma = 17 <= B <= 128 and not self.exact
        kmax = max(d, self.hq * hd, self.f)
        self.proj_scratch = torch.empty((ops.int8_gemm_scratch_bytes(B, kmax, 0) + 3) // 4, **f32) if self.i8_mma else None
        # The kernels that produce the normalised rows (RMSNorm, the one-barrier sum over ranks) write those planes
        # themselves, so q|k|v and gate|up need no quantizer launch of their own ($TLALOC_B200_NORM_PLANES=0: they do).
        self.norm_planes = self.i8_mma and d % 16 == 0 and d <= 8192 and os.environ.get("TLALOC_B200_NORM_PLANES", "1") != "0"
        # Likewise the row-distributed exchange: the normalised rows travel as those planes instead of bf16 (same bytes).
        # Only where the projections that read them are sure to take the int8 form: the region then holds no bf16 rows.
        self.rows_planes = (self.rows_residual and self.norm_planes and nqkv % 16 == 0 and (2 * self.f) % 16 == 0
                            and os.environ.get("TLALOC_B200_GEMM_I8", "1") != "0" and os.environ.get("TLALOC_B200_TP_PLANES", "1") != "0")
        self.logits = torch.empty((B, cfg.vocab // world), **f32)
        self.next_ids = torch.zeros((B,), **i32)
        self.best = torch.empty((B,), **f32)
        shape = ops.parse_paged_attention(self.q_rot, self.key_pools[0], self.value_pools[0], self.block_tables,
                                          self.seq_lens, scale=cfg.scale)
        self.att_scratch = ops.paged_attention_scratch(shape, dev)
        self._graph = None

    # ------------------------------------------------------------------ weights

    def load_host_weights(self, w) -> None:
        """Weights in the reference's staged layout (`oracle.DecoderWeights`-shaped: int8 codes [in, out] + f32
        scales [out] per projection, embedding/head values, norm gains), sharded for this rank."""
        cfg, dev = self.cfg, self.device
        t = lambda a, dt=None: (torch.from_numpy(np.ascontiguousarray(a)).to(dev) if dt is None
                                else torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(dt))
        self.embed = t(w.embed, torch.bfloat16)
        self.final_norm = t(w.final_norm)
        self.layers = []
        for lw in w.layers:
            s = sharding.shard_layer(lw, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.ffn, self.rank, self.world,
                                     fuse_swiglu=self.fuse_swiglu)
            self.layers.append({k: (tuple(t(x) for x in v) if isinstance(v, tuple) else t(v)) for k, v in s.items()})
        head = sharding.shard_head(w.head, cfg.vocab, self.rank, self.world)
        self.head = tuple(t(x) for x in head) if isinstance(head, tuple) else t(head, torch.bfloat16)

    def init_random_weights(self, seed: int = 0) -> None:
        """Random int8 codes (uniform in [-127, 127]) and scales on the device, for throughput runs at sizes whose
        weights would not fit through host memory.  Scales are sized so activations stay O(1) through the layers."""
        cfg, dev = self.cfg, self.device
        g = torch.Generator(device=dev)
        g.manual_seed(seed * 1000 + self.rank)
        d, hd = cfg.d_model, cfg.head_dim

        def lin(k, n):
            codes = torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev, generator=g)
            scales = torch.empty((n,), dtype=torch.float32, device=dev).uniform_(0.5, 1.5, generator=g) / (73.0 * np.sqrt(k))
            return codes, scales

        self.embed = (torch.randn((cfg.vocab, d), device=dev, generator=g) * 0.02).to(torch.bfloat16)
        self.final_norm = torch.ones((d,), dtype=torch.float32, device=dev)
        self.layers = []
        for _ in range(cfg.num_layers):
            self.layers.append({
                "qkv": lin(d, (self.hq + 2 * self.hk) * hd), "o": lin(self.hq * hd, d),
                "gate_up": lin(d, 2 * self.f), "down": lin(self.f, d),
                "ln1": torch.ones((d,), dtype=torch.float32, device=dev),
                "ln2": torch.ones((d,), dtype=torch.float32, device=dev),
            })
        self.head = lin(d, cfg.vocab // self.world)

    def weight_bytes(self) -> int:
        n = 0
        for lw in self.layers:
            for key in ("qkv", "o", "gate_up", "down"):
                n += lw[key][0].numel() + 4 * lw[key][1].numel()
        n += (self.head[0].numel() + 4 * self.head[1].numel()) if isinstance(self.head, tuple) else 2 * self.head.numel()
        return n

    # ------------------------------------------------------------------ the step

    def set_inputs(self, token_ids, positions, block_tables, seq_lens, slot_mapping) -> None:
        """Host (NumPy or pinned torch) step inputs -> the device buffers the graph reads."""
        for dst, src in ((self.token_ids, token_ids), (self.positions, positions), (self.block_tables, block_tables),
                         (self.seq_lens, seq_lens), (self.slot_mapping, slot_mapping)):
            if src is None:
                continue
            if isinstance(src, np.ndarray):
                src = torch.from_numpy(np.ascontiguousarray(src, dtype=np.int32))
            dst.copy_(src.reshape(dst.shape), non_blocking=True)

    def _all_reduce(self, x: torch.Tensor) -> None:
        if self.world == 1:
            return
        if self.peer is not None:
            self.peer.all_reduce_(0 if x is self.h else 1)
        else:
            torch.distributed.all_reduce(x, group=self.group)

    def _run_step(self) -> None:
        if not self.exact:
            return self._launch_step()
        before = ops.set_order_faithful(True)
        try:
            self._launch_step()
        finally:
            ops.set_order_faithful(before)

    def _launch_step(self) -> None:
        if self.one_shot:
            return self._launch_step_one_shot()
        if self.rows_residual:
            return self._launch_step_rows()
        cfg, B = self.cfg, self.batch
        hd, hq, hk = cfg.head_dim, self.hq, self.hk
        ops.embedding(self.embed, self.token_ids, out=self.h)
        h, h2 = self.h, self.h2
        res_rank = self.rank == 0  # under tensor parallelism the residual enters the all-reduced sum once
        q3, k3, v3 = self._qkv_views()
        fused = self.fuse_norm  # the sum over ranks also produces the next RMSNorm's output
        pl = self.proj_scratch if self.norm_planes else None  # RMSNorm leaves hn's int8 planes there for the projection
        how = dict(weights_const=True, scratch=self.proj_scratch, i8_mma=self.i8_mma)
        for l, lw in enumerate(self.layers):
            xp = False  # hn's planes are in the scratch (only when this rank's own RMSNorm kernel produced hn)
            if l == 0 or not fused:
                ops.rmsnorm(h, lw["ln1"], cfg.rms_eps, out=self.hn, planes=pl)
                xp = pl is not None
            ops.int8_gemm(self.hn, *lw["qkv"], out=self.qkv, x_planes=xp, **how)
            ops.rope_kv_write(q3, k3, v3, self.positions, self.cos, self.sin, self.slot_mapping, self.key_pools[l],
                              self.value_pools[l], q_out=self.q_rot)
            ops.paged_attention(self.q_rot, self.key_pools[l], self.value_pools[l], self.block_tables, self.seq_lens,
                                scale=cfg.scale, out=self.att, scratch=self.att_scratch)
            ops.int8_gemm(self.att.view(B, hq * hd), *lw["o"], residual=h if res_rank else None, out=h2, **how)
            if fused:
                self.peer.all_reduce_norm_(1, lw["ln2"], cfg.rms_eps)
                xp = False
            else:
                self._all_reduce(h2)
                ops.rmsnorm(h2, lw["ln2"], cfg.rms_eps, out=self.hn, planes=pl)
                xp = pl is not None
            self.gate_up_proj(lw, x_planes=xp)
            ops.int8_gemm(self.act, *lw["down"], residual=h2 if res_rank else None, out=h, **how)
            if fused:
                nxt = self.layers[l + 1]["ln1"] if l + 1 < len(self.layers) else self.final_norm
                self.peer.all_reduce_norm_(0, nxt, cfg.rms_eps)
            else:
                self._all_reduce(h)
        if not fused:
            ops.rmsnorm(h, self.final_norm, cfg.rms_eps, out=self.hn)
        self._head_and_greedy()

    def _launch_step_rows(self) -> None:
        """The tensor-parallel step with the residual stream distributed by rows: o_proj and down_proj write bare partial
        sums into the two peer buffers; the exchange kernel adds this rank's rows of the residual stream and every
        rank's partial, keeps the sums in `h_rows` and gathers only the next RMSNorm's bf16 output."""
        cfg, B = self.cfg, self.batch
        hd, hq = cfg.head_dim, self.hq
        p_down, p_o = self.peer.tensors
        ops.embedding(self.embed, self.token_ids, out=p_down)  # the whole embedding on every rank: its norm is local
        self.h_rows.copy_(p_down[self.row_lo:self.row_hi])
        q3, k3, v3 = self._qkv_views()
        how = dict(weights_const=True, scratch=self.proj_scratch, i8_mma=self.i8_mma)
        pl = self.proj_scratch if self.norm_planes else None
        ops.rmsnorm(p_down, self.layers[0]["ln1"], cfg.rms_eps, out=self.hn, planes=pl)
        rp = self.rows_planes  # the exchange hands the next projection its int8 planes (in the peer block) instead of bf16 rows
        from_peer = dict(how, scratch=self.peer.norm_planes, x_planes=True)
        last = len(self.layers) - 1
        for l, lw in enumerate(self.layers):
            if l == 0:
                ops.int8_gemm(self.hn, *lw["qkv"], out=self.qkv, x_planes=pl is not None, **how)
            else:
                ops.int8_gemm(self.hn, *lw["qkv"], out=self.qkv, **(from_peer if rp else how))
            ops.rope_kv_write(q3, k3, v3, self.positions, self.cos, self.sin, self.slot_mapping, self.key_pools[l],
                              self.value_pools[l], q_out=self.q_rot)
            ops.paged_attention(self.q_rot, self.key_pools[l], self.value_pools[l], self.block_tables, self.seq_lens,
                                scale=cfg.scale, out=self.att, scratch=self.att_scratch)
            ops.int8_gemm(self.att.view(B, hq * hd), *lw["o"], out=p_o, **how)
            self.peer.reduce_norm_rows_(1, self.h_rows, lw["ln2"], cfg.rms_eps, planes=rp)
            self.gate_up_proj(lw, x_planes=rp, scratch=self.peer.norm_planes if rp else None)
            ops.int8_gemm(self.act, *lw["down"], out=p_down, **how)
            nxt = self.layers[l + 1]["ln1"] if l < last else self.final_norm
            self.peer.reduce_norm_rows_(0, self.h_rows, nxt, cfg.rms_eps, planes=rp and l < last)  # the head reads bf16 rows
        self._head_and_greedy()

    def _launch_step_one_shot(self) -> None:
        """The tensor-parallel step on the one-barrier sum: the residual stream `h` is local and identical on every rank;
        o_proj and down_proj write their partial results into the two peer buffers in turn, and the sum kernel adds
        every rank's partial to `h` and leaves the next RMSNorm's output in `hn`."""
        cfg, B = self.cfg, self.batch
        hd, hq = cfg.head_dim, self.hq
        ops.embedding(self.embed, self.token_ids, out=self.h)
        h, (p_o, p_down) = self.h, self.peer.tensors
        q3, k3, v3 = self._qkv_views()
        pl = self.proj_scratch if self.norm_planes else None  # the kernels that write hn also leave its int8 planes there
        xp = pl is not None
        how = dict(weights_const=True, scratch=self.proj_scratch, i8_mma=self.i8_mma)
        ops.rmsnorm(h, self.layers[0]["ln1"], cfg.rms_eps, out=self.hn, planes=pl)
        for l, lw in enumerate(self.layers):
            ops.int8_gemm(self.hn, *lw["qkv"], out=self.qkv, x_planes=xp, **how)
            ops.rope_kv_write(q3, k3, v3, self.positions, self.cos, self.sin, self.slot_mapping, self.key_pools[l],
                              self.value_pools[l], q_out=self.q_rot)
            ops.paged_attention(self.q_rot, self.key_pools[l], self.value_pools[l], self.block_tables, self.seq_lens,
                                scale=cfg.scale, out=self.att, scratch=self.att_scratch)
            ops.int8_gemm(self.att.view(B, hq * hd), *lw["o"], out=p_o, **how)
            self.peer.sum_rows_(0, h, h, lw["ln2"], cfg.rms_eps, norm_out=self.hn, planes=pl)
            self.gate_up_proj(lw, x_planes=xp)
            ops.int8_gemm(self.act, *lw["down"], out=p_down, **how)
            nxt = self.layers[l + 1]["ln1"] if l + 1 < len(self.layers) else self.final_norm
            self.peer.sum_rows_(1, h, h, nxt, cfg.rms_eps, norm_out=self.hn, planes=pl)
        self._head_and_greedy()

    def _qkv_views(self):
        hd, hq, hk = self.cfg.head_dim, self.hq, self.hk
        return (self.qkv[:, :hq * hd].unflatten(1, (hq, hd)), self.qkv[:, hq * hd:(hq + hk) * hd].unflatten(1, (hk, hd)),
                self.qkv[:, (hq + hk) * hd:].unflatten(1, (hk, hd)))

    def _head_and_greedy(self) -> None:
        if isinstance(self.head, tuple):
            ops.int8_gemm(self.hn, *self.head, out=self.logits, weights_const=True)  # the logits stay on f32 accumulation
        else:
            self.logits.copy_(ops.dense_gemm_exact(self.hn, self.head))
        ops.argmax(self.logits, out=self.next_ids)
        if self.world > 1:
            self._merge_greedy()

    def gate_up_proj(self, lw, x_planes: bool = False, scratch=None) -> None:
        """The MLP's first half for one layer: normalised rows `hn` -> `act` = silu(gate) * up, as one projection with
        SwiGLU in its epilogue where the shape allows, else the fused gate|up projection and the SwiGLU kernel.
        `scratch`: where the planes of `hn` are (x_planes) or go; the step's shared projection scratch by default."""
        scratch = self.proj_scratch if scratch is None else scratch
        if self.fuse_swiglu:
            ops.int8_gemm_swiglu(self.hn, *lw["gate_up"], out=self.act, weights_const=True, scratch=scratch, i8_mma=self.i8_mma,
                                 x_planes=x_planes)
        else:
            ops.int8_gemm(self.hn, *lw["gate_up"], out=self.gu, weights_const=True, scratch=scratch, i8_mma=self.i8_mma,
                          x_planes=x_planes)
            ops.swiglu(self.gu[:, :self.f], self.gu[:, self.f:], out=self.act)

    def _merge_greedy(self) -> None:
        """Each rank's best (logit, local id) -> the global greedy token on every rank (sharding.merge_greedy)."""
        B, g, vp = self.batch, self.world, self.cfg.vocab // self.world
        best = self.logits.gather(1, self.next_ids.long()[:, None])[:, 0].contiguous()
        vals = torch.empty((g, B), dtype=torch.float32, device=self.device)
        ids = torch.empty((g, B), dtype=torch.int32, device=self.device)
        torch.distributed.all_gather_into_tensor(vals, best, group=self.group)
        torch.distributed.all_gather_into_tensor(ids, self.next_ids, group=self.group)
        # the largest value; among equals the lowest rank, whose ids are the lowest: argmax returns the first maximum
        win = vals.argmax(dim=0)
        glob = ids.long() + (torch.arange(g, device=self.device) * vp)[:, None]
        self.next_ids.copy_(glob.gather(0, win[None, :])[0].to(torch.int32))

    def capture(self) -> None:
        """Capture the step into a CUDA graph (after one eager warm-up step on a side stream)."""
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self._run_step()
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._run_step()

    def exchange_status(self) -> int:
        """0, or the code a timed-out wait of the tensor-parallel sum left behind (see PeerBuffers.status)."""
        return self.peer.status() if self.peer is not None else 0

    def step(self) -> torch.Tensor:
        """One decode step over the current inputs; returns the device tensor of next token ids [batch]."""
        if self._graph is not None:
            self._graph.replay()
        else:
            self._run_step()
        return self.next_ids

    # ------------------------------------------------------------------ traffic model

    def step_bytes(self, seq_lens: np.ndarray) -> dict:
        """Algorithmic HBM bytes of one step on this rank: every weight byte once, every live K/V element once."""
        cfg = self.cfg
        kv = 2 * int(np.sum(seq_lens)) * self.hk * cfg.head_dim * self.key_pools[0].element_size() * cfg.num_layers
        return {"weights": self.weight_bytes(), "kv": kv}
