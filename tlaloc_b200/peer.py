"""Peer-mapped step buffers and the in-place sum over tensor-parallel ranks (one process per GPU).

The reference leaves the `stablehlo.all_reduce` after o_proj and down_proj to XLA
(stablehlo/.../StablehloEmitter.kt:3048-3072).  Here each rank allocates ONE device buffer that holds the tensors to be
summed plus the flag words, every rank maps every other rank's buffer (CUDA IPC handles exchanged over the process
group), and `PeerBuffers.all_reduce_(i)` launches the library's one-kernel exchange (csrc/peer_allreduce.cu) on the
current stream.  The launch has no host synchronisation, so it can be captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _native as N

_ALIGN = 256


class _DeviceSpan:
    """A raw device address range, exposed to torch through the CUDA array interface."""

    def __init__(self, ptr: int, words: int):
        self.__cuda_array_interface__ = {"shape": (words,), "typestr": "<f4", "data": (ptr, False), "version": 3}


class PeerBuffers:
    """`shapes` f32 tensors living in a buffer every rank of `group` can read and write, with `all_reduce_` over them.

    All ranks must construct it with the same shapes (a collective: handles are all-gathered), call `all_reduce_`
    in the same order, and `close()` it together.
    """

    def __init__(self, shapes, *, rank: int, world: int, group=None, device="cuda:0", norm_shape=None):
        if not 1 <= world <= 8:
            raise ValueError(f"world {world} outside [1, 8]")
        self.rank, self.world, self.group, self.device = rank, world, group, torch.device(device)
        self.offsets, off = [], 0
        for shp in shapes:
            n = int(np.prod(shp))
            if n % 4:
                raise ValueError(f"a summed tensor needs a multiple of 4 elements, got shape {tuple(shp)}")
            self.offsets.append(off)
            off += (4 * n + _ALIGN - 1) // _ALIGN * _ALIGN
        # one bf16 matrix for the fused sum + RMSNorm (all_reduce_norm_): every rank receives every normalised row
        self.norm_offset, self.norm_shape = off, None
        if norm_shape is not None:
            self.norm_shape = tuple(int(v) for v in norm_shape)
            # bf16 rows, or the same rows as two int8 planes and a step per row (reduce_norm_rows_ with planes)
            self.norm_bytes = (2 * int(np.prod(self.norm_shape)) + 4 * self.norm_shape[0] + _ALIGN - 1) // _ALIGN * _ALIGN
            off += self.norm_bytes
        self.flag_offset = off
        self.nbytes = off + _ALIGN
        lib = N.lib()
        torch.cuda.set_device(self.device)
        local, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        N.check(lib.tlaloc_b200_peer_alloc(self.nbytes, ctypes.byref(local), handle))
        self._local = local.value
        handles = [None] * world
        if world > 1:
            torch.distributed.all_gather_object(handles, handle.raw, group=group)
        else:
            handles[0] = handle.raw
        self._bases = (ctypes.c_void_p * world)()
        self._opened = []
        for q in range(world):
            if q == rank:
                self._bases[q] = self._local
                continue
            p = ctypes.c_void_p()
            N.check(lib.tlaloc_b200_peer_open(handles[q], ctypes.byref(p)))
            self._bases[q] = p.value
            self._opened.append(p.value)
        whole = torch.as_tensor(_DeviceSpan(self._local, self.nbytes // 4), device=self.device)
        self.tensors = [whole[o // 4:o // 4 + int(np.prod(s))].view(*s) for o, s in zip(self.offsets, shapes)]
        self.norm_out = self.norm_planes = None
        if self.norm_shape is not None:
            n = int(np.prod(self.norm_shape))
            self.norm_out = whole[self.norm_offset // 4:self.norm_offset // 4 + (n + 1) // 2].view(torch.bfloat16)[:n].view(*self.norm_shape)
            self.norm_planes = whole[self.norm_offset // 4:(self.norm_offset + self.norm_bytes) // 4]  # the same region as a scratch
        self.state = torch.zeros((4,), dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        if world > 1:
            torch.distributed.barrier(group=group)  # every rank has mapped every buffer before the first exchange

    def all_reduce_(self, index: int) -> torch.Tensor:
        """Sum tensor `index` over the ranks, in place, on the current stream; every rank ends with identical bits."""
        t = self.tensors[index]
        N.check(N.lib().tlaloc_b200_peer_allreduce_f32(self._bases, self.offsets[index], self.flag_offset,
                                                       self.state.data_ptr(), self.rank, self.world, t.numel(),
                                                       torch.cuda.current_stream(self.device).cuda_stream))
        return t

    def can_fuse_norm(self, index: int) -> bool:
        """Whether all_reduce_norm_ takes tensor `index`: a [rows, cols] matrix the shape of the norm region, rows
        divisible by the ranks, cols a multiple of 16 up to 32768."""
        t = self.tensors[index]
        return (self.world > 1 and self.norm_out is not None and t.dim() == 2 and tuple(t.shape) == self.norm_shape
                and t.shape[0] % self.world == 0 and t.shape[1] % 16 == 0 and t.shape[1] <= 32768)

    def all_reduce_norm_(self, index: int, gain, eps: float):
        """Sum tensor `index` over the ranks in place AND leave RMSNorm(sum) * gain as bf16 in `norm_out`, on every rank."""
        t = self.tensors[index]
        N.check(N.lib().tlaloc_b200_peer_allreduce_rmsnorm_f32(
            self._bases, self.offsets[index], self.norm_offset, self.flag_offset, self.state.data_ptr(),
            None if gain is None else gain.data_ptr(), float(eps), self.rank, self.world, t.shape[0], t.shape[1],
            torch.cuda.current_stream(self.device).cuda_stream))
        return t, self.norm_out

    def reduce_norm_rows_(self, index: int, own_rows, gain, eps: float, planes: bool = False):
        """Tensor `index` holds this rank's PARTIAL result.  Adds this rank's rows of the residual stream (`own_rows`,
        local f32 [rows / world, cols], updated in place) and every rank's partial for those rows, and leaves
        RMSNorm(sum) * gain of ALL rows as bf16 in `norm_out` on every rank.  The f32 sums never travel.
        `planes`: the rows arrive as the int8 tensor-core projection's activation planes instead (`norm_planes`, to be
        passed as that projection's scratch with x_planes=True); `norm_out` then holds no bf16 rows."""
        t = self.tensors[index]
        if (own_rows.dtype != torch.float32 or not own_rows.is_contiguous() or own_rows.dim() != 2
                or own_rows.shape[0] * self.world != t.shape[0] or own_rows.shape[1] != t.shape[1]):
            raise ValueError("reduce_norm_rows_: own_rows must be contiguous f32 [rows / world, cols]")
        N.check(N.lib().tlaloc_b200_peer_reduce_rmsnorm_rows_f32(
            self._bases, self.offsets[index], self.norm_offset, self.flag_offset, self.state.data_ptr(), own_rows.data_ptr(),
            None if gain is None else gain.data_ptr(), float(eps), self.rank, self.world, t.shape[0], t.shape[1],
            1 if planes else 0, torch.cuda.current_stream(self.device).cuda_stream))
        return self.norm_planes if planes else self.norm_out

    def sum_rows_(self, index: int, residual, out, gain, eps: float, norm_out=None, planes=None):
        """The one-barrier form: out = residual + sum over ranks of tensor `index` (every rank's partial, added in rank
        order) into LOCAL `out` (f32, may be `residual` itself), and RMSNorm(out) * gain as bf16 into local `norm_out`;
        `planes` (the scratch of the int8 tensor-core projection that reads norm_out) also receives the normalised rows
        as that projection's activation planes.
        The caller must not overwrite tensor `index` again before one more sum_rows_ (on another tensor) has run."""
        t = self.tensors[index]
        if t.dim() != 2 or tuple(out.shape) != tuple(t.shape) or out.dtype != torch.float32 or not out.is_contiguous():
            raise ValueError("sum_rows_: out must be a contiguous f32 tensor of the partial's [rows, cols] shape")
        if norm_out is not None and (tuple(norm_out.shape) != tuple(t.shape) or norm_out.dtype != torch.bfloat16 or not norm_out.is_contiguous()):
            raise ValueError("sum_rows_: norm_out must be a contiguous bf16 tensor of the partial's shape")
        N.check(N.lib().tlaloc_b200_peer_sum_rows_f32(
            self._bases, self.offsets[index], self.flag_offset, self.state.data_ptr(),
            None if residual is None else residual.data_ptr(), out.data_ptr(), None if norm_out is None else norm_out.data_ptr(),
            None if gain is None else gain.data_ptr(), float(eps), self.rank, self.world, t.shape[0], t.shape[1],
            None if planes is None else planes.data_ptr(), 0 if planes is None else planes.numel() * planes.element_size(),
            torch.cuda.current_stream(self.device).cuda_stream))
        return out

    def can_sum_rows(self, index: int) -> bool:
        t = self.tensors[index]
        return t.dim() == 2 and t.shape[1] % 4 == 0 and t.shape[1] <= 8192

    def status(self) -> int:
        """0, or the code a timed-out wait left (1 + 16 * phase + the rank that did not arrive).  Synchronises."""
        return int(self.state[2].item())

    def close(self) -> None:
        """Unmap the peers' buffers, then (after a barrier) free the local one.  The tensors must not be used after."""
        if self._local is None:
            return
        torch.cuda.synchronize(self.device)
        lib = N.lib()
        for p in self._opened:
            lib.tlaloc_b200_peer_close(p)
        self._opened = []
        if self.world > 1:
            torch.distributed.barrier(group=self.group)
        self.tensors = []
        lib.tlaloc_b200_peer_free(self._local)
        self._local = None
