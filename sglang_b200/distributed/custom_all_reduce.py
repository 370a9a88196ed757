"""All-reduce of the row-parallel linear's partial outputs with this library's own NVLink kernels.

Takes the place of the reference's custom all-reduce
(sgl-kernel/csrc/allreduce/custom_all_reduce.cuh; Python side
python/sglang/srt/distributed/device_communicators/custom_all_reduce.py) and of the NCCL call behind
tensor_model_parallel_all_reduce (python/sglang/srt/distributed/communication_op.py:11-13).

The partial outputs live in a symmetric buffer: the same allocation on every rank, mapped into every
process, and -- on an NVSwitch machine -- bound to an NVLink multicast object.
`torch.distributed._symmetric_memory` does the allocation and the address exchange (plumbing); the
reduction itself is `b200_allreduce`: a two-shot kernel that pulls each rank's slice of the sum out of
the switch with `multimem.ld_reduce` and pushes it to every rank with `multimem.st` (plain peer loads and
stores when there is no multicast address), or a one-shot kernel for small buffers.  The row-parallel
linear writes its GEMM output straight into the buffer (`out=`), so no copy precedes the reduction.

One process per GPU.  The kernels of different ranks wait for one another: every rank must make the
same calls in the same order.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib

_DT = {torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}
# below this many bytes one pass over every peer's buffer beats two passes over a slice
ONE_SHOT_MAX_BYTES = 512 * 1024


class SymmetricAllReduce:
    """A symmetric buffer of `max_bytes` on every rank of `group` plus the all-reduce over it.

    autotune(nbytes)          times the multicast and the peer-pointer form and keeps the faster one
    buffer(shape, dtype)      a view of the buffer's start to write partial results into
    all_reduce_(t)            in place over a row-contiguous view of the buffer (two-shot)
    all_reduce_small(t, out)  one-shot into a local tensor (small buffers)
    check()                   raises if a wait for a peer ever ran out on this rank
    """

    def __init__(self, max_bytes: int, group=None, device: Optional[torch.device] = None, use_multicast: bool = True,
                 num_blocks: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world < 2 or self.world > 8:
            raise ValueError(f"world size {self.world}: the kernels are built for 2..8 ranks of one NVSwitch domain")
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        L = _lib.lib()
        flag_bytes = 4 * L.b200_allreduce_flag_words(self.world)
        if symm_mem.get_signal_pad_size() < flag_bytes:
            symm_mem.set_signal_pad_size(flag_bytes)
        granule = 16 * self.world
        self.nbytes = (int(max_bytes) + granule - 1) // granule * granule
        self._buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self._hdl = symm_mem.rendezvous(self._buf, self.group)
        # The handle's pointers address the start of the symmetric ALLOCATION on every rank; the tensor may sit at
        # an offset inside it (the same offset on every rank).
        self.base_offset = int(self._buf.data_ptr()) - int(self._hdl.buffer_ptrs[self.rank])
        self._peer_ptrs = (ctypes.c_void_p * self.world)(*[int(p) + self.base_offset for p in self._hdl.buffer_ptrs])
        self._signal_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self._hdl.signal_pad_ptrs])
        mc = int(self._hdl.multicast_ptr) if use_multicast else 0
        self._mc_addr = mc + self.base_offset if mc else 0
        self.multicast = mc != 0
        self.has_multicast = mc != 0
        self._mc = ctypes.c_void_p(self._mc_addr if mc else None)
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.num_blocks = int(num_blocks)
        self._hdl.barrier()   # every rank's flags are zero before the first kernel touches them

    def set_form(self, form: str) -> None:
        """"multicast": sums come out of the NVSwitch (multimem.ld_reduce / multimem.st); "peer": plain loads from and
        stores to every rank's buffer.  Every rank must choose the same form."""
        if form == "multicast":
            if not self._mc_addr:
                raise ValueError("no multicast address for this buffer")
            self.multicast, self._mc = True, ctypes.c_void_p(self._mc_addr)
        elif form == "peer":
            self.multicast, self._mc = False, ctypes.c_void_p(None)
        else:
            raise ValueError(form)

    def autotune(self, nbytes: int, iters: int = 10) -> dict:
        """Times the two-shot all-reduce of `nbytes` in both forms (max over ranks) and keeps the faster one; every
        rank must call it.  Which form wins depends on the rank count: through the switch every rank's own slice
        crosses NVLink too, with peer pointers only remote data does, but every SM's loads pay the NVLink latency.
        The buffer's contents are overwritten.  Returns {form: microseconds}."""
        granule = 16 * self.world
        nbytes = min(self.nbytes, (int(nbytes) + granule - 1) // granule * granule)
        view = self._buf[:nbytes].view(torch.bfloat16)
        forms = (["multicast"] if self._mc_addr else []) + ["peer"]
        times = {}
        for form in forms:
            self.set_form(form)
            view.zero_()
            for _ in range(2):
                self.all_reduce_(view)
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                self.all_reduce_(view)
            b.record()
            torch.cuda.synchronize(self.device)
            t = torch.tensor([a.elapsed_time(b) / iters * 1e3], device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            times[form] = float(t.item())
        self.check()
        self.set_form(min(times, key=times.get))      # same numbers on every rank, so the same choice
        return times

    def buffer(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if nbytes > self.nbytes:
            raise ValueError(f"{nbytes} bytes asked of a {self.nbytes}-byte symmetric buffer")
        return self._buf[:nbytes].view(dtype).view(*shape)

    def _offset(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self._buf.data_ptr()
        if off < 0 or off + t.numel() * t.element_size() > self.nbytes or not t.is_contiguous():
            raise ValueError("the tensor must be a contiguous view of this symmetric buffer")
        return off

    def _launch(self, t: torch.Tensor, out: Optional[torch.Tensor], one_shot: bool) -> None:
        if t.dtype not in _DT:
            raise TypeError("bf16 or fp16 only")
        off = self._offset(t)
        nbytes = t.numel() * t.element_size()
        pad = 16 if one_shot else 16 * self.world
        if off % 16 != 0 or nbytes % pad != 0:
            raise ValueError(f"offset must be a multiple of 16 bytes and the length of {pad} bytes")
        with torch.cuda.device(self.device):
            rc = _lib.lib().b200_allreduce(
                self._peer_ptrs, self._signal_ptrs, self._mc, out.data_ptr() if out is not None else None,
                self._status.data_ptr(), off, nbytes, _DT[t.dtype], self.rank, self.world, 1 if one_shot else 0,
                self.num_blocks, 0, torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check("b200_allreduce", rc)

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        """Sum over ranks, in place; `t` is a contiguous view of the buffer at the same offset on every rank."""
        self._launch(t, None, False)
        return t

    def all_reduce_small(self, t: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum over ranks of a small view of the buffer into a local tensor (one pass)."""
        if out is None:
            out = torch.empty(t.shape, dtype=t.dtype, device=t.device)
        self._launch(t, out, True)
        return out

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """Size-based choice between the two forms; returns the tensor that holds the sum."""
        if t.numel() * t.element_size() <= ONE_SHOT_MAX_BYTES:
            return self.all_reduce_small(t)
        return self.all_reduce_(t)

    def check(self) -> None:
        """Synchronises and raises if any wait for a peer gave up on this rank (the sums are then wrong)."""
        code = int(self._status.item())
        if code != 0:
            self._status.zero_()
            raise _lib.B200Error("b200_allreduce", -10, f"a wait for a peer rank gave up (barrier code {code})")
