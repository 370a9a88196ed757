"""Expert-parallel block-FP8 MoE.

Sharding follows the reference: experts are split contiguously, E/p per rank
(python/sglang/srt/layers/moe/fused_moe_triton/layer.py:165-185); tokens stay sharded across ranks.
The reference moves tokens with DeepEP (python/sglang/srt/layers/moe/token_dispatcher/deepep.py:314-480,
which dispatches ALREADY-QUANTISED fp8 rows + scales, :328-336) or replicates tokens and all-reduces
(layer.py:813-818,850-851).  Two exchanges are built here:

  backend "nvlink" (CUDA, default): this library's own dispatch / combine kernels (csrc/ep_moe.cu) over a
      symmetric buffer that `torch.distributed._symmetric_memory` allocates and maps into every rank.  Each
      (token, choice) row -- e4m3 codes, fp32 scales, local expert id, source slot -- is stored straight into
      the owning rank's receive region with peer stores; the expert outputs come back the same way.  Nothing
      on the host looks at a count (no device->host copy, no host-side split sizes): the receive region
      holds `capacity` rows per source rank and unused rows carry expert id -1.
  backend "nccl": `all_to_all_single` of codes, scales and ids with host-side split sizes (one small
      device->host copy per call).  Works on any process group (the CPU tests run it over gloo).

Either way the routing-weighted sum happens at the source rank in fp32, choices in ascending order --
the same arithmetic, in the same order, as the single-GPU path, so the result is bitwise the single-GPU
result.

The quantiser, the local expert computation and the weighted sum are injectable so the exchange
logic runs on CPU ranks (gloo) in the tests; the defaults are the CUDA kernels (no CPU fallback).
"""
from __future__ import annotations

import ctypes
from typing import Callable, Optional

import torch
import torch.distributed as dist


def _default_quant(x):
    from ..layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    return sglang_per_token_group_quant_fp8(x, 128)


def _default_local(a_q, a_s, ids, w13, w2, w13_s, w2_s, out_dtype):
    from ..layers.moe.cutlass_moe import grouped_experts_prequantized
    return grouped_experts_prequantized(a_q, a_s, ids, w13, w2, w13_s, w2_s, out_dtype)


def _default_weighted_sum(rows, perm, weights, m):
    from ..sgl_kernel import apply_shuffle_mul_sum
    out = torch.empty((m, rows.shape[1]), dtype=rows.dtype, device=rows.device)
    apply_shuffle_mul_sum(rows, out, perm, weights)
    return out


class _NvlinkExchange:
    """The symmetric buffer and scratch of the "nvlink" backend for one (tokens, topk, hidden, dtype) bound."""

    def __init__(self, group, device, max_tokens: int, topk: int, hidden: int, out_dtype: torch.dtype,
                 capacity_factor: float):
        import torch.distributed._symmetric_memory as symm_mem
        from .. import _lib

        self.lib = _lib
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_slots = max_tokens * topk
        cap = int(-(-int(capacity_factor * self.max_slots) // self.world))
        self.capacity = max(8, min(self.max_slots, (cap + 7) // 8 * 8))
        self.hidden, self.topk, self.out_dtype = hidden, topk, out_dtype
        esz = torch.empty((), dtype=out_dtype).element_size()
        self.layout = (ctypes.c_int64 * 5)()
        nbytes = _lib.lib().b200_ep_buffer_bytes(self.world, self.capacity, hidden, self.max_slots, esz, self.layout)
        if nbytes <= 0:
            raise ValueError("bad expert-parallel buffer shape")
        L = _lib.lib()
        flag_bytes = 4 * max(L.b200_allreduce_flag_words(self.world), 4 * self.world)
        if symm_mem.get_signal_pad_size() < flag_bytes:
            symm_mem.set_signal_pad_size(flag_bytes)
        self.buf = symm_mem.empty(int(nbytes), dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group)
        base_offset = int(self.buf.data_ptr()) - int(self.hdl.buffer_ptrs[self.rank])   # tensor inside the allocation
        self.peer_ptrs = (ctypes.c_void_p * self.world)(*[int(p) + base_offset for p in self.hdl.buffer_ptrs])
        self.signal_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self.hdl.signal_pad_ptrs])
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.pos = torch.empty(self.max_slots, dtype=torch.int32, device=device)
        self.counts = torch.zeros(8, dtype=torch.int32, device=device)
        self.counter = torch.zeros(2, dtype=torch.int32, device=device)
        R = self.world * self.capacity
        off = [int(v) for v in self.layout]
        self.recv_q = self.buf[off[0]:off[0] + R * hidden].view(torch.float8_e4m3fn).view(R, hidden)
        self.recv_s_bytes = self.buf[off[1]:off[1] + R * (hidden // 128) * 4]
        self.back = self.buf[off[4]:off[4] + self.max_slots * hidden * esz].view(out_dtype).view(self.max_slots, hidden)
        self.ids = torch.empty(R, dtype=torch.int32, device=device)
        self.identity = torch.arange(self.max_slots, dtype=torch.int32, device=device)
        self.device = device
        torch.cuda.synchronize(device)
        self.hdl.barrier()   # every rank's buffer and flags are zero before the first kernel touches them

    def dispatch(self, q, s, topk_ids, experts_per_rank):
        """s [m, W]: one contiguous row of W 32-bit scale words per token -- fp32 scales (W = hidden / 128) or packed
        power-of-two exponents (int32, W a multiple of 4).  Returns the receive regions; the scale region is viewed
        with s's type and width."""
        m = q.shape[0]
        assert s.dim() == 2 and s.is_contiguous() and s.element_size() == 4 and s.shape[0] == m
        W = s.shape[1]
        st = torch.cuda.current_stream(self.device).cuda_stream
        rc = self.lib.lib().b200_ep_dispatch(
            q.data_ptr(), s.data_ptr(), W, topk_ids.data_ptr(), m, self.topk, self.hidden, experts_per_rank,
            self.peer_ptrs, self.signal_ptrs, self.layout, self.capacity, self.rank, self.world, 0,
            self.status.data_ptr(), self.pos.data_ptr(), self.counts.data_ptr(), self.counter.data_ptr(), st)
        self.lib.check("b200_ep_dispatch", rc)
        rc = self.lib.lib().b200_ep_received_expert_ids(self.buf.data_ptr(), self.layout, self.capacity, self.hidden,
                                                        self.world, self.ids.data_ptr(), st)
        self.lib.check("b200_ep_received_expert_ids", rc)
        R = self.world * self.capacity
        recv_s = self.recv_s_bytes[:R * W * 4].view(s.dtype).view(R, W)
        return self.recv_q, recv_s, self.ids

    def combine(self, rows, row_of):
        dt = {torch.float16: self.lib.DT_F16, torch.bfloat16: self.lib.DT_BF16}[rows.dtype]
        st = torch.cuda.current_stream(self.device).cuda_stream
        rc = self.lib.lib().b200_ep_combine(
            rows.data_ptr(), row_of.data_ptr() if row_of is not None else None, dt, self.hidden, self.peer_ptrs,
            self.signal_ptrs, self.layout, self.capacity, self.rank, self.world, self.world,
            self.status.data_ptr(), self.counter.data_ptr() + 4, st)
        self.lib.check("b200_ep_combine", rc)
        return self.back


class ExpertParallelBlockFp8MoE:
    """w13 [E_local, 2n, H], w2 [E_local, H, n] e4m3 and their block scales: this rank's experts
    (global ids [rank*E_local, (rank+1)*E_local)).

    backend: "nvlink", "nccl" or "auto" (nvlink on CUDA with the default compute functions, else nccl).
    capacity_factor (nvlink): a receive region holds ceil(capacity_factor * tokens * topk / world) rows per
    source rank (never more than tokens * topk, which cannot overflow).  A source that routes more rows than
    that to one rank drops the excess and `check()` raises; the default 2.0 is about twenty standard deviations
    above the mean for uniformly random routing of a few thousand rows.
    max_tokens (nvlink): bound on the tokens per rank and call the exchange buffer is sized for (default: the
    first call's count; a larger later call re-allocates, which is a collective: all ranks must do it together).
    scale_ue8m0 (nvlink): the block-scaling path -- activations quantised to power-of-two scales, dispatched with
    their packed exponent words, expert GEMMs on the block-scaling MMA; the weights' block scales must be powers of
    two (requant_weight_ue8m0).  Bitwise equal to fused_experts_block_fp8_ue8m0 on one GPU."""

    def __init__(self, w13, w2, w13_scale, w2_scale, group=None, quant_fn: Callable = _default_quant,
                 local_fn: Callable = _default_local, weighted_sum_fn: Callable = _default_weighted_sum,
                 backend: str = "auto", capacity_factor: float = 2.0, max_tokens: Optional[int] = None,
                 scale_ue8m0: bool = False):
        self.w13, self.w2, self.w13_scale, self.w2_scale = w13, w2, w13_scale, w2_scale
        self.scale_ue8m0 = bool(scale_ue8m0)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.e_local = w13.shape[0]
        self._quant, self._local, self._wsum = quant_fn, local_fn, weighted_sum_fn
        default_fns = quant_fn is _default_quant and local_fn is _default_local and weighted_sum_fn is _default_weighted_sum
        if backend == "auto":
            backend = "nvlink" if (self.world > 1 and w13.is_cuda and default_fns) else "nccl"
        if backend not in ("nvlink", "nccl"):
            raise ValueError(f"unknown backend {backend!r}")
        if backend == "nvlink" and not (self.world > 1 and w13.is_cuda and default_fns):
            raise ValueError("the nvlink backend needs CUDA ranks (world size > 1) and the default compute functions")
        if self.scale_ue8m0 and backend != "nvlink":
            raise ValueError("power-of-two scales (scale_ue8m0) are built for the nvlink backend")
        self.backend = backend
        self.capacity_factor = float(capacity_factor)
        self.max_tokens = max_tokens
        self._xchg: Optional[_NvlinkExchange] = None

    # ------------------------------------------------------------------ nvlink backend
    def _exchange(self, m: int, topk: int, H: int, dtype: torch.dtype, device) -> _NvlinkExchange:
        x = self._xchg
        bound = max(m, self.max_tokens or 0)
        if x is None or x.max_slots < m * topk or x.topk != topk or x.hidden != H or x.out_dtype != dtype:
            self._xchg = x = _NvlinkExchange(self.group if self.group is not None else dist.group.WORLD, device, bound,
                                             topk, H, dtype, self.capacity_factor)
        return x

    def _forward_nvlink(self, x, topk_weights, topk_ids):
        from ..layers.moe.cutlass_moe import grouped_experts_prequantized
        m, H = x.shape
        topk = topk_ids.shape[1]
        xc = self._exchange(m, topk, H, x.dtype, x.device)
        ids = topk_ids.to(torch.int32).contiguous()
        if self.scale_ue8m0:
            # block-scaling path: power-of-two activation scales travel as packed exponent words (a quarter of the
            # fp32 scale bytes), weights carry power-of-two block scales
            from ..layers.moe.cutlass_moe import grouped_experts_prequantized_ue8m0
            from ..layers.quantization.fp8_kernel import per_token_group_quant_fp8_ue8m0_rows
            q, s = per_token_group_quant_fp8_ue8m0_rows(x)
            recv_q, recv_s, recv_ids = xc.dispatch(q, s, ids, self.e_local)
            c2, row_of = grouped_experts_prequantized_ue8m0(recv_q, recv_s, recv_ids, self.w13, self.w2, self.w13_scale,
                                                            self.w2_scale, x.dtype, return_sorted=True)
        else:
            q, s = self._quant(x)                                        # quantise once per token
            recv_q, recv_s, recv_ids = xc.dispatch(q, s.contiguous(), ids, self.e_local)
            c2, row_of = grouped_experts_prequantized(recv_q, recv_s, recv_ids, self.w13, self.w2, self.w13_scale,
                                                      self.w2_scale, x.dtype, return_sorted=True)
        back = xc.combine(c2, row_of)
        return self._wsum(back[:m * topk], xc.identity[:m * topk], topk_weights.to(x.dtype).contiguous(), m)

    def check(self) -> None:
        """Synchronises and raises if a receive region overflowed or a wait for a peer gave up on this rank."""
        if self._xchg is None:
            return
        code = int(self._xchg.status.item())
        if code != 0:
            self._xchg.status.zero_()
            from .. import _lib
            what = "a receive region overflowed: raise capacity_factor" if code == 31 else "a wait for a peer rank gave up"
            raise _lib.B200Error("expert-parallel exchange", -10 if code != 31 else -9, f"{what} (code {code})")

    # ------------------------------------------------------------------ nccl / gloo backend
    def _forward_a2a(self, x, topk_weights, topk_ids):
        m, H = x.shape
        topk = topk_ids.shape[1]
        p, dev = self.world, x.device
        q, s = self._quant(x)                                            # quantise once per token
        flat_ids = topk_ids.reshape(-1).to(torch.int64)
        dest = torch.div(flat_ids, self.e_local, rounding_mode="floor")
        order = torch.argsort(dest, stable=True)                          # send order: by destination rank
        send_counts = torch.bincount(dest, minlength=p).to(torch.int64)
        recv_counts = torch.empty_like(send_counts)
        if p > 1:
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        else:
            recv_counts.copy_(send_counts)
        send_split, recv_split = send_counts.tolist(), recv_counts.tolist()   # the one host sync
        n_recv = int(sum(recv_split))
        tok = torch.div(order, topk, rounding_mode="floor")
        send_q = q.view(torch.uint8)[tok].contiguous()
        send_s = s.contiguous()[tok].contiguous()
        send_e = (flat_ids[order] - dest[order] * self.e_local).to(torch.int32).contiguous()
        recv_q = torch.empty((n_recv, H), dtype=torch.uint8, device=dev)
        recv_s = torch.empty((n_recv, s.shape[1]), dtype=torch.float32, device=dev)
        recv_e = torch.empty((n_recv,), dtype=torch.int32, device=dev)
        if p > 1:
            dist.all_to_all_single(recv_q, send_q, recv_split, send_split, group=self.group)
            dist.all_to_all_single(recv_s, send_s, recv_split, send_split, group=self.group)
            dist.all_to_all_single(recv_e, send_e, recv_split, send_split, group=self.group)
        else:
            recv_q, recv_s, recv_e = send_q, send_s, send_e
        y = self._local(recv_q.view(torch.float8_e4m3fn), recv_s, recv_e, self.w13, self.w2, self.w13_scale,
                        self.w2_scale, x.dtype)
        back = torch.empty((order.numel(), H), dtype=x.dtype, device=dev)
        if p > 1:
            dist.all_to_all_single(back, y.contiguous(), send_split, recv_split, group=self.group)
        else:
            back = y
        # back[i] belongs to flat slot order[i]; the weighted sum reads slot f at row inv[f]
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=dev)
        return self._wsum(back, inv.to(torch.int32), topk_weights.to(x.dtype).contiguous(), m)

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        if self.backend == "nvlink":
            return self._forward_nvlink(x, topk_weights, topk_ids)
        return self._forward_a2a(x, topk_weights, topk_ids)

    __call__ = forward
