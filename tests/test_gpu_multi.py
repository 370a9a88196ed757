"""GPU, 2 ranks over NCCL (skipped on a single-GPU box): tensor-parallel linears and the
expert-parallel MoE against the single-GPU result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import block_fp8_oracle as O

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _tp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from sglang_b200.distributed import ColumnParallelBlockFp8Linear, RowParallelBlockFp8Linear
        from sglang_b200.layers.quantization.fp8_utils import w8a8_block_fp8_linear
        M, K, N = 200, 1024, 512
        x = O.gen_activation(M, K, seed=1).cuda()
        wq, ws = O.gen_weight(N, K, seed=2)
        wq, ws = wq.cuda(), ws.cuda()
        full = w8a8_block_fp8_linear(x, wq, [128, 128], ws)
        y_col = ColumnParallelBlockFp8Linear(wq, ws)(x)
        parts = [torch.empty_like(y_col) for _ in range(world)]
        dist.all_gather(parts, y_col)
        kp = K // world
        y_row = RowParallelBlockFp8Linear(wq, ws)(x[:, rank * kp:(rank + 1) * kp].contiguous())
        torch.cuda.synchronize()
        if rank == 0:
            q.put((bool(torch.equal(torch.cat(parts, 1), full)),
                   O.rel_l2(y_row.float().cpu(), full.float().cpu())))
    finally:
        dist.destroy_process_group()


def _ep_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from sglang_b200.distributed import ExpertParallelBlockFp8MoE
        from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
        E, H, I, m_per, topk = 8, 512, 256, 40, 2
        g = torch.Generator().manual_seed(3)
        w13q, w13s, w2q, w2s = [], [], [], []
        for _ in range(E):
            a_, b_ = O.per_block_cast_to_fp8(torch.randn(2 * I, H, generator=g) * 0.05); w13q.append(a_); w13s.append(b_)
            a_, b_ = O.per_block_cast_to_fp8(torch.randn(H, I, generator=g) * 0.05); w2q.append(a_); w2s.append(b_)
        w13q, w13s, w2q, w2s = [torch.stack(v).cuda() for v in (w13q, w13s, w2q, w2s)]
        x = (torch.randn(world * m_per, H, generator=g) / 4).to(torch.bfloat16).cuda()
        w, ids = O.fused_topk_native(torch.randn(world * m_per, E, generator=g), topk)
        w, ids = w.cuda(), ids.cuda()
        ref = fused_experts_block_fp8(x, w13q, w2q, w13s, w2s, w, ids)
        el = E // world
        sl = slice(rank * el, (rank + 1) * el)
        rows = slice(rank * m_per, (rank + 1) * m_per)
        results = {}
        for backend in ("nvlink", "nccl"):
            moe = ExpertParallelBlockFp8MoE(w13q[sl].contiguous(), w2q[sl].contiguous(), w13s[sl].contiguous(),
                                            w2s[sl].contiguous(), backend=backend)
            for it in range(2):          # the second call reuses the exchange buffers and barrier flags
                y = moe(x[rows].contiguous(), w[rows].contiguous(), ids[rows].contiguous())
                parts = [torch.empty_like(y) for _ in range(world)]
                dist.all_gather(parts, y)
                torch.cuda.synchronize()
                moe.check()
                results[f"{backend}_{it}"] = bool(torch.equal(torch.cat(parts, 0), ref))
        # a routing that sends every row to rank 0's experts: with capacity = tokens * topk nothing may be dropped
        moe = ExpertParallelBlockFp8MoE(w13q[sl].contiguous(), w2q[sl].contiguous(), w13s[sl].contiguous(),
                                        w2s[sl].contiguous(), backend="nvlink", capacity_factor=float(world))
        ids0 = (ids % el).contiguous()
        ref0 = fused_experts_block_fp8(x, w13q, w2q, w13s, w2s, w, ids0)
        y = moe(x[rows].contiguous(), w[rows].contiguous(), ids0[rows].contiguous())
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y)
        torch.cuda.synchronize()
        moe.check()
        results["all_to_rank0"] = bool(torch.equal(torch.cat(parts, 0), ref0))
        # the block-scaling path: power-of-two weight scales, activations dispatched with packed exponent words
        from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8_ue8m0
        g2 = torch.Generator().manual_seed(33)
        p13q, p13s, p2q, p2s = [], [], [], []
        for _ in range(E):
            a_, b_ = O.per_block_quant_mxfp8(torch.randn(2 * I, H, generator=g2) * 0.05); p13q.append(a_); p13s.append(b_)
            a_, b_ = O.per_block_quant_mxfp8(torch.randn(H, I, generator=g2) * 0.05); p2q.append(a_); p2s.append(b_)
        p13q, p13s, p2q, p2s = [torch.stack(v).cuda() for v in (p13q, p13s, p2q, p2s)]
        refp = fused_experts_block_fp8_ue8m0(x, p13q, p2q, p13s, p2s, w, ids)
        moe = ExpertParallelBlockFp8MoE(p13q[sl].contiguous(), p2q[sl].contiguous(), p13s[sl].contiguous(),
                                        p2s[sl].contiguous(), backend="nvlink", scale_ue8m0=True)
        for it in range(2):
            y = moe(x[rows].contiguous(), w[rows].contiguous(), ids[rows].contiguous())
            parts = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(parts, y)
            torch.cuda.synchronize()
            moe.check()
            results[f"nvlink_ue8m0_{it}"] = bool(torch.equal(torch.cat(parts, 0), refp))
        if rank == 0:
            q.put(results)
    finally:
        dist.destroy_process_group()


def _ar_worker(rank, world, port, q):
    """The library's own all-reduce kernels: two-shot in place (multicast when the machine offers it, and the
    peer-pointer form), one-shot, whole buffers and a row slice; every element must be the fp32 sum rounded once,
    identical on both ranks, and later calls must work on the same flags."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from sglang_b200.distributed.custom_all_reduce import SymmetricAllReduce
        results = {}
        for use_mc in (True, False):
            ar = SymmetricAllReduce(8 << 20, use_multicast=use_mc)
            results[f"multicast_{use_mc}"] = ar.multicast
            results[f"info_{use_mc}"] = f"tensor offset in allocation {ar.base_offset}"
            for it, (rows, cols, dtype) in enumerate([(512, 7168, torch.bfloat16), (48, 1024, torch.float16),
                                                       (512, 7168, torch.bfloat16)]):
                g = torch.Generator(device="cuda").manual_seed(100 * it + rank)
                mine = torch.randn(rows, cols, generator=g, device="cuda").to(dtype)
                parts = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(parts, mine)
                want = sum(p_.float() for p_ in parts).to(dtype)
                buf = ar.buffer((rows, cols), dtype)
                buf.copy_(mine)
                got2 = ar.all_reduce_(buf).clone()
                buf.copy_(mine)
                torch.cuda.synchronize(); dist.barrier()
                got1 = ar.all_reduce_small(buf[:16])     # one-shot over the first rows
                # a row slice in the middle of the buffer (what the chunked row-parallel linear reduces)
                buf.copy_(mine)
                torch.cuda.synchronize(); dist.barrier()
                ar.all_reduce_(buf[rows // 2:])
                got_half = buf[rows // 2:].clone()
                untouched = torch.equal(buf[:rows // 2], mine[:rows // 2])
                ar.check()
                key = f"mc{int(use_mc)}_{it}"
                # peer-pointer form: the fp32 sum rounded to nearest, bit for bit.  Multicast form: the switch adds in
                # fp32 but rounds the result its own way (results one unit in the last place away from
                # round-to-nearest occur), so: within one ulp of the input type, and the SAME bits on every rank.
                def same(a_, b_):
                    if not use_mc:
                        return bool(torch.equal(a_, b_))
                    ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
                    return bool(((a_.float() - b_.float()).abs() <= ulp * b_.float().abs() + 1e-6).all())
                both = [torch.empty_like(got2) for _ in range(world)]
                dist.all_gather(both, got2)
                results[key] = (same(got2, want), same(got1, want[:16]), same(got_half, want[rows // 2:]),
                                bool(untouched) and bool(torch.equal(both[0], both[1])))
                if not all(results[key]):
                    results["detail_" + key] = (f"two-shot max|diff| {(got2.float() - want.float()).abs().max().item():.4g}, "
                                                f"equals own input: {bool(torch.equal(got2, mine))}, one-shot max|diff| "
                                                f"{(got1.float() - want[:16].float()).abs().max().item():.4g}, "
                                                f"ranks agree: {bool(torch.equal(both[0], both[1]))}")
            if use_mc and ar.multicast:
                # autotune keeps one of the two forms (the same on every rank) and the buffer still reduces right
                times = ar.autotune(4 << 20, iters=3)
                picked = "multicast" if ar.multicast else "peer"
                g = torch.Generator(device="cuda").manual_seed(900 + rank)
                mine = torch.randn(256, 4096, generator=g, device="cuda").to(torch.bfloat16)
                parts = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(parts, mine)
                want = sum(p_.float() for p_ in parts).to(torch.bfloat16)
                buf = ar.buffer((256, 4096), torch.bfloat16)
                buf.copy_(mine)
                torch.cuda.synchronize(); dist.barrier()
                got = ar.all_reduce_(buf).clone()
                ar.check()
                close = bool(((got.float() - want.float()).abs() <= 2.0 ** -7 * want.float().abs() + 1e-6).all())
                results["autotune"] = (sorted(times) == ["multicast", "peer"], picked == min(times, key=times.get), close)
            del ar
        gathered = [None] * world
        dist.all_gather_object(gathered, results)
        if rank == 0:
            q.put(gathered)
    finally:
        dist.destroy_process_group()


def _tp_custom_worker(rank, world, port, q):
    """Row-parallel linear with the custom all-reduce, whole and in overlapped row chunks, against the
    unsharded linear; NCCL-reduced overlapped chunks against NCCL unchunked (bias on rank 0 only)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from sglang_b200.distributed import RowParallelBlockFp8Linear
        from sglang_b200.distributed.custom_all_reduce import SymmetricAllReduce
        from sglang_b200.layers.quantization.fp8_utils import w8a8_block_fp8_linear
        M, K, N = 640, 2048, 1024
        x = O.gen_activation(M, K, seed=11).cuda()
        wq, ws = O.gen_weight(N, K, seed=12)
        wq, ws = wq.cuda(), ws.cuda()
        bias = torch.randn(N, generator=torch.Generator().manual_seed(13)).to(torch.bfloat16).cuda()
        full = w8a8_block_fp8_linear(x, wq, [128, 128], ws, bias=bias)
        kp = K // world
        xs = x[:, rank * kp:(rank + 1) * kp].contiguous()
        ar = SymmetricAllReduce(M * N * 2)
        y_nccl = RowParallelBlockFp8Linear(wq, ws, bias)(xs).clone()
        y_nccl_chunked = RowParallelBlockFp8Linear(wq, ws, bias, overlap_chunks=2)(xs).clone()
        y_custom = RowParallelBlockFp8Linear(wq, ws, bias, all_reduce=ar)(xs).clone()
        y_custom_chunked = RowParallelBlockFp8Linear(wq, ws, bias, all_reduce=ar, overlap_chunks=2)(xs).clone()
        # chunks with SMs reserved for the collective: GEMMs on the remaining SMs, multicast all-reduce beside them;
        # the limit and the all-reduce's form must be back to what they were afterwards
        from sglang_b200 import _lib
        form_before = ar.multicast
        y_reserved = RowParallelBlockFp8Linear(wq, ws, bias, all_reduce=ar, overlap_chunks=2, reserve_sms=16)(xs).clone()
        limit_after = _lib.lib().b200_set_sm_limit(0)
        torch.cuda.synchronize()
        ar.check()
        ulp_ok = bool(((y_reserved.float() - y_custom.float()).abs() <= 2.0 ** -7 * y_custom.float().abs() + 1e-6).all())
        both = [torch.empty_like(y_custom) for _ in range(world)]
        dist.all_gather(both, y_custom)
        both_r = [torch.empty_like(y_reserved) for _ in range(world)]
        dist.all_gather(both_r, y_reserved)
        if rank == 0:
            q.put({"nccl_chunked_equal": bool(torch.equal(y_nccl, y_nccl_chunked)),
                   "reserved_ok": ulp_ok and bool(torch.equal(both_r[0], both_r[1])) and limit_after == 0
                                  and ar.multicast == form_before,
                   "custom_chunked_equal": bool(torch.equal(y_custom, y_custom_chunked)),
                   "custom_same_on_ranks": bool(torch.equal(both[0], both[1])),
                   "custom_err": O.rel_l2(y_custom.float().cpu(), full.float().cpu()),
                   "nccl_err": O.rel_l2(y_nccl.float().cpu(), full.float().cpu())})
    finally:
        dist.destroy_process_group()


def _run(worker, world=2, timeout=240):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(timeout)
        codes = [p.exitcode for p in procs]
        assert all(c == 0 for c in codes), f"rank exit codes {codes} (None = still running after {timeout} s)"
        return q.get(timeout=30)
    finally:
        # never leave a rank behind holding a GPU: a stalled collective or kernel ends here
        for p in procs:
            if p.exitcode is None:
                p.terminate()
                p.join(10)
            if p.exitcode is None:
                p.kill()
                p.join(10)


needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


@needs2
def test_tp2_nccl():
    col_equal, row_err = _run(_tp_worker)
    assert col_equal                      # column-parallel: the same columns, bit for bit
    assert row_err < 1e-2                 # row-parallel: bf16 partials summed in bf16


@needs2
def test_allreduce_kernels_2gpu():
    per_rank = _run(_ar_worker)
    for res in per_rank:
        assert res["multicast_False"] is False
        assert res.get("autotune", (True, True, True)) == (True, True, True), res.get("autotune")
        bad = {k: v for k, v in res.items() if k.startswith("mc") and v != (True, True, True, True)}
        assert not bad, {k: v for k, v in res.items() if not (k.startswith("mc") and k not in bad)}


@needs2
def test_tp2_custom_all_reduce_and_overlapped_chunks():
    r = _run(_tp_custom_worker)
    assert r["nccl_chunked_equal"] and r["custom_chunked_equal"] and r["custom_same_on_ranks"] and r["reserved_ok"], r
    # two bf16 partial outputs summed: each carries its own rounding (about 2^-9 relative)
    assert r["custom_err"] < 5e-3 and r["nccl_err"] < 5e-3, r


@needs2
def test_ep2_bitwise_both_exchanges():
    """Expert-parallel layer on 2 ranks, NVLink dispatch/combine kernels and the NCCL all-to-all form, each
    twice, plus a skewed routing at full capacity: bit for bit the single-GPU fused layer."""
    res = _run(_ep_worker)
    assert all(res.values()), res
