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
        moe = ExpertParallelBlockFp8MoE(w13q[sl].contiguous(), w2q[sl].contiguous(), w13s[sl].contiguous(),
                                        w2s[sl].contiguous())
        y = moe(x[rows].contiguous(), w[rows].contiguous(), ids[rows].contiguous())
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y)
        torch.cuda.synchronize()
        if rank == 0:
            q.put(bool(torch.equal(torch.cat(parts, 0), ref)))
    finally:
        dist.destroy_process_group()


def _run(worker):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs: p.start()
    for p in procs:
        p.join(180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    return q.get()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_nccl():
    col_equal, row_err = _run(_tp_worker)
    assert col_equal                      # column-parallel: the same columns, bit for bit
    assert row_err < 1e-2                 # row-parallel: bf16 partials summed in bf16


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep2_nccl_bitwise():
    assert _run(_ep_worker)
