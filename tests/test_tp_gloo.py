"""CPU, world_size 2, gloo: tensor-parallel sharding and the row-parallel all-reduce.
The local linear is the CPU oracle here (the product has no CPU path); what is under test is
the shard arithmetic, bias placement and the collective."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import block_fp8_oracle as O


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _oracle_linear(x, w, ws, bias):
    return O.block_fp8_linear(x, w, ws, bias=bias, out_dtype=torch.bfloat16)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sglang_b200.distributed import ColumnParallelBlockFp8Linear, RowParallelBlockFp8Linear
        M, K, N = 24, 512, 256
        x = O.gen_activation(M, K, seed=1)
        wq, ws = O.gen_weight(N, K, seed=2)
        bias = torch.randn(N, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
        col = ColumnParallelBlockFp8Linear(wq, ws, bias=bias, linear_fn=_oracle_linear)
        y_col = col(x)
        gathered = [torch.empty_like(y_col) for _ in range(world)]
        dist.all_gather(gathered, y_col)
        row = RowParallelBlockFp8Linear(wq, ws, bias=bias, linear_fn=_oracle_linear)
        kp = K // world
        y_row = row(x[:, rank * kp:(rank + 1) * kp].contiguous())
        if rank == 0:
            q.put((torch.cat(gathered, 1).float(), y_row.float()))
    finally:
        dist.destroy_process_group()


def test_tp2_matches_single_rank():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs: p.start()
    y_col, y_row = q.get()
    for p in procs:
        p.join(120); assert p.exitcode == 0
    M, K, N = 24, 512, 256
    x = O.gen_activation(M, K, seed=1)
    wq, ws = O.gen_weight(N, K, seed=2)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    full = O.block_fp8_linear(x, wq, ws, bias=bias).float()
    assert torch.equal(y_col, full)                       # column-parallel: bitwise the same columns
    assert O.rel_l2(y_row, full) < 1e-2                    # row-parallel: bf16 partials summed in bf16


def test_shard_rules():
    from sglang_b200.distributed import shard_block_fp8_weight
    wq, ws = O.gen_weight(512, 1024, seed=5)
    w1, s1 = shard_block_fp8_weight(wq, ws, 0, 1, 2)
    assert w1.shape == (256, 1024) and s1.shape == (2, 8)
    assert torch.equal(w1.view(torch.uint8), wq[256:].view(torch.uint8)) and torch.equal(s1, ws[2:])
    w2, s2 = shard_block_fp8_weight(wq, ws, 1, 3, 4)
    assert w2.shape == (512, 256) and s2.shape == (4, 2) and torch.equal(s2, ws[:, 6:8])
    with pytest.raises(ValueError, match="quantization block"):
        shard_block_fp8_weight(wq, ws, 0, 0, 8)           # 64 rows per rank: not a multiple of 128
    with pytest.raises(ValueError, match="divisible by tp size"):
        shard_block_fp8_weight(wq, ws, 0, 0, 3)
