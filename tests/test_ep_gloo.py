"""CPU, world_size 2, gloo: expert-parallel dispatch / combine.  The quantiser, the local expert
computation and the weighted sum are the CPU oracle here (the product has no CPU path); under test
are the routing of rows to the ranks that own their experts, the split sizes, the order in which
rows come back and the final weighted sum -- checked against the single-rank oracle MoE."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import block_fp8_oracle as O

E, H, I, M_PER_RANK, TOPK = 8, 256, 128, 11, 2


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _make(seed=0):
    g = torch.Generator().manual_seed(seed)
    w13q, w13s, w2q, w2s = [], [], [], []
    for _ in range(E):
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(2 * I, H, generator=g) * 0.05); w13q.append(q_); w13s.append(s_)
        q_, s_ = O.per_block_cast_to_fp8(torch.randn(H, I, generator=g) * 0.05); w2q.append(q_); w2s.append(s_)
    x = (torch.randn(2 * M_PER_RANK, H, generator=g) / 4).to(torch.bfloat16)
    w, ids = O.fused_topk_native(torch.randn(2 * M_PER_RANK, E, generator=g), TOPK)
    return x, w, ids, torch.stack(w13q), torch.stack(w13s), torch.stack(w2q), torch.stack(w2s)


def _oracle_local(a_q, a_s, ids, w13, w2, w13_s, w2_s, out_dtype):
    out = torch.zeros((a_q.shape[0], a_q.shape[1]), dtype=out_dtype)
    for e in range(w13.shape[0]):
        rows = (ids == e).nonzero().flatten()
        if rows.numel():
            c1 = O.block_fp8_matmul_fp32(a_q[rows], w13[e], a_s[rows], w13_s[e]).to(out_dtype)
            iq, isc = O.quant_group_fp8_cuda_semantics(O.silu_and_mul(c1), 128)
            out[rows] = O.block_fp8_matmul_fp32(iq, w2[e], isc, w2_s[e]).to(out_dtype)
    return out


def _oracle_wsum(rows, perm, weights, m):
    return O.apply_shuffle_mul_sum(rows, perm, weights, m)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sglang_b200.distributed import ExpertParallelBlockFp8MoE
        x, w, ids, w13q, w13s, w2q, w2s = _make()
        el = E // world
        sl = slice(rank * el, (rank + 1) * el)
        moe = ExpertParallelBlockFp8MoE(w13q[sl], w2q[sl], w13s[sl], w2s[sl],
                                        quant_fn=lambda t: O.quant_group_fp8_cuda_semantics(t, 128),
                                        local_fn=_oracle_local, weighted_sum_fn=_oracle_wsum)
        rows = slice(rank * M_PER_RANK, (rank + 1) * M_PER_RANK)
        y = moe(x[rows].contiguous(), w[rows].contiguous(), ids[rows].contiguous())
        gathered = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        if rank == 0:
            q.put(torch.cat(gathered, 0).float())
    finally:
        dist.destroy_process_group()


def test_ep2_matches_single_rank_bitwise():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs: p.start()
    y = q.get()
    for p in procs:
        p.join(120); assert p.exitcode == 0
    x, w, ids, w13q, w13s, w2q, w2s = _make()
    ref = O.cutlass_fused_experts_fp8(x, w13q, w2q, w13s, w2s, w, ids).float()
    assert torch.equal(y, ref)      # rows are independent and the weighted sum keeps its order
