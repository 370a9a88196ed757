"""GPU: the allocation-free routing-table entry point gives exactly what the regular one gives.

`b200_moe_prepare_noalloc` is for callers that cannot get device memory at that point (a server
whose pool owns the whole GPU, a section where allocator calls are not permitted): its work table is an array built into
the library instead of scratch supplied by the caller.  Both entry points are called through the
C ABI, twice in a row with different routings, so the second call runs on a table that still holds
the first call's numbers.  This file sorts last on purpose: a run that stops at the first failure
has already run every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(entry, ids, E, n, k, scratch=None):
    from sglang_b200 import _lib
    L = _lib.lib()
    m, topk = ids.shape
    d = dict(dtype=torch.int32, device="cuda")
    offs, bs_offs = torch.full((E + 1,), -3, **d), torch.full((E + 1,), -3, **d)
    ps1, ps2 = torch.full((E, 3), -3, **d), torch.full((E, 3), -3, **d)
    a_map, c_map = torch.full((m * topk,), -3, **d), torch.full((m * topk,), -3, **d)
    stream = torch.cuda.current_stream().cuda_stream
    if entry == "regular":
        rc = L.b200_moe_prepare(ids.data_ptr(), m, topk, E, n, k, offs.data_ptr(), bs_offs.data_ptr(), ps1.data_ptr(),
                                ps2.data_ptr(), a_map.data_ptr(), c_map.data_ptr(), scratch.data_ptr(),
                                scratch.numel(), stream)
    else:
        rc = L.b200_moe_prepare_noalloc(ids.data_ptr(), m, topk, E, n, k, offs.data_ptr(), bs_offs.data_ptr(),
                                        ps1.data_ptr(), ps2.data_ptr(), a_map.data_ptr(), c_map.data_ptr(), stream)
    _lib.check(entry, rc)
    torch.cuda.synchronize()
    total = int(offs[-1])
    return offs, bs_offs, ps1, ps2, a_map[:total], c_map


def test_noalloc_matches_regular_twice_in_a_row():
    from sglang_b200 import _lib
    E, n, k = 256, 2048, 7168
    for call, (m, topk, seed) in enumerate([(4096, 8, 0), (777, 6, 1)]):
        g = torch.Generator().manual_seed(seed)
        ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(m)]).to(torch.int32)
        ids[3, 1] = -1                                        # one masked id
        ids = ids.cuda()
        nbytes = _lib.lib().b200_moe_prepare_scratch_bytes(m * topk, E)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        ref = _run("regular", ids, E, n, k, scratch)
        got = _run("noalloc", ids, E, n, k)
        for name, r, o in zip(("expert_offsets", "blockscale_offsets", "problem_sizes1", "problem_sizes2",
                               "input_permutation", "output_permutation"), ref, got):
            assert torch.equal(r, o), f"call {call}: {name} differs"


def test_noalloc_rejects_sizes_beyond_its_table():
    from sglang_b200 import _lib
    L = _lib.lib()
    # 2048 chunks x 64 experts = 131072 table entries > 65536: refused on the host, nothing is launched
    rc = L.b200_moe_prepare_noalloc(16, 2048 * 2048, 1, 64, 8, 8, 16, None, 16, 16, 16, 16, None)
    assert rc == -9
    assert b"exceeds" in L.b200_strerror(rc)
