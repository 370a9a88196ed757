"""Benchmark of the W8A8 block-FP8 linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (config.workload): the DeepSeek-V3-shaped dense MLP as two block-FP8 linears at
M = 4096 tokens -- gate_up (K=7168, N=36864) then down (K=18432, N=7168).  One step =
group-quantise x, GEMM, group-quantise h, GEMM (4 kernels).  Inputs are seeded synthetic
tensors (activations N(0,1), weights N(0,0.02) block-quantised); weights (396 MB of e4m3) and
activations (210 MB of bf16) exceed the 126 MB L2, so no explicit flush is needed.

N > 1 (launched by torchrun, one rank per GPU, NCCL): the same MLP tensor-parallel as in the
reference -- gate_up column-parallel (N/p per rank, no communication), down row-parallel
(K/p per rank) followed by one bf16 all-reduce of [4096,7168].  Total work is fixed: strong scaling.

The JSON line carries: value = whole-job TFLOP/s with inputs resident in HBM; e2e = the same
through the public linear call with HOST activations (pinned) copied in and the bf16 results
copied out inside the timed region; roofline for the dominant kernel (the gate_up GEMM) from
CUDA events placed around its launches inside the timed region; cpu_baseline = the reference's
own CPU block-FP8 matmul (oracle/_ref, built from the reference sources) or, where the host
lacks AMX, the torch restatement, timed on the host cores on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M_TOKENS = 4096
HIDDEN = 7168
INTER2 = 36864      # gate_up output (2 x 18432)
INTER = 18432
WORKLOAD = "deepseek_v3_dense_mlp_block_fp8_M4096(gate_up K7168 N36864 + down K18432 N7168)"
FLOPS_PER_STEP = 2.0 * M_TOKENS * (INTER2 * HIDDEN + HIDDEN * INTER)
NOMINAL_FP8_TFLOPS = 4500.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the gate_up GEMM at M=4096, from the ncu
# capture summarised in profiles/gemm_block_fp8_gate_up_M4096_dram.md (algorithmic bytes: 596.9e6)
GEMM_TRAFFIC_BYTES = 586.4e6


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_sustained": p["bf16_tflops_sustained"],
                "bf16_burst": p["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_sustained": 1400.0, "bf16_burst": 1590.0, "src": "fallback"}


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxc, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                clocks.append(float(f[1])); maxc.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load = upper half of the power readings
        order = sorted(range(len(clocks)), key=lambda i: power[i])
        load = [clocks[i] for i in order[len(order) // 2:]]
        load.sort()
        return {"sm_mhz": load[len(load) // 2], "sm_max_mhz": max(maxc), "power_w_max": max(power),
                "samples": len(clocks), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# CPU reference arm / baseline
# ------------------------------------------------------------------------------------------
def cpu_reference_run(steps: int, warmup: int, sample_rows: int = 64):
    """Times the reference CPU block-FP8 matmul on `sample_rows` tokens of the workload (both
    layers).  Returns (tflops, info dict)."""
    import torch

    from oracle import block_fp8_oracle as O
    from oracle import build_ref

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    layers = []
    for (n, k) in ((INTER2, HIDDEN), (HIDDEN, INTER)):
        # codes/scales drawn directly (quantising 264 MB on the host would dominate start-up);
        # distribution does not affect CPU matmul time
        wq = torch.randint(0, 120, (n, k), dtype=torch.uint8, generator=g).view(torch.float8_e4m3fn)
        ws = torch.rand((n // 128, k // 128), generator=g) * 1e-3 + 1e-4
        x = torch.randn((sample_rows, k), generator=g).to(torch.bfloat16)
        layers.append((x, wq, ws))
    kind = "port"
    if build_ref.load():
        kind = "reference"
        ops = torch.ops.sgl_kernel_ref
        packed = [(x, ops.convert_weight_packed(wq), ws) for (x, wq, ws) in layers]

        def step():
            for (x, wp, ws) in packed:
                ops.fp8_scaled_mm_cpu(x, wp, ws, [128, 128], None, torch.bfloat16, True)
    else:
        quant = [(O.quant_group_fp8_cuda_semantics(x, 128), wq, ws) for (x, wq, ws) in layers]

        def step():
            for ((q, s), wq, ws) in quant:
                O.block_fp8_matmul_fp32(q, wq, s, ws).to(torch.bfloat16)
    for _ in range(max(1, warmup)):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    flops = 2.0 * sample_rows * (INTER2 * HIDDEN + HIDDEN * INTER)
    tflops = flops / dt / 1e12
    info = {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"{sample_rows} of {M_TOKENS} tokens through both layers, {steps} timed passes "
                      f"({dt * 1e3:.1f} ms each); "
                      + ("reference fp8_scaled_mm_cpu (W8A16, AMX), weights pre-packed" if kind == "reference"
                         else "torch restatement of native_w8a8_block_fp8_matmul")}
    return tflops, dt, info


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    # the full 4096-token workload takes about 1.6 s per pass on 8 AMX cores; shrink the sample
    # for long runs so the arm still ends within a few minutes
    rows = M_TOKENS if steps <= 30 else 512
    tflops, dt, info = cpu_reference_run(steps, min(args.warmup, 2), rows)
    line = {"impl": "reference", "metric": "block_fp8_linear_tflops", "value": tflops, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x e4m3 (W8A16)",
            "data": "synthetic", "config": {"workload": WORKLOAD, "sample": info["sample"]},
            "cpu_baseline": info,
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def gen_weight_device(n, k, seed, device):
    """N(0,0.02^2) weight block-quantised on the device (amax.clamp(1e-4)/448 per 128x128 block,
    the per_block_cast_to_fp8 recipe of sgl-kernel/tests/test_fp8_blockwise_moe.py:51-64)."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.empty((n, k), dtype=torch.float8_e4m3fn, device=device)
    s = torch.empty((n // 128, k // 128), dtype=torch.float32, device=device)
    rows = 2048
    for r0 in range(0, n, rows):
        r1 = min(n, r0 + rows)
        w = torch.randn((r1 - r0, k), generator=g, device=device) * 0.02
        wv = w.view((r1 - r0) // 128, 128, k // 128, 128)
        amax = wv.abs().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
        q[r0:r1] = (wv * (448.0 / amax)).to(torch.float8_e4m3fn).view(r1 - r0, k)
        s[r0 // 128:r1 // 128] = (amax / 448.0).view((r1 - r0) // 128, k // 128)
    return q, s


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from sglang_b200 import _lib
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    from sglang_b200.layers.quantization.fp8_utils import w8a8_block_fp8_linear
    from sglang_b200.sgl_kernel import fp8_blockwise_scaled_mm

    _lib.lib()  # fail loudly if the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch with torchrun for N>1)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    p = world
    n1, k2 = INTER2 // p, INTER // p        # column-parallel gate_up, row-parallel down

    w1q, w1s = gen_weight_device(n1, HIDDEN, 100 + rank, dev)
    w2q, w2s = gen_weight_device(HIDDEN, k2, 200 + rank, dev)
    w1_t, w1s_t, w2_t, w2s_t = w1q.T, w1s.T, w2q.T, w2s.T
    g = torch.Generator(device=dev).manual_seed(7)           # x is replicated: same seed on all ranks
    x = torch.randn((M_TOKENS, HIDDEN), generator=g, device=dev).to(torch.bfloat16)
    gh = torch.Generator(device=dev).manual_seed(300 + rank)
    h = torch.randn((M_TOKENS, k2), generator=gh, device=dev).to(torch.bfloat16)

    ev = lambda: torch.cuda.Event(enable_timing=True)
    kernel_events = []   # (name, start, stop) inside the timed region
    TP_CHUNKS = args.tp_chunks or 4
    y2_buf = torch.empty((M_TOKENS, HIDDEN), dtype=torch.bfloat16, device=dev)
    comm_stream = torch.cuda.Stream(device=dev) if world > 1 else None

    def step(record=False):
        def timed(name, fn):
            if not record:
                return fn()
            a, b = ev(), ev()
            a.record(); r = fn(); b.record()
            kernel_events.append((name, a, b))
            return r
        xq, xs = timed("quant_x", lambda: sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True))
        y1 = timed("gemm_gate_up", lambda: fp8_blockwise_scaled_mm(xq, w1_t, xs, w1s_t, torch.bfloat16))
        if world == 1:
            hq, hs = timed("quant_h", lambda: sglang_per_token_group_quant_fp8(h, 128, column_major_scales=True))
            y2 = timed("gemm_down", lambda: fp8_blockwise_scaled_mm(hq, w2_t, hs, w2s_t, torch.bfloat16))
        else:
            # row-parallel down projection in TP_CHUNKS row chunks: the bf16 all-reduce of chunk i runs on
            # a side stream while chunk i+1 is quantised and multiplied
            y2 = y2_buf
            main = torch.cuda.current_stream()
            rows = M_TOKENS // TP_CHUNKS
            for c in range(TP_CHUNKS):
                sl = slice(c * rows, (c + 1) * rows)
                hq, hs = sglang_per_token_group_quant_fp8(h[sl], 128, column_major_scales=True)
                fp8_blockwise_scaled_mm(hq, w2_t, hs, w2s_t, torch.bfloat16, out=y2[sl])
                ready = torch.cuda.Event()
                ready.record(main)
                with torch.cuda.stream(comm_stream):
                    comm_stream.wait_event(ready)
                    dist.all_reduce(y2[sl])
            main.wait_stream(comm_stream)
        return y1, y2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    # Tensor-parallel ranks replay the step from a CUDA graph (kernels, the side-stream fork/join and the
    # NCCL all-reduces captured once): a rank's share of the step is a few hundred microseconds of device
    # work, less than the Python calls that enqueue it.
    graph = None

    def capture_step():
        """The step captured into a CUDA graph on every rank, or None on every rank (the ranks agree)."""
        cap = torch.cuda.Stream(device=dev)
        cap.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cap):
            step()
        torch.cuda.current_stream().wait_stream(cap)
        barrier()
        # thread-local capture mode: the process group's watchdog thread polls events while this thread
        # captures.  Nothing executes during capture, so a rank whose capture fails can still agree with
        # the others (one small all-reduce afterwards) to run eagerly.
        captured = 1
        g_ = None
        try:
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_, stream=cap, capture_error_mode="thread_local"):
                step()
        except Exception as e:  # noqa: BLE001
            captured = 0
            g_ = None
            print(f"[bench rank {rank}] graph capture failed, running eagerly: {e}", file=sys.stderr, flush=True)
        torch.cuda.synchronize()
        flag = torch.tensor([captured], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            if g_ is not None:
                g_.reset()
            return None
        for _ in range(3):
            g_.replay()
            torch.cuda.synchronize()
        barrier()
        return g_

    if world > 1 and not args.eager:
        # How many row chunks the row-parallel projection is cut into is a trade between overlap (the
        # all-reduce of one chunk under the GEMM of the next) and the fixed cost of each collective; which
        # wins depends on the rank count.  With --tp-chunks 0 the warm-up measures the candidates (ten
        # replays each, slowest rank counts) and the timed region runs the fastest.
        candidates = [args.tp_chunks] if args.tp_chunks else [4, 2, 1]
        best = None
        chunk_ms = {}
        for c in candidates:
            TP_CHUNKS = c
            g_ = capture_step()
            if g_ is None:
                break
            if len(candidates) == 1:
                best = (0.0, c, g_)
                break
            a, b = ev(), ev()
            barrier()
            a.record()
            for _ in range(10):
                g_.replay()
            b.record()
            barrier()
            t = torch.tensor([a.elapsed_time(b)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t = float(t.item()) / 10
            chunk_ms[str(c)] = round(t, 4)
            if best is None or t < best[0]:
                if best is not None:
                    best[2].reset()
                best = (t, c, g_)
            else:
                g_.reset()
        if best is not None:
            _, TP_CHUNKS, graph = best
        else:
            TP_CHUNKS = args.tp_chunks or 4
        barrier()
    elif world > 1:
        TP_CHUNKS = args.tp_chunks or 4
        chunk_ms = {}
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- timed region 1: device-resident inputs
    t0, t1 = ev(), ev()
    barrier()
    t0.record()
    for _ in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            step(record=True)
    t1.record()
    barrier()
    ms = t0.elapsed_time(t1) / args.steps
    if graph is not None:
        # per-kernel times from a few eager steps (events cannot be timed inside a graph); the capture emptied
        # the allocator's cache, so two unrecorded steps first take the device allocations out of the figures
        for _ in range(2):
            step()
        barrier()
        for _ in range(5):
            step(record=True)
        barrier()
    per_kernel = {}
    for name, a, b in kernel_events:
        per_kernel.setdefault(name, []).append(a.elapsed_time(b))
    per_kernel = {k: sum(v) / len(v) for k, v in per_kernel.items()}

    # ---- timed region 2: end to end through the public linear call with host buffers.
    # Every step copies its activations in from pinned host memory and its results back; the three legs
    # (copy in, compute, copy out) of consecutive steps overlap on three streams with double buffers, so
    # the steady-state step costs the slowest leg (PCIe is full duplex) instead of their sum.
    DEPTH = 2
    x_host = x.cpu().pin_memory()
    h_host = h.cpu().pin_memory()
    y1_host = [torch.empty((M_TOKENS, n1), dtype=torch.bfloat16).pin_memory() for _ in range(DEPTH)]
    y2_host = [torch.empty((M_TOKENS, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(DEPTH)]
    x_dev = [torch.empty_like(x) for _ in range(DEPTH)]
    h_dev = [torch.empty_like(h) for _ in range(DEPTH)]
    s_in, s_comp, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
    ev_in = [torch.cuda.Event() for _ in range(DEPTH)]
    ev_comp = [torch.cuda.Event() for _ in range(DEPTH)]
    ev_out = [torch.cuda.Event() for _ in range(DEPTH)]
    step_no = [0]

    def e2e_step():
        i = step_no[0]
        step_no[0] += 1
        b = i % DEPTH
        with torch.cuda.stream(s_in):
            if i >= DEPTH:
                s_in.wait_event(ev_comp[b])          # the device input buffers of step i - DEPTH have been consumed
            x_dev[b].copy_(x_host, non_blocking=True)
            h_dev[b].copy_(h_host, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(ev_in[b])
            y1 = w8a8_block_fp8_linear(x_dev[b], w1q, [128, 128], w1s)
            y2 = w8a8_block_fp8_linear(h_dev[b], w2q, [128, 128], w2s)
            if world > 1:
                dist.all_reduce(y2)
            ev_comp[b].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])
            y1.record_stream(s_out)
            y2.record_stream(s_out)
            y1_host[b].copy_(y1, non_blocking=True)
            y2_host[b].copy_(y2, non_blocking=True)
            ev_out[b].record(s_out)

    def e2e_join():
        main = torch.cuda.current_stream()
        for st_ in (s_in, s_comp, s_out):
            main.wait_stream(st_)

    e2e_steps = max(4, min(args.steps, 10))
    for st_ in (s_in, s_comp, s_out):
        st_.wait_stream(torch.cuda.current_stream())
    for _ in range(2):
        e2e_step()
    e2e_join()
    barrier()
    step_no[0] = 0
    t2, t3 = ev(), ev()
    t2.record()
    for st_ in (s_in, s_comp, s_out):
        st_.wait_stream(torch.cuda.current_stream())
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()
    t3.record()
    barrier()
    e2e_ms = t2.elapsed_time(t3) / e2e_steps
    clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(times[0]), float(times[1])

    import ctypes
    st = ctypes.c_int(0)
    _lib.check("status", _lib.lib().b200_gemm_device_status(ctypes.byref(st)))
    assert st.value == 0, f"GEMM device status word {st.value}"

    if rank == 0:
        pk = _peaks()
        gemm_ms = per_kernel["gemm_gate_up"]
        gemm_flops = 2.0 * M_TOKENS * n1 * HIDDEN
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
        peak = 2.0 * pk["bf16_sustained"]
        quant_bytes = 3.03125 * M_TOKENS * HIDDEN
        quant_gbs = quant_bytes / (per_kernel["quant_x"] * 1e-3) / 1e9
        # our kernels per step: two quant launches (one per row chunk when tensor-parallel), the GEMMs, and one
        # small reduce launch after every GEMM whose last wave of tiles the library splits
        from sglang_b200.sgl_kernel.gemm import _splitk_plan
        split1 = _splitk_plan(M_TOKENS, n1, HIDDEN, dev)[0] > 1
        rows2 = M_TOKENS if world == 1 else M_TOKENS // TP_CHUNKS
        split2 = _splitk_plan(rows2, HIDDEN, k2, dev)[0] > 1
        chunks2 = 1 if world == 1 else TP_CHUNKS
        launches_per_step = (1 + 1 + int(split1)) + chunks2 * (1 + 1 + int(split2))
        h2d = x.numel() * 2 + h.numel() * 2
        d2h = y1_host[0].numel() * 2 + y2_host[0].numel() * 2
        line = {
            "metric": "block_fp8_linear_tflops", "value": FLOPS_PER_STEP / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 -> bf16",
            "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "parallelism": (f"tp{world}: gate_up column-parallel, down row-parallel in {TP_CHUNKS} row chunks "
                                       "with the bf16 NCCL all-reduce of each chunk overlapped"
                                       + ("; step replayed from a CUDA graph" if graph is not None else "")) if world > 1 else "single",
                       "l2": "inputs larger than L2 (weights 396 MB e4m3 + activations 210 MB bf16 per step)",
                       "kernels_ms": per_kernel,
                       **({"row_chunk_candidates_ms": chunk_ms} if world > 1 and chunk_ms else {})},
            "e2e": {"value": FLOPS_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "note": "every step copies its activations from pinned host memory and its bf16 results back; the "
                            "copy-in / compute / copy-out legs of consecutive steps overlap on three streams "
                            "(double buffers); weights stay resident (they are layer parameters)"},
            "gpu_launches": args.steps * launches_per_step,
            "roofline": {"bound": "tensor", "kernel": "gemm_block_fp8_kernel<BLOCK_N=256, 16 epilogue warps, 32-column chunks, bf16> (gate_up)",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": f"2 x bf16_tflops_sustained of {pk['src']} (the fp8 pipe does twice the "
                                        "bf16 MACs per clock; the file holds no fp8 entry)",
                         "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
                         "traffic": GEMM_TRAFFIC_BYTES, "algorithmic_flops_per_launch": gemm_flops},
            "quant": {"bound": "hbm", "kernel": "quant_group_kernel<bf16,128> on [4096,7168]",
                      "achieved": quant_gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": quant_gbs / pk["hbm_gbs"],
                      "algorithmic_bytes_per_launch": quant_bytes},
            "clocks": clocks,
        }
        if world == 1:
            _, _, info = cpu_reference_run(steps=5, warmup=1, sample_rows=M_TOKENS)
            line["cpu_baseline"] = info
        print(json.dumps(line))
        sys.stdout.flush()
    if world > 1:
        # release the captured graph before the communicator it references, and never let a slow
        # communicator teardown keep a finished benchmark alive
        if graph is not None:
            graph.reset()
            graph = None
        torch.cuda.synchronize()
        dist.barrier()
        guard = threading.Timer(20.0, lambda: os._exit(0))
        guard.daemon = True
        guard.start()
        dist.destroy_process_group()
        guard.cancel()


def run_kernel_case(args):
    """One kernel alone on one GPU (used for the M sweeps and as the small case for ncu captures):
    --kernel gemm_gate_up|gemm_down|quant --m M.  Prints one JSON line per case."""
    import torch

    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    from sglang_b200.sgl_kernel import fp8_blockwise_scaled_mm

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pk = _peaks()
    ms_list = [int(v) for v in str(args.m).split(",")]
    for m in ms_list:
        g = torch.Generator(device=dev).manual_seed(m)
        if args.kernel == "moe":
            # DeepSeek-V3 MoE layer on one GPU: 256 experts, top-8, hidden 7168, intermediate 2048.
            # Codes and scales are drawn directly (11.3 GB of weights); parity is covered by the tests.
            from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
            E, H, I, topk = args.experts, 7168, 2048, 8
            def codes(*shape):
                c = torch.randint(0, 0x78, shape, generator=g, device=dev, dtype=torch.uint8)
                sign = torch.randint(0, 2, shape, generator=g, device=dev, dtype=torch.uint8) << 7
                return (c | sign).view(torch.float8_e4m3fn)
            w13 = torch.empty((E, 2 * I, H), dtype=torch.float8_e4m3fn, device=dev)
            w2 = torch.empty((E, H, I), dtype=torch.float8_e4m3fn, device=dev)
            for e in range(E):
                w13[e] = codes(2 * I, H)
                w2[e] = codes(H, I)
            w13s = torch.rand((E, 2 * I // 128, H // 128), generator=g, device=dev) * 2e-4 + 1e-5
            w2s = torch.rand((E, H // 128, I // 128), generator=g, device=dev) * 2e-4 + 1e-5
            x = torch.randn((m, H), generator=g, device=dev).to(torch.bfloat16)
            logits = torch.randn((m, E), generator=g, device=dev)
            tw, ti = torch.topk(torch.softmax(logits.float(), dim=-1), topk, dim=-1)
            ti = ti.to(torch.int32)

            def fn():
                return fused_experts_block_fp8(x, w13, w2, w13s, w2s, tw, ti)
            work, unit, peak = 2.0 * m * topk * (2 * I * H + H * I) / 1e12, "TFLOP/s", 2.0 * pk["bf16_sustained"]
        elif args.kernel == "quant":
            nbuf = max(2, min(8, int(300e6 // (m * HIDDEN * 2)) + 1))   # rotate buffers: > L2 in total
            xs = []
            for _ in range(nbuf):
                x = torch.randn((m, HIDDEN), generator=g, device=dev)
                x = torch.where(torch.rand((m, HIDDEN), generator=g, device=dev) < 1e-3, x * 100, x)
                xs.append(x.to(torch.bfloat16))
            it = [0]

            def fn():
                it[0] += 1
                return sglang_per_token_group_quant_fp8(xs[it[0] % nbuf], 128, column_major_scales=True,
                                                        scale_tma_aligned=True)
            work, unit, peak = 3.03125 * m * HIDDEN / 1e9, "GB/s", pk["hbm_gbs"]
        else:
            if args.kernel == "gemm":   # e.g. the Llama-3-70B tensor-parallel shard shapes (N/p or K/p)
                assert args.n > 0 and args.k > 0 and args.n % 128 == 0 and args.k % 128 == 0, "--n/--k: multiples of 128"
                n, k = args.n, args.k
            else:
                n, k = (INTER2, HIDDEN) if args.kernel == "gemm_gate_up" else (HIDDEN, INTER)
            # small batches are weight-streaming: rotate through enough weight copies (> 2x L2) that no
            # call finds its weights in L2
            ncopy = 1 if m > 512 else max(2, int(300e6 // (n * k)) + 1)
            copies = [gen_weight_device(n, k, 1 + c, dev) for c in range(ncopy)]
            x = torch.randn((m, k), generator=g, device=dev).to(torch.bfloat16)
            xq, xs_ = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True)
            views = [(wq.T, ws.T) for wq, ws in copies]
            it = [0]

            def fn():
                it[0] += 1
                w_t, ws_t = views[it[0] % ncopy]
                return fp8_blockwise_scaled_mm(xq, w_t, xs_, ws_t, torch.bfloat16)
            work, unit, peak = 2.0 * m * n * k / 1e12, "TFLOP/s", 2.0 * pk["bf16_sustained"]
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.graph:
            # the launches of all timed steps captured once and replayed: device time without the
            # Python call overhead (a decode loop runs this way)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()                                   # per-stream workspace allocated before capture
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(args.steps):
                    fn()
            graph.replay()
            torch.cuda.synchronize()
            a.record()
            graph.replay()
            b.record()
        else:
            a.record()
            for _ in range(args.steps):
                fn()
            b.record()
        torch.cuda.synchronize()
        sec = a.elapsed_time(b) / args.steps * 1e-3
        rec = {"kernel": args.kernel if args.kernel != "gemm" else f"gemm N={args.n} K={args.k}", "M": m,
               "us": sec * 1e6, "achieved": work / sec, "unit": unit,
               "frac_of_measured_peak": work / sec / peak, "graph": bool(args.graph)}
        if args.kernel == "moe":
            rec["experts"] = args.experts
            rec["weight_GBps_if_all_experts_read"] = args.experts * (2 * 2048 * 7168 + 7168 * 2048) / sec / 1e9
        print(json.dumps(rec))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default=None, choices=["gemm_gate_up", "gemm_down", "gemm", "quant", "moe"],
                    help="time one kernel alone instead of the whole step (gemm: any shape, see --n / --k)")
    ap.add_argument("--n", type=int, default=0, help="--kernel gemm: output features (multiple of 128)")
    ap.add_argument("--k", type=int, default=0, help="--kernel gemm: input features (multiple of 128)")
    ap.add_argument("--m", default="4096", help="token count(s) for --kernel, comma separated")
    ap.add_argument("--experts", type=int, default=256,
                    help="--kernel moe: experts held on this GPU (256 = whole layer, 32 = one rank of 8)")
    ap.add_argument("--tp-chunks", type=int, default=0, choices=[0, 1, 2, 4, 8],
                    help="N > 1: row chunks of the row-parallel projection whose all-reduces overlap the next chunk")
    ap.add_argument("--eager", action="store_true", help="N > 1: enqueue every step from Python instead of graph replay")
    ap.add_argument("--graph", action="store_true",
                    help="--kernel: replay the timed steps from a CUDA graph (excludes Python call overhead)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    if args.kernel is not None:
        run_kernel_case(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
