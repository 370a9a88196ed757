"""Benchmark of the W8A8 block-FP8 linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Headline workload (config.workload): the DeepSeek-V3-shaped dense MLP as two block-FP8 linears at
M = 4096 tokens -- gate_up (K=7168, N=36864) then down (K=18432, N=7168).  One step =
group-quantise x, GEMM, group-quantise h, GEMM.  Inputs are seeded synthetic tensors (activations
N(0,1), weights N(0,0.02) block-quantised once on the full matrix); weights (396 MB of e4m3) and
activations (210 MB of bf16) exceed the 126 MB L2, so no explicit flush is needed.

N > 1 (torchrun, one rank per GPU): the same MLP tensor-parallel as in the reference -- gate_up
column-parallel (N/p per rank, no communication), down row-parallel (K/p per rank) followed by the sum of
the bf16 partial outputs [4096,7168] across ranks (this library's NVLink all-reduce kernels; --allreduce
nccl for the NCCL collective).  Total work is fixed: strong scaling.  Every run checks itself before it
is timed: sampled rows of each rank's outputs against an fp32 torch restatement of the block-scaled product
on unsharded weights, and at N > 1 the expert-parallel MoE layer against the single-GPU fused path
(bitwise); a failed check ends the run with a non-zero exit code.

At every N the step is replayed from a CUDA graph inside the timed region (per-kernel times come from a
separate eager pass with events around each call).  The JSON line carries: value = whole-job TFLOP/s with inputs resident
in HBM; e2e = the same through the public linear call with HOST activations (pinned) copied in and the
bf16 results copied out inside the timed region; roofline for the dominant kernel (the gate_up GEMM);
quant = the group-quantisation kernel on its own benchmark configuration (M=16384 x 7168); config3 /
config4 = the Llama-3-70B tensor-parallel layer set and the DeepSeek-V3 MoE layer; gpu_comparator = the
reference's own sm_100a kernels (when their build is present) timed on the same inputs; cpu_baseline =
the reference's CPU block-FP8 matmul on the host cores.
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
NOMINAL_HBM_GBS = 8000.0
# DRAM bytes (read + write) of one launch of the gate_up GEMM at M=4096 on one GPU, from an ncu capture of
# that launch (dram__bytes_read.sum + dram__bytes_write.sum; algorithmic bytes: 596.9e6)
GEMM_TRAFFIC_BYTES_1GPU = 586.4e6
PARITY_ROWS = 64
TOL_LINEAR = 1e-3        # rel-L2 of a linear's bf16 output vs the fp32 restatement rounded to bf16
TOL_ROW_PARALLEL = 5e-3  # p bf16 partial outputs, each rounded on its own, then summed (as in the reference)


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_sustained": p["bf16_tflops_sustained"],
                "bf16_burst": p["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_sustained": 1400.0, "bf16_burst": 1590.0, "src": "fallback"}


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed regions run."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []
        self.marks = {}

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def mark(self, name):
        self.marks[name] = time.perf_counter()

    def _parse(self, lines):
        clocks, maxc, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for _, ln in lines:
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
        return clocks, maxc, power, reasons

    def window(self, begin, end):
        """Median SM clock and peak power of the samples taken between two marks."""
        t0, t1 = self.marks.get(begin), self.marks.get(end)
        if t0 is None or t1 is None:
            return None
        clocks, _, power, reasons = self._parse([x for x in self.lines if t0 <= x[0] <= t1])
        if not clocks:
            return None
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2], "power_w_max": max(power), "samples": len(clocks),
                "reasons": sorted(reasons)}

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxc, power, reasons = self._parse(self.lines)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load = upper half of the power readings
        order = sorted(range(len(clocks)), key=lambda i: power[i])
        load = sorted(clocks[i] for i in order[len(order) // 2:])
        return {"sm_mhz": load[len(load) // 2], "sm_max_mhz": max(maxc), "power_w_max": max(power),
                "samples": len(clocks), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# CPU reference arm / baseline
# ------------------------------------------------------------------------------------------
def cpu_reference_run(steps: int, warmup: int, sample_rows: int = 64):
    """Times the reference CPU block-FP8 matmul on `sample_rows` tokens of the workload (both
    layers).  Returns (tflops, seconds per pass, info dict)."""
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
    # the full 4096-token workload takes about 0.5 s per pass on 16 AMX cores; shrink the sample
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
# shared helpers of the GPU arm
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


def torch_group_quant(x):
    """Group quantisation restated in torch (the arithmetic of python/sglang/test/test_block_fp8.py:24-49
    with the fp32 eps of the CUDA kernel): the checker's own codes and scales, not the library's."""
    import torch
    m, k = x.shape
    xf = x.float().view(m, k // 128, 128)
    amax = xf.abs().amax(-1).clamp(min=1e-10)
    s = amax / torch.full_like(amax, 448.0)   # tensor / tensor: torch divides by a Python scalar with a reciprocal multiply on CUDA
    q = (xf / s[..., None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(m, k)
    return q, s


def torch_block_matmul_fp32(a_q, b_q, sa, sb):
    """fp32 restatement of the block-scaled product (python/sglang/test/test_block_fp8.py:274-326 before the
    cast): per 128-wide k-block an fp32 matmul of the dequantised codes times sa[m,kb] * sb[n/128,kb]."""
    import torch
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        m, k = a_q.shape
        n = b_q.shape[0]
        c = torch.zeros((m, n), dtype=torch.float32, device=a_q.device)
        sb_rows = sb.repeat_interleave(128, 0)[:n]
        for kb in range(k // 128):
            ak = a_q[:, kb * 128:(kb + 1) * 128].float()
            bk = b_q[:, kb * 128:(kb + 1) * 128].float()
            c += (ak @ bk.t()) * (sa[:, kb:kb + 1] * sb_rows[:, kb][None, :])
        return c
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def rel_l2(x, ref):
    return float(((x.float() - ref.float()).norm() / ref.float().norm().clamp(min=1e-30)).item())


def time_graph(fn, steps, barrier, stream_setup=None):
    """Captures `fn` once, replays it `steps` times between events; returns (ms per step, graph)."""
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
        fn()
    for _ in range(3):
        g.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    for _ in range(steps):
        g.replay()
    b.record()
    barrier()
    return a.elapsed_time(b) / steps, g


def time_eager(fn, steps, warmup=3):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def gemm_status_ok():
    import ctypes
    from sglang_b200 import _lib
    st = ctypes.c_int(0)
    _lib.check("status", _lib.lib().b200_gemm_device_status(ctypes.byref(st)))
    return st.value == 0


# ------------------------------------------------------------------------------------------
# extra keys: quant (config 2), Llama-3-70B layer set (config 3), MoE layer (config 4), comparator
# ------------------------------------------------------------------------------------------
def quant_config2(dev, pk, steps=20):
    """Config 2: [16384, 7168] bf16 with 0.1 % outliers -> e4m3 + column-major padded fp32 scales; the inputs
    rotate through enough buffers to exceed L2."""
    import torch
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    m = 16384
    g = torch.Generator(device=dev).manual_seed(2000)
    xs = []
    for _ in range(3):
        x = torch.randn((m, HIDDEN), generator=g, device=dev)
        x = torch.where(torch.rand((m, HIDDEN), generator=g, device=dev) < 1e-3, x * 100, x)
        xs.append(x.to(torch.bfloat16))
    it = [0]

    def fn():
        it[0] += 1
        return sglang_per_token_group_quant_fp8(xs[it[0] % 3], 128, column_major_scales=True, scale_tma_aligned=True)
    ms, g_ = time_graph(lambda: [fn() for _ in range(6)], steps, torch.cuda.synchronize)
    g_.reset()
    ms /= 6
    nbytes = 3.03125 * m * HIDDEN
    gbs = nbytes / (ms * 1e-3) / 1e9
    # the producer-side fusion: RMSNorm -> quant in one pass against the norm kernel followed by the quant kernel
    from sglang_b200.layers.quantization.fp8_kernel import rmsnorm, rmsnorm_per_token_group_quant_fp8
    w = (1.0 + 0.1 * torch.randn(HIDDEN, generator=g, device=dev)).to(torch.bfloat16)

    def fused():
        it[0] += 1
        return rmsnorm_per_token_group_quant_fp8(xs[it[0] % 3], w, 1e-6, column_major_scales=True, scale_tma_aligned=True)

    def pair():
        it[0] += 1
        return sglang_per_token_group_quant_fp8(rmsnorm(xs[it[0] % 3], w, 1e-6), 128, column_major_scales=True,
                                                scale_tma_aligned=True)
    ms_f, g_ = time_graph(lambda: [fused() for _ in range(6)], steps, torch.cuda.synchronize)
    g_.reset()
    ms_p, g_ = time_graph(lambda: [pair() for _ in range(6)], steps, torch.cuda.synchronize)
    g_.reset()
    # the same operator with its int8 destination
    from sglang_b200.layers.quantization.int8_kernel import sglang_per_token_group_quant_int8

    def int8():
        it[0] += 1
        return sglang_per_token_group_quant_int8(xs[it[0] % 3], 128)
    ms_i, g_ = time_graph(lambda: [int8() for _ in range(6)], steps, torch.cuda.synchronize)
    g_.reset()
    return {"bound": "hbm", "kernel": "quant_group_kernel<bf16,128> on [16384,7168] (config 2), graph replay, 3 rotating "
                                      "inputs (705 MB)", "us": ms * 1e3, "achieved": gbs, "peak": pk["hbm_gbs"],
            "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS,
            "algorithmic_bytes_per_launch": nbytes,
            "rmsnorm_quant_fused_us": ms_f / 6 * 1e3, "rmsnorm_then_quant_us": ms_p / 6 * 1e3,
            "rmsnorm_quant_fused_gbs": nbytes / (ms_f / 6 * 1e-3) / 1e9,
            "int8_destination_us": ms_i / 6 * 1e3, "int8_destination_gbs": nbytes / (ms_i / 6 * 1e-3) / 1e9}


def fp8_ceiling(dev, steps=20):
    """Yardstick only: per-tensor-scaled e4m3 torch._scaled_mm at 8192^3 (a library GEMM without block scales)."""
    import torch
    try:
        x = torch.randn((8192, 8192), device=dev).to(torch.float8_e4m3fn)
        w = torch.randn((8192, 8192), device=dev).to(torch.float8_e4m3fn)
        one = torch.ones((), device=dev)
        ms = time_eager(lambda: torch._scaled_mm(x, w.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16), steps)
        return 2.0 * 8192 ** 3 / (ms * 1e-3) / 1e12
    except Exception as e:  # noqa: BLE001
        print(f"[bench] fp8 ceiling not measured: {e}", file=sys.stderr)
        return None


def ue8m0_mlp(dev, ceiling, steps=10):
    """The headline MLP step with POWER-OF-TWO scales (the reference's DeepGEMM / UE8M0 mode, its default on
    Blackwell): weights re-quantised to power-of-two block scales, activations quantised with packed UE8M0 scales,
    products on the tensor core's block-scaling path (no fp32 promotion).  Same shapes and FLOPs as the headline."""
    import torch
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8, w8a8_block_fp8_matmul_deepgemm
    from sglang_b200.layers.quantization.fp8_utils import deepgemm_w8a8_block_fp8_linear_with_fallback, requant_weight_ue8m0
    w1q, w1s = gen_weight_device(INTER2, HIDDEN, 100, dev)
    w2q, w2s = gen_weight_device(HIDDEN, INTER, 200, dev)
    w1q, w1s = requant_weight_ue8m0(w1q, w1s, [128, 128])
    w2q, w2s = requant_weight_ue8m0(w2q, w2s, [128, 128])
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn((M_TOKENS, HIDDEN), generator=g, device=dev).to(torch.bfloat16)
    h = torch.randn((M_TOKENS, INTER), generator=g, device=dev).to(torch.bfloat16)

    def step():
        y1 = deepgemm_w8a8_block_fp8_linear_with_fallback(x, w1q, [128, 128], w1s, weight_scale_ue8m0=True)
        y2 = deepgemm_w8a8_block_fp8_linear_with_fallback(h, w2q, [128, 128], w2s, weight_scale_ue8m0=True)
        return y1, y2
    ms, g_ = time_graph(step, steps, torch.cuda.synchronize)
    g_.reset()
    q, sp = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
    hw = w8a8_block_fp8_matmul_deepgemm(q, w1q, sp, w1s, [128, 128], torch.bfloat16, weight_scale_ue8m0=True)
    sw = w8a8_block_fp8_matmul_deepgemm(q, w1q, sp, w1s, [128, 128], torch.bfloat16)
    err = rel_l2(hw, sw)
    us, g_ = time_graph(lambda: [w8a8_block_fp8_matmul_deepgemm(q, w1q, sp, w1s, [128, 128], torch.bfloat16,
                                                                weight_scale_ue8m0=True) for _ in range(4)], 5,
                        torch.cuda.synchronize)
    g_.reset()
    gemm_ms = us / 4
    gemm_tf = 2.0 * M_TOKENS * INTER2 * HIDDEN / (gemm_ms * 1e-3) / 1e12
    out = {"workload": WORKLOAD + " with power-of-two (UE8M0) activation and weight scales",
           "kernel": "gemm_mx_kernel (tcgen05.mma kind::mxf8f6f4.block_scale, all k-blocks accumulated in tensor memory)",
           "ms_per_step": ms, "step_tflops": FLOPS_PER_STEP / (ms * 1e-3) / 1e12,
           "gemm_gate_up_ms": gemm_ms, "gemm_gate_up_tflops": gemm_tf,
           "frac_of_nominal_4500": gemm_tf / NOMINAL_FP8_TFLOPS,
           "rel_l2_vs_fp32_promotion_kernel_on_the_same_codes": err}
    if ceiling:
        out["frac_of_fp8_ceiling"] = gemm_tf / ceiling
    # the same two projections as a CHAIN (down consumes SiLU(gate) * up of gate_up's output): with the activation and
    # the second quantisation in gate_up's epilogue, and as separate kernels; the two produce the same bits
    from sglang_b200.layers.quantization.deep_gemm_wrapper import gate_up_silu_quant_pow2
    from sglang_b200.layers.quantization.fp8_kernel import silu_and_mul_per_token_group_quant_fp8

    def chain_fused():
        q_, s_ = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
        hq, hs = gate_up_silu_quant_pow2(q_, s_, w1q, w1s)
        return w8a8_block_fp8_matmul_deepgemm(hq, w2q, hs, w2s, [128, 128], torch.bfloat16, weight_scale_ue8m0=True)

    def chain_separate():
        q_, s_ = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
        c1 = w8a8_block_fp8_matmul_deepgemm(q_, w1q, s_, w1s, [128, 128], torch.bfloat16, weight_scale_ue8m0=True)
        hq, hs = silu_and_mul_per_token_group_quant_fp8(c1, 128, scale_ue8m0=True)
        return w8a8_block_fp8_matmul_deepgemm(hq, w2q, hs, w2s, [128, 128], torch.bfloat16, weight_scale_ue8m0=True)
    same = bool(torch.equal(chain_fused(), chain_separate()))
    ms_f, g_ = time_graph(chain_fused, steps, torch.cuda.synchronize)
    g_.reset()
    ms_s, g_ = time_graph(chain_separate, steps, torch.cuda.synchronize)
    g_.reset()
    out["mlp_chain"] = {"what": "quant -> gate_up -> SiLU*mul -> quant -> down as one dependent chain (4096 tokens)",
                        "fused_epilogue_ms": ms_f, "separate_kernels_ms": ms_s, "same_bits": same,
                        "tflops_fused": FLOPS_PER_STEP / (ms_f * 1e-3) / 1e12}
    del w1q, w1s, w2q, w2s
    torch.cuda.empty_cache()
    return out


LLAMA = {"qkv": ("col", 10240, 8192), "gate_up": ("col", 57344, 8192), "o_proj": ("row", 8192, 8192),
         "down": ("row", 8192, 28672)}


def llama_config3(dev, world, rank, ar, steps=10):
    """Config 3: the four Llama-3-70B projections tensor-parallel over `world` ranks at M = 128 and 8192, each
    through the product's parallel linear (quantisation + GEMM + the all-reduce of the row-parallel ones),
    replayed from a CUDA graph.  Returns {layer: {M: ms}} (max over ranks taken by the caller)."""
    import torch
    import torch.distributed as dist
    from sglang_b200.distributed import ColumnParallelBlockFp8Linear, RowParallelBlockFp8Linear

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    out = {}
    for li, (name, (kind, n, k)) in enumerate(LLAMA.items()):
        n_r, k_r = (n // world, k) if kind == "col" else (n, k // world)
        wq, ws = gen_weight_device(n_r, k_r, 3000 + 10 * li + rank, dev)
        if kind == "col":
            layer = ColumnParallelBlockFp8Linear(wq, ws, already_sharded=True)
        else:
            layer = RowParallelBlockFp8Linear(wq, ws, already_sharded=True, all_reduce=ar)
        out[name] = {}
        for m in (128, 8192):
            g = torch.Generator(device=dev).manual_seed(31 + m)
            x = torch.randn((m, k_r), generator=g, device=dev).to(torch.bfloat16)
            ms, g_ = time_graph(lambda: layer(x), steps, barrier)
            g_.reset()
            out[name][str(m)] = ms
        del layer, wq, ws
    return out


def moe_weights(dev, experts, seed0, H=7168, I=2048):
    """Expert weights with directly drawn codes and scales (11.3 GB for 256 experts), expert e from seed0 + e so
    that any rank can rebuild any expert."""
    import torch
    w13 = torch.empty((len(experts), 2 * I, H), dtype=torch.float8_e4m3fn, device=dev)
    w2 = torch.empty((len(experts), H, I), dtype=torch.float8_e4m3fn, device=dev)
    w13s = torch.empty((len(experts), 2 * I // 128, H // 128), dtype=torch.float32, device=dev)
    w2s = torch.empty((len(experts), H // 128, I // 128), dtype=torch.float32, device=dev)

    def codes(g, *shape):
        c = torch.randint(0, 0x78, shape, generator=g, device=dev, dtype=torch.uint8)
        sign = torch.randint(0, 2, shape, generator=g, device=dev, dtype=torch.uint8) << 7
        return (c | sign).view(torch.float8_e4m3fn)
    for i, e in enumerate(experts):
        g = torch.Generator(device=dev).manual_seed(seed0 + e)
        w13[i] = codes(g, 2 * I, H)
        w2[i] = codes(g, H, I)
        w13s[i] = torch.rand((2 * I // 128, H // 128), generator=g, device=dev) * 2e-4 + 1e-5
        w2s[i] = torch.rand((H // 128, I // 128), generator=g, device=dev) * 2e-4 + 1e-5
    return w13, w2, w13s, w2s


def moe_routing(dev, tokens, E=256, topk=8, seed=4000):
    import torch
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn((tokens, 7168), generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn((tokens, E), generator=g, device=dev)
    tw, ti = torch.topk(torch.softmax(logits.float(), dim=-1), topk, dim=-1)
    return x, tw.contiguous(), ti.to(torch.int32).contiguous()


def moe_config4_single(dev, pk, steps=5):
    """Config 4 on one GPU: 256 experts, 4096 tokens, top-8 through the fused layer."""
    import torch
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
    E, H, I, topk, tokens = 256, 7168, 2048, 8, 4096
    w13, w2, w13s, w2s = moe_weights(dev, list(range(E)), 5000)
    x, tw, ti = moe_routing(dev, tokens)
    ms, g_ = time_graph(lambda: fused_experts_block_fp8(x, w13, w2, w13s, w2s, tw, ti), steps, torch.cuda.synchronize)
    g_.reset()
    flops = 2.0 * tokens * topk * (2 * I * H + H * I)
    wbytes = float(E) * (2 * I * H + H * I)
    floor_ms = wbytes / (pk["hbm_gbs"] * 1e9) * 1e3
    # the same layer with power-of-two scales on both sides (the reference's DeepGEMM expert path on Blackwell):
    # the codes stay, the drawn weight scales are rounded up to powers of two
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8_ue8m0
    w13s.copy_(torch.exp2(torch.ceil(torch.log2(w13s))))
    w2s.copy_(torch.exp2(torch.ceil(torch.log2(w2s))))
    ms2, g_ = time_graph(lambda: fused_experts_block_fp8_ue8m0(x, w13, w2, w13s, w2s, tw, ti), steps,
                         torch.cuda.synchronize)
    g_.reset()
    del w13, w2, w13s, w2s
    torch.cuda.empty_cache()
    return {"workload": "deepseek_v3_moe_block_fp8(256 experts, top-8, 4096 tokens, hidden 7168, intermediate 2048)",
            "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "weight_gbs": wbytes / (ms * 1e-3) / 1e9,
            "weight_read_floor_ms": floor_ms, "frac_of_floor": floor_ms / ms,
            "ue8m0_path": {"kernel": "gemm_mx_kernel<grouped> (tcgen05.mma kind::mxf8f6f4.block_scale), power-of-two "
                                     "activation and weight scales",
                           "ms": ms2, "tflops": flops / (ms2 * 1e-3) / 1e12, "weight_gbs": wbytes / (ms2 * 1e-3) / 1e9,
                           "frac_of_floor": floor_ms / ms2}}


def moe_config4_ep(dev, world, rank, steps=5):
    """Config 4 expert-parallel: 256 experts split contiguously over the ranks, 4096 tokens sharded over the
    ranks, dispatch / local experts / combine.  Rank 0 also holds all experts and compares its own tokens with
    the single-GPU fused layer, bit for bit."""
    import torch
    import torch.distributed as dist
    from sglang_b200.distributed import ExpertParallelBlockFp8MoE
    from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
    E, H, I, topk, tokens = 256, 7168, 2048, 8, 4096
    el, tl = E // world, tokens // world
    w13, w2, w13s, w2s = moe_weights(dev, list(range(rank * el, (rank + 1) * el)), 5000)
    x_all, tw_all, ti_all = moe_routing(dev, tokens)        # same seed on every rank: identical routing
    sl = slice(rank * tl, (rank + 1) * tl)
    x, tw, ti = x_all[sl].contiguous(), tw_all[sl].contiguous(), ti_all[sl].contiguous()
    moe = ExpertParallelBlockFp8MoE(w13, w2, w13s, w2s)
    y = moe(x, tw, ti)
    torch.cuda.synchronize()
    ok = 1
    if rank == 0:
        fw13, fw2, fw13s, fw2s = moe_weights(dev, list(range(E)), 5000)
        ref = fused_experts_block_fp8(x, fw13, fw2, fw13s, fw2s, tw, ti)
        ok = int(torch.equal(y, ref))
        del fw13, fw2, fw13s, fw2s, ref
        torch.cuda.empty_cache()
    flag = torch.tensor([ok], device=dev, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()
    ms = []
    for _ in range(2):
        moe(x, tw, ti)
    for _ in range(steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        moe(x, tw, ti)
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b))
    t = torch.tensor([sorted(ms)[len(ms) // 2]], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    stages = getattr(moe, "last_stage_ms", None)
    res = {"workload": f"deepseek_v3_moe_block_fp8 expert-parallel: {el} experts and {tl} tokens per rank, top-8",
           "ms": float(t.item()), "tflops": 2.0 * tokens * topk * (2 * I * H + H * I) / (float(t.item()) * 1e-3) / 1e12,
           "bitwise_equal_to_single_gpu_on_rank0_tokens": bool(int(flag.item()))}
    if stages:
        res["stages_ms_rank0"] = stages
    # the same layer on the block-scaling path: power-of-two weight scales (the drawn ones rounded up), activations
    # dispatched with packed exponent words
    w13s.copy_(torch.exp2(torch.ceil(torch.log2(w13s))))
    w2s.copy_(torch.exp2(torch.ceil(torch.log2(w2s))))
    moe2 = ExpertParallelBlockFp8MoE(w13, w2, w13s, w2s, scale_ue8m0=True)
    ms2 = []
    for _ in range(2):
        moe2(x, tw, ti)
    for _ in range(steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        moe2(x, tw, ti)
        b.record()
        torch.cuda.synchronize()
        ms2.append(a.elapsed_time(b))
    moe2.check()
    t2 = torch.tensor([sorted(ms2)[len(ms2) // 2]], device=dev)
    dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    res["ue8m0_path_ms"] = float(t2.item())
    return res, bool(int(flag.item()))


def gpu_comparator(dev, steps=10):
    """The reference's own sm_100a kernels (built by oracle/build_ref_cuda.py from the reference checkout into
    baseline/_ref/), timed beside this library's kernels on the same inputs in this process.  Comparison
    only: nothing here is on the product path.  Each side runs from a CUDA graph of `steps` calls."""
    import torch
    from oracle import build_ref_cuda as R
    from sglang_b200.layers.quantization.fp8_kernel import sglang_per_token_group_quant_fp8
    from sglang_b200.sgl_kernel import fp8_blockwise_scaled_mm
    out = {"built_from": "sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu, per_token_group_quant_8bit.cu, "
                         "csrc/moe/fp8_blockwise_moe_kernel.cu (CUTLASS headers of the flashinfer package, not the "
                         "commit the reference pins)"}
    have = {}
    for fam in ("quant", "gemm"):
        try:
            have[fam] = R.load(fam)
        except Exception as e:  # noqa: BLE001
            have[fam] = False
            out[f"{fam}_load_error"] = str(e)[:200]
    if not any(have.values()):
        out["unavailable"] = "baseline/_ref holds no built comparator library"
        return out
    ops = torch.ops.sgl_kernel_ref
    g = torch.Generator(device=dev).manual_seed(77)

    def graph_us(fn):
        ms, g_ = time_graph(lambda: [fn() for _ in range(4)], steps, torch.cuda.synchronize)
        g_.reset()
        return ms / 4 * 1e3
    if have["quant"]:
        m = 16384
        xs = [torch.randn((m, HIDDEN), generator=g, device=dev).to(torch.bfloat16) for _ in range(3)]
        q = torch.empty((m, HIDDEN), device=dev, dtype=torch.float8_e4m3fn)
        s = torch.empty((HIDDEN // 128, m), device=dev, dtype=torch.float32).t()
        it = [0]

        def ref_q():
            it[0] += 1
            ops.sgl_per_token_group_quant_fp8(xs[it[0] % 3], q, s, 128, 1e-10, -448.0, 448.0, False)

        def our_q():
            it[0] += 1
            sglang_per_token_group_quant_fp8(xs[it[0] % 3], 128, column_major_scales=True)
        ref_q()
        q2, s2 = sglang_per_token_group_quant_fp8(xs[it[0] % 3], 128, column_major_scales=True)
        same = bool(torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2))
        t_ref, t_us = graph_us(ref_q), graph_us(our_q)
        out["quant_M16384"] = {"reference_us": t_ref, "ours_us": t_us, "speedup": t_ref / t_us, "bit_identical": same}
        del xs, q, s
    if have["gemm"]:
        for name, (m, n, k) in {"gate_up_M4096": (4096, INTER2, HIDDEN), "down_M4096": (4096, HIDDEN, INTER),
                                "gate_up_M128": (128, INTER2, HIDDEN), "down_M128": (128, HIDDEN, INTER)}.items():
            ncopy = 1 if m > 512 else 3       # small M streams weights: rotate copies so that they come from HBM
            ws = [gen_weight_device(n, k, 700 + c, dev) for c in range(ncopy)]
            x = torch.randn((m, k), generator=g, device=dev).to(torch.bfloat16)
            a, sa = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True)
            it = [0]

            def ref_mm():
                it[0] += 1
                wq, wsc = ws[it[0] % ncopy]
                return ops.fp8_blockwise_scaled_mm(a, wq.t(), sa, wsc.t(), torch.bfloat16)

            def our_mm():
                it[0] += 1
                wq, wsc = ws[it[0] % ncopy]
                return fp8_blockwise_scaled_mm(a, wq.t(), sa, wsc.t(), torch.bfloat16)
            it[0] = 0
            o_ref = ref_mm()
            it[0] = 0
            o_us = our_mm()
            err = rel_l2(o_us, o_ref)
            t_ref, t_us = graph_us(ref_mm), graph_us(our_mm)
            out[name] = {"reference_us": t_ref, "ours_us": t_us, "speedup": t_ref / t_us, "rel_l2_between": err,
                         "ours_tflops": 2.0 * m * n * k / (t_us * 1e-6) / 1e12,
                         "reference_tflops": 2.0 * m * n * k / (t_ref * 1e-6) / 1e12}
            del ws
    try:
        have_moe = R.load("moe")
    except Exception as e:  # noqa: BLE001
        have_moe = False
        out["moe_load_error"] = str(e)[:200]
    if have_moe:
        # the two expert GEMMs of config 4 (256 experts, 4096 tokens, top-8) on the reference's CUTLASS grouped kernel
        # (sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu), on this library's fp32-scale grouped kernel (same inputs,
        # outputs compared) and on its block-scaling grouped kernel (power-of-two scales)
        from sglang_b200.layers.quantization.deep_gemm_wrapper import grouped_gemm_pow2
        from sglang_b200.layers.quantization.fp8_kernel import silu_and_mul_per_token_group_quant_fp8
        from sglang_b200.sgl_kernel import (fp8_blockwise_scaled_grouped_mm, prepare_moe_input, shuffle_packed_scales,
                                            shuffle_rows)
        E, H, I, topk, m = 256, 7168, 2048, 8, 4096
        w13, w2, w13s, w2s = moe_weights(dev, list(range(E)), 5000)
        a, tw, ti = moe_routing(dev, m, E=E)
        i32, i64 = dict(dtype=torch.int32, device=dev), dict(dtype=torch.int64, device=dev)
        eo, ps1, ps2 = torch.empty(E + 1, **i32), torch.empty((E, 3), **i32), torch.empty((E, 3), **i32)
        a_map, c_map = torch.zeros(m * topk, **i32), torch.empty(m * topk, **i32)
        prepare_moe_input(ti, eo, ps1, ps2, a_map, c_map, E, I, H)
        a_q, a_s = sglang_per_token_group_quant_fp8(a, 128)
        rq, rs = shuffle_rows(a_q, a_map, (m * topk, H)), shuffle_rows(a_s, a_map, (m * topk, H // 128))
        a_qp, a_sp = sglang_per_token_group_quant_fp8(a, 128, column_major_scales=True, scale_tma_aligned=True,
                                                      scale_ue8m0=True)
        rqp, rsp = shuffle_rows(a_qp, a_map, (m * topk, H)), shuffle_packed_scales(a_sp, a_map)
        w13p, w2p = torch.exp2(torch.ceil(torch.log2(w13s))), torch.exp2(torch.ceil(torch.log2(w2s)))
        ptrs = [torch.empty(E, **i64) for _ in range(5)]
        lay = [torch.empty((E, 5), **i32) for _ in range(2)]
        wsp = torch.empty(90000, dtype=torch.uint8, device=dev)
        c1r, c1 = (torch.zeros((m * topk, 2 * I), dtype=torch.bfloat16, device=dev) for _ in range(2))
        c2r, c2 = (torch.zeros((m * topk, H), dtype=torch.bfloat16, device=dev) for _ in range(2))

        def our_mm(c, x, xs_, w, wsc, ps):
            fp8_blockwise_scaled_grouped_mm(c, None, None, None, None, None, x, w.transpose(1, 2), xs_,
                                            wsc.transpose(1, 2), None, None, None, None, None, ps, eo[:-1], None)
        st1 = (torch.full((E,), H, **i64), torch.full((E,), 2 * I, **i64))
        st2 = (torch.full((E,), I, **i64), torch.full((E,), H, **i64))

        def ref1():
            ops.fp8_blockwise_scaled_grouped_mm(c1r, *ptrs, rq, w13.transpose(1, 2), rs, w13s.transpose(1, 2), st1[0], st1[0],
                                                st1[1], lay[0], lay[1], ps1, eo[:-1], wsp)
        ref1()
        our_mm(c1, rq, rs, w13, w13s, ps1)
        iq, is_ = silu_and_mul_per_token_group_quant_fp8(c1, 128)
        iqp, isp = silu_and_mul_per_token_group_quant_fp8(c1, 128, scale_ue8m0=True)

        def ref2():
            ops.fp8_blockwise_scaled_grouped_mm(c2r, *ptrs, iq, w2.transpose(1, 2), is_, w2s.transpose(1, 2), st2[0], st2[0],
                                                st2[1], lay[0], lay[1], ps2, eo[:-1], wsp)
        ref2()
        our_mm(c2, iq, is_, w2, w2s, ps2)
        torch.cuda.synchronize()
        for name, fr, fo, fp, cr, co in (
                ("moe_gemm1_E256_T4096", ref1, lambda: our_mm(c1, rq, rs, w13, w13s, ps1),
                 lambda: grouped_gemm_pow2(rqp, rsp, w13, w13p, c1, eo[:-1], ps1[:, 0]), c1r, c1),
                ("moe_gemm2_E256_T4096", ref2, lambda: our_mm(c2, iq, is_, w2, w2s, ps2),
                 lambda: grouped_gemm_pow2(iqp, isp, w2, w2p, c2, eo[:-1], ps1[:, 0]), c2r, c2)):
            err = rel_l2(co, cr)
            t_ref, t_us, t_p2 = graph_us(fr), graph_us(fo), graph_us(fp)
            out[name] = {"reference_us": t_ref, "ours_us": t_us, "speedup": t_ref / t_us, "rel_l2_between": err,
                         "ours_power_of_two_scales_us": t_p2, "speedup_power_of_two_scales": t_ref / t_p2}
        del w13, w2, w13s, w2s, w13p, w2p
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from sglang_b200 import _lib
    from sglang_b200.distributed import ColumnParallelBlockFp8Linear, RowParallelBlockFp8Linear
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
    pk = _peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    t_start = time.time()
    ar = None

    snaps = []

    def dbg(msg):
        if os.environ.get("B200_BENCH_TRACE") and ar is not None:
            # stage marker without a host synchronisation: a stream-ordered copy of the all-reduce status word
            h_ = torch.empty(1, dtype=torch.int32).pin_memory()
            h_.copy_(ar._status, non_blocking=True)
            snaps.append((msg, h_))
        if os.environ.get("B200_BENCH_DEBUG"):
            torch.cuda.synchronize()
            st_ = f" all-reduce status {int(ar._status.item())}" if ar is not None else ""
            print(f"[bench r{rank} +{time.time() - t_start:.2f}s] {msg}{st_}", file=sys.stderr, flush=True)

    # Weights are quantised once on the FULL matrix (same seed on every rank) and sharded by the product's
    # parallel linears, so the tensor-parallel result is comparable with the unsharded one.
    w1q, w1s = gen_weight_device(INTER2, HIDDEN, 100, dev)
    w2q, w2s = gen_weight_device(HIDDEN, INTER, 200, dev)
    if world > 1 and args.allreduce == "custom":
        from sglang_b200.distributed.custom_all_reduce import SymmetricAllReduce
        ar = SymmetricAllReduce(max(M_TOKENS, 8192) * 8192 * 2)
        ar_forms_us = ar.autotune(M_TOKENS * HIDDEN * 2)       # multicast or peer pointers: whichever is faster here
        # NCCL's all-reduce of the same bytes, for comparison only (it is not used in this configuration)
        t_nccl = torch.zeros((M_TOKENS, HIDDEN), dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            dist.all_reduce(t_nccl)
        torch.cuda.synchronize()
        dist.barrier()
        e0_, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0_.record()
        for _ in range(10):
            dist.all_reduce(t_nccl)
        e1_.record()
        torch.cuda.synchronize()
        tn_ = torch.tensor([e0_.elapsed_time(e1_) / 10 * 1e3], device=dev)
        dist.all_reduce(tn_, op=dist.ReduceOp.MAX)
        ar_forms_us["nccl_for_comparison"] = float(tn_.item())
        del t_nccl
    col = ColumnParallelBlockFp8Linear(w1q, w1s)
    row = RowParallelBlockFp8Linear(w2q, w2s, all_reduce=ar)
    g = torch.Generator(device=dev).manual_seed(7)           # x is replicated: same seed on all ranks
    x = torch.randn((M_TOKENS, HIDDEN), generator=g, device=dev).to(torch.bfloat16)
    gh = torch.Generator(device=dev).manual_seed(300)        # h: every rank draws the full matrix, keeps its K slice
    h_full = torch.randn((M_TOKENS, INTER), generator=gh, device=dev).to(torch.bfloat16)
    h = h_full[:, rank * k2:(rank + 1) * k2].contiguous()

    # ---- self-check before anything is timed
    rows = torch.arange(0, M_TOKENS, M_TOKENS // PARITY_ROWS, device=dev)
    dbg("inputs ready")
    y1 = col(x)
    dbg("column-parallel done")
    y2 = row(h).clone()
    dbg("row-parallel done")
    xq_r, xs_r = torch_group_quant(x[rows])
    ref1 = torch_block_matmul_fp32(xq_r, w1q[rank * n1:(rank + 1) * n1], xs_r, w1s[rank * n1 // 128:(rank + 1) * n1 // 128])
    hq_r, hs_r = torch_group_quant(h_full[rows])
    ref2 = torch_block_matmul_fp32(hq_r, w2q, hs_r, w2s)
    err1 = rel_l2(y1[rows], ref1.to(torch.bfloat16))
    err2 = rel_l2(y2[rows], ref2.to(torch.bfloat16))
    same_on_ranks = True
    if world > 1:
        y2_0 = y2[rows].clone()
        dist.broadcast(y2_0, 0)
        same_on_ranks = bool(torch.equal(y2_0, y2[rows]))
    tol2 = TOL_LINEAR if world == 1 else TOL_ROW_PARALLEL
    ok_local = int(err1 <= TOL_LINEAR and err2 <= tol2 and (same_on_ranks or ar is None) and gemm_status_ok())
    errs = torch.tensor([err1, err2, float(ok_local)], device=dev, dtype=torch.float64)
    if world > 1:
        emax = errs.clone()
        dist.all_reduce(emax, op=dist.ReduceOp.MAX)
        emin = errs.clone()
        dist.all_reduce(emin, op=dist.ReduceOp.MIN)
        err1, err2, ok_all = float(emax[0]), float(emax[1]), bool(emin[2] > 0)
    else:
        ok_all = bool(ok_local)
    parity = {"rows_checked": PARITY_ROWS, "checker": "fp32 torch restatement of quantisation and block-scaled product "
                                                      "on the unsharded weights",
              "column_parallel_rel_l2": err1, "row_parallel_rel_l2": err2,
              "tolerance": {"linear": TOL_LINEAR, "row_parallel_sum_of_bf16_partials": tol2},
              "all_reduced_rows_identical_on_all_ranks": same_on_ranks if world > 1 else None, "ok": ok_all}
    del h_full, ref1, ref2
    if ar is not None:
        ar.check()

    chunk_ms = {}
    chunks_used, reserve_used = 1, 0

    def step():
        return col(x), row(h)

    if world > 1:
        # How many row chunks the row-parallel projection is cut into is a trade between overlap (the all-reduce
        # of one chunk under the GEMM of the next) and the fixed cost of each collective.  The warm-up measures
        # the candidates (graph replays, slowest rank counts) and the timed region runs the fastest.
        # A candidate is (row chunks, SMs left to the all-reduce): with SMs reserved the chunk GEMMs run on the rest
        # and the all-reduce runs in its multicast form beside them; with none the two kernels compete for the SMs.
        cands = [(args.tp_chunks, 0)] if args.tp_chunks else [(1, 0), (2, 0), (4, 0)]
        if not args.tp_chunks and ar is not None and ar.has_multicast:
            cands += [(2, 16), (4, 16), (8, 16), (2, 8), (4, 8), (2, 4)]
        best = None
        for c, r in cands:
            row.overlap_chunks, row.reserve_sms = c, r
            ms_c, g_c = time_graph(step, 10, barrier)
            g_c.reset()
            t = torch.tensor([ms_c], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            name = str(c) if r == 0 else f"{c} (+{r} SMs reserved)"
            chunk_ms[name] = round(float(t.item()), 4)
            dbg(f"row chunks {name}: {chunk_ms[name]} ms")
            if best is None or float(t.item()) < best[0]:
                best = (float(t.item()), c, r)
        chunks_used, reserve_used = best[1], best[2]
        row.overlap_chunks, row.reserve_sms = chunks_used, reserve_used
        if ar is not None:
            ar.check()

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    # ---- timed region 1: device-resident inputs, the step replayed from a CUDA graph (same at every N)
    sampler.mark("burst0")
    ms, graph = time_graph(step, args.steps, barrier)
    sampler.mark("burst1")
    dbg("timed region done")
    # ---- per-kernel times: a separate eager pass with events around each call (one GPU's share of the step),
    # directly after the timed region and before the long loop, so that it sees the clocks the timed region saw
    per_kernel = {}
    xq, xs = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True)
    hq, hs = sglang_per_token_group_quant_fp8(h, 128, column_major_scales=True)
    w1r, w1sr, w2r, w2sr = col.weight, col.weight_scale, row.weight, row.weight_scale
    calls = {"quant_x": lambda: sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True),
             "gemm_gate_up": lambda: fp8_blockwise_scaled_mm(xq, w1r.T, xs, w1sr.T, torch.bfloat16),
             "quant_h": lambda: sglang_per_token_group_quant_fp8(h, 128, column_major_scales=True),
             "gemm_down": lambda: fp8_blockwise_scaled_mm(hq, w2r.T, hs, w2sr.T, torch.bfloat16)}
    # one call of each per pass, in the order of the step, events around every call (eager): the clocks a kernel
    # sees are those of the step it is part of, not those of a kernel repeated back to back under the power cap
    for _ in range(2):
        for fn in calls.values():
            fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(5):
        for name, fn in calls.items():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            evs.append((name, a, b))
    torch.cuda.synchronize()
    for name, a, b in evs:
        per_kernel.setdefault(name, []).append(a.elapsed_time(b))
    per_kernel = {k_: sum(v_) / len(v_) for k_, v_ in per_kernel.items()}
    if world > 1:
        y2b = row._out_buffer(M_TOKENS, h) if ar is not None else torch.empty((M_TOKENS, HIDDEN), dtype=torch.bfloat16, device=dev)
        us, g_ = time_graph(lambda: row._reduce(y2b), 5, barrier)
        g_.reset()
        per_kernel["all_reduce_[4096,7168]_bf16"] = us
    dbg("per-kernel pass done")

    # ---- the same step back to back for >= 2 s: the clocks settle under the power cap
    ms_all = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms_all, op=dist.ReduceOp.MAX)      # every rank must replay the SAME number of steps
    reps = max(args.steps, int(2000.0 / max(float(ms_all.item()), 1e-3)) + 1)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark("sus0")
    t0.record()
    trace_replays = bool(os.environ.get("B200_BENCH_TRACE"))
    worst, worst_i, tprev = 0.0, -1, time.perf_counter()
    for i_ in range(reps):
        graph.replay()
        if trace_replays:
            tn = time.perf_counter()
            if tn - tprev > worst:
                worst, worst_i = tn - tprev, i_
            tprev = tn
    t1.record()
    barrier()
    if trace_replays:
        print(f"[bench r{rank}] sustained loop: {reps} replays, longest host-side gap between two launches "
              f"{worst * 1e3:.1f} ms at replay {worst_i}, device time {t0.elapsed_time(t1):.1f} ms", file=sys.stderr, flush=True)
    sampler.mark("sus1")
    sustained_ms = t0.elapsed_time(t1) / reps
    graph.reset()
    dbg("sustained loop done")

    # ---- timed region 2: end to end through the public linear call with host buffers.  Every step copies its
    # activations in from pinned host memory and its results back; the three legs (copy in, compute, copy out) of
    # consecutive steps overlap on three streams with double buffers.  With p ranks each rank moves 1/p of every
    # replicated tensor over its own PCIe link: its row slice of x (the ranks exchange the slices over NVLink),
    # its own K slice of h, its own N slice of y1 and its row slice of the summed y2.
    DEPTH = 2
    mr = M_TOKENS // p
    x_host = x[rank * mr:(rank + 1) * mr].cpu().pin_memory()
    h_host = h.cpu().pin_memory()
    y1_host = [torch.empty((M_TOKENS, n1), dtype=torch.bfloat16).pin_memory() for _ in range(DEPTH)]
    y2_host = [torch.empty((mr, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(DEPTH)]
    x_dev = [torch.empty_like(x) for _ in range(DEPTH)]
    h_dev = [torch.empty_like(h) for _ in range(DEPTH)]
    s_in, s_comp, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
    ev_in = [torch.cuda.Event() for _ in range(DEPTH)]
    ev_comp = [torch.cuda.Event() for _ in range(DEPTH)]
    ev_out = [torch.cuda.Event() for _ in range(DEPTH)]
    ev_y2 = [torch.cuda.Event() for _ in range(DEPTH)]
    step_no = [0]
    row.overlap_chunks = 1

    def e2e_step():
        i = step_no[0]
        step_no[0] += 1
        b = i % DEPTH
        with torch.cuda.stream(s_in):
            if i >= DEPTH:
                s_in.wait_event(ev_comp[b])          # the device input buffers of step i - DEPTH have been consumed
            x_dev[b][rank * mr:(rank + 1) * mr].copy_(x_host, non_blocking=True)
            h_dev[b].copy_(h_host, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(ev_in[b])
            if world > 1:
                dist.all_gather_into_tensor(x_dev[b], x_dev[b][rank * mr:(rank + 1) * mr])
            y1 = col(x_dev[b])
            if ar is not None and i >= 1:
                # the summed outputs live in the one symmetric buffer: the previous step's copy-out of it must be done
                s_comp.wait_event(ev_y2[(i - 1) % DEPTH])
            y2 = row(h_dev[b])
            ev_comp[b].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])
            y1.record_stream(s_out)
            y2.record_stream(s_out)
            y2_host[b].copy_(y2[rank * mr:(rank + 1) * mr], non_blocking=True)
            ev_y2[b].record(s_out)
            y1_host[b].copy_(y1, non_blocking=True)
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
    t2, t3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t2.record()
    for st_ in (s_in, s_comp, s_out):
        st_.wait_stream(torch.cuda.current_stream())
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()
    t3.record()
    barrier()
    e2e_ms = t2.elapsed_time(t3) / e2e_steps
    dbg("end-to-end region done")

    times = torch.tensor([ms, e2e_ms, sustained_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, sustained_ms = float(times[0]), float(times[1]), float(times[2])
    status_ok = gemm_status_ok()
    if snaps:
        print(f"[bench r{rank}] all-reduce status after each stage: " + "; ".join(f"{m_}={int(h_[0])}" for m_, h_ in snaps),
              file=sys.stderr, flush=True)
    if ar is not None:
        ar.check()

    # ---- extra keys (outside every timed region above)
    extras = {}
    del x_dev, h_dev, y1_host, y2_host
    if not args.skip_extras:
        c3 = llama_config3(dev, world, rank, ar)
        flat = torch.tensor([c3[n_][m_] for n_ in LLAMA for m_ in ("128", "8192")], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(flat, op=dist.ReduceOp.MAX)
        it = iter(flat.tolist())
        cfg3 = {}
        for n_, (kind, n, k) in LLAMA.items():
            cfg3[n_] = {"parallel": "column (N split, no collective)" if kind == "col" else
                        ("row (K split + all-reduce of the bf16 partial outputs)" if world > 1 else "row (K split)"),
                        "N": n, "K": k}
            for m_ in ("128", "8192"):
                t_ms = next(it)
                cfg3[n_][f"M{m_}_ms"] = t_ms
                cfg3[n_][f"M{m_}_tflops"] = 2.0 * int(m_) * n * k / (t_ms * 1e-3) / 1e12
        cfg3["note"] = (f"Llama-3-70B projections over {world} GPU(s): quantisation + GEMM" +
                        (" + all-reduce" if world > 1 else "") + ", graph replay, max over ranks")
        extras["config3"] = cfg3
        if world == 1:
            del w1q, w1s, w2q, w2s, col, row
            torch.cuda.empty_cache()
            extras["quant"] = quant_config2(dev, pk)
            extras["config4"] = moe_config4_single(dev, pk)
            extras["fp8_ceiling_tflops"] = fp8_ceiling(dev)
            try:
                extras["ue8m0_path"] = ue8m0_mlp(dev, extras["fp8_ceiling_tflops"])
            except Exception as e:  # noqa: BLE001
                extras["ue8m0_path"] = {"unavailable": str(e)[:300]}
            try:
                extras["gpu_comparator"] = gpu_comparator(dev)
            except Exception as e:  # noqa: BLE001
                extras["gpu_comparator"] = {"unavailable": f"comparator failed: {str(e)[:300]}"}
        else:
            cfg4, ep_ok = moe_config4_ep(dev, world, rank)
            extras["config4"] = cfg4
            parity["expert_parallel_bitwise_ok"] = ep_ok
            parity["ok"] = parity["ok"] and ep_ok
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        gemm_ms = per_kernel["gemm_gate_up"]
        gemm_flops = 2.0 * M_TOKENS * n1 * HIDDEN
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
        peak_burst = 2.0 * pk["bf16_burst"]
        peak_sust = 2.0 * pk["bf16_sustained"]
        sus_clk = sampler.window("sus0", "sus1")
        burst_clk = sampler.window("burst0", "burst1")
        sustained_tflops = FLOPS_PER_STEP / (sustained_ms * 1e-3) / 1e12
        from sglang_b200.sgl_kernel.gemm import _splitk_plan
        split1 = _splitk_plan(M_TOKENS, n1, HIDDEN, dev)[0] > 1
        rows2 = M_TOKENS // chunks_used
        split2 = _splitk_plan(rows2, HIDDEN, k2, dev)[0] > 1
        launches_per_step = (1 + 1 + int(split1)) + chunks_used * (1 + 1 + int(split2)) + (chunks_used if ar is not None else 0)
        h2d = x_host.numel() * 2 + h.numel() * 2
        d2h = M_TOKENS * n1 * 2 + mr * HIDDEN * 2
        roof = {"bound": "tensor", "kernel": "gemm_block_fp8_kernel<BLOCK_N=256, 16 epilogue warps, 32-column chunks, bf16> "
                                             f"(gate_up{'' if world == 1 else f' shard N={n1}'})",
                "achieved": achieved, "peak": peak_burst, "unit": "TFLOP/s", "frac": achieved / peak_burst,
                "peak_source": f"2 x bf16_tflops (burst) of {pk['src']}: the kernel is timed with events inside a short eager pass "
                               "of the step, and the fp8 pipe does twice the bf16 MACs per clock (the file holds no fp8 entry)",
                "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
                "traffic": GEMM_TRAFFIC_BYTES_1GPU if world == 1 else None,
                "algorithmic_flops_per_launch": gemm_flops,
                "sustained": {"step_tflops": sustained_tflops, "ms_per_step": sustained_ms, "seconds": sustained_ms * reps / 1e3,
                              "sm_mhz_median": sus_clk["sm_mhz"] if sus_clk else None,
                              "power_w_max": sus_clk["power_w_max"] if sus_clk else None,
                              "peak": peak_sust * world, "frac": sustained_tflops / (peak_sust * world),
                              "peak_source": f"{world} GPU(s) x 2 x bf16_tflops_sustained of {pk['src']} (whole step, all "
                                             "ranks, back to back for >= 2 s)"}}
        if extras.get("fp8_ceiling_tflops"):
            roof["fp8_ceiling_measured"] = extras["fp8_ceiling_tflops"]
            roof["frac_of_fp8_ceiling"] = achieved / extras["fp8_ceiling_tflops"]
            roof["fp8_ceiling_source"] = "torch._scaled_mm, per-tensor e4m3, 8192^3, this run (yardstick only)"
        line = {
            "metric": "block_fp8_linear_tflops", "value": FLOPS_PER_STEP / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 -> bf16",
            "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "parallelism": (f"tp{world}: gate_up column-parallel, down row-parallel in {chunks_used} row chunk(s), "
                                       f"partial outputs summed by {'this library NVLink all-reduce kernel' + (' (multicast, on ' + str(reserve_used) + ' SMs the GEMMs leave free)' if reserve_used else (' (multicast)' if ar.multicast else ' (peer pointers)')) if ar is not None else 'NCCL all-reduce'}"
                                       ) if world > 1 else "single",
                       "timing": "step replayed from a CUDA graph at every N; per-kernel times from a separate eager pass with events around each call, at every N",
                       "l2": "inputs larger than L2 (weights 396 MB e4m3 + activations 210 MB bf16 per step)",
                       "kernels_ms": per_kernel,
                       **({"row_chunk_candidates_ms": chunk_ms} if world > 1 else {}),
                       **({"all_reduce_forms_us": ar_forms_us} if ar is not None else {})},
            "parity": parity,
            "e2e": {"value": FLOPS_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "note": "every step copies its activations from pinned host memory and its bf16 results back; the "
                            "copy-in / compute / copy-out legs of consecutive steps overlap on three streams (double "
                            "buffers); weights stay resident (they are layer parameters); bytes are per rank: each rank "
                            "moves 1/p of every replicated tensor"},
            "gpu_launches": args.steps * launches_per_step,
            "roofline": roof,
            "clocks": {**(clocks or {}), "burst_region": burst_clk, "sustained_region": sus_clk},
            "status_ok": status_ok,
        }
        for k_ in ("quant", "config3", "config4", "ue8m0_path", "gpu_comparator"):
            if k_ in extras:
                line[k_] = extras[k_]
        if world == 1 and not args.skip_extras:
            _, _, info = cpu_reference_run(steps=5, warmup=1, sample_rows=M_TOKENS)
            line["cpu_baseline"] = info
        print(json.dumps(line))
        sys.stdout.flush()
    rc = 0 if (parity["ok"] and status_ok) else 3
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        guard = threading.Timer(20.0, lambda: os._exit(rc))
        guard.daemon = True
        guard.start()
        dist.destroy_process_group()
        guard.cancel()
    if rc != 0:
        print(f"[bench rank {rank}] self-check failed: {json.dumps(parity)}", file=sys.stderr, flush=True)
        sys.exit(rc)


def run_kernel_case(args):
    """One kernel alone on one GPU (used for the M sweeps and as the small case for ncu captures):
    --kernel gemm_gate_up|gemm_down|gemm|quant|moe --m M.  Prints one JSON line per case."""
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
            # DeepSeek-V3 MoE layer on one GPU: `--experts` experts, top-8, hidden 7168, intermediate 2048.
            # Codes and scales are drawn directly (11.3 GB of weights); parity is covered by the tests.
            from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8
            E, H, I, topk = args.experts, 7168, 2048, 8
            w13, w2, w13s, w2s = moe_weights(dev, list(range(E)), 5000)
            x, tw, ti = moe_routing(dev, m, E=E)

            if args.scales == "pow2":
                from sglang_b200.layers.moe.cutlass_moe import fused_experts_block_fp8_ue8m0 as fused_experts_block_fp8
                w13s.copy_(torch.exp2(torch.ceil(torch.log2(w13s))))
                w2s.copy_(torch.exp2(torch.ceil(torch.log2(w2s))))

            def fn():
                return fused_experts_block_fp8(x, w13, w2, w13s, w2s, tw, ti)
            work, unit, peak = 2.0 * m * topk * (2 * I * H + H * I) / 1e12, "TFLOP/s", 2.0 * pk["bf16_burst"]
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
            it = [0]
            if args.scales == "pow2":
                # power-of-two scales on both sides: the block-scaling MMA (gemm_mx.cu)
                from sglang_b200.layers.quantization.fp8_kernel import w8a8_block_fp8_matmul_deepgemm
                from sglang_b200.layers.quantization.fp8_utils import requant_weight_ue8m0
                copies = [requant_weight_ue8m0(wq, ws, [128, 128]) for wq, ws in copies]
                xq, xs_ = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True,
                                                           scale_ue8m0=True)

                def fn():
                    it[0] += 1
                    wq, ws = copies[it[0] % ncopy]
                    return w8a8_block_fp8_matmul_deepgemm(xq, wq, xs_, ws, [128, 128], torch.bfloat16,
                                                          weight_scale_ue8m0=True)
            else:
                xq, xs_ = sglang_per_token_group_quant_fp8(x, 128, column_major_scales=True)
                views = [(wq.T, ws.T) for wq, ws in copies]

                def fn():
                    it[0] += 1
                    w_t, ws_t = views[it[0] % ncopy]
                    return fp8_blockwise_scaled_mm(xq, w_t, xs_, ws_t, torch.bfloat16)
            work, unit, peak = 2.0 * m * n * k / 1e12, "TFLOP/s", 2.0 * pk["bf16_burst"]
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
        rec = {"kernel": (args.kernel if args.kernel != "gemm" else f"gemm N={args.n} K={args.k}") +
               (" (power-of-two scales)" if args.scales == "pow2" and args.kernel != "quant" else ""), "M": m,
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
    ap.add_argument("--scales", default="fp32", choices=["fp32", "pow2"],
                    help="--kernel gemm*: fp32 scales (promotion kernels) or power-of-two scales (block-scaling MMA)")
    ap.add_argument("--experts", type=int, default=256,
                    help="--kernel moe: experts held on this GPU (256 = whole layer, 32 = one rank of 8)")
    ap.add_argument("--tp-chunks", type=int, default=0, choices=[0, 1, 2, 4, 8],
                    help="N > 1: row chunks of the row-parallel projection whose all-reduces overlap the next chunk "
                         "(0 = measure 1, 2 and 4 during warm-up and take the fastest)")
    ap.add_argument("--allreduce", default="custom", choices=["custom", "nccl"],
                    help="N > 1: this library's NVLink all-reduce kernels, or NCCL")
    ap.add_argument("--skip-extras", action="store_true", help="only the headline workload (no config3/config4/quant keys)")
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
