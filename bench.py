"""Benchmark of the block-FP8 W8A8 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--sections main,moe,tp]

Workload (BASELINE config 1): the six DeepSeek-V3 dense layers at M = 4096 tokens.  One step = for each
layer: quantise a bf16 activation [M,K] into 1x128 FP8 groups, then the 128x128 block-scaled GEMM
against that layer's [N,K] FP8 weight (bf16 out).  Metric: TFLOP/s = sum(2*M*N*K) / time, whole job.
With N > 1 ranks every rank runs its own batch (weak scaling, no data-path collective); the tensor-
and expert-parallel layers of configs 2 and 3, which do have collectives, are reported beside it under
"tp_layer" and "moe_layer".

Inputs are synthetic (seeded N(0,1) activations, N(0,0.02) weights quantised per 128x128 block) with the
shapes of the DeepSeek-V3 / Llama-3-70B checkpoints, which are not needed.  The per-step working set
(583 MB of weights + activations + outputs) is larger than the 126 MB L2, so no flush is used.

--impl reference times the reference's own CPU kernels (sgl-kernel fp8_scaled_mm_cpu, compiled into
oracle/_ref) on the host cores for the same layers on a bounded row sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# (name, N, K) of BASELINE config 1
DSV3_LAYERS = [
    ("fused_qkv_a", 2112, 7168), ("q_b", 24576, 1536), ("kv_b", 32768, 512),
    ("o_proj", 7168, 16384), ("gate_up", 36864, 7168), ("down", 7168, 18432),
]
M_TOKENS = 4096
METRIC = "block-FP8 GEMM TFLOPS (quantize + 128x128 block-scaled GEMM, DeepSeek-V3 dense layers, M=4096)"
FP8_NOMINAL_TFLOPS = 4500.0


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# CPU side: the reference's own kernels (oracle/_ref) or, failing that, the oracle port
# ------------------------------------------------------------------------------------------------


def _cpu_flags_ok() -> bool:
    try:
        flags = open("/proc/cpuinfo").read()
    except OSError:
        return False
    return all(f in flags for f in ("avx512f", "avx512_bf16", "amx_bf16"))


def _load_ref_cpu():
    import torch
    so = os.path.join(ROOT, "oracle", "_ref", "libsgl_cpu_ref.so")
    if os.path.exists(so) and _cpu_flags_ok():
        torch.ops.load_library(so)
        return "reference"
    return "port"


def cpu_reference_pass(rows: int, steps: int, warmup: int):
    """Times `steps` passes of the six layers on `rows` tokens on the host cores.  Returns
    (kind, cores, seconds per pass, flops per pass)."""
    import numpy as np
    import torch
    kind = _load_ref_cpu()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    layers = []
    for name, N, K in DSV3_LAYERS:
        x = torch.randn(rows, K, generator=g).bfloat16()
        wq = torch.randint(0, 0x78, (N, K), generator=g, dtype=torch.uint8)
        wq = (wq | (torch.randint(0, 2, (N, K), generator=g, dtype=torch.uint8) << 7)).view(torch.float8_e4m3fn)
        ws = torch.rand((N + 127) // 128, K // 128, generator=g) * 1e-3 + 1e-4
        if kind == "reference":
            wq = torch.ops.sgl_cpu_ref.convert_weight_packed(wq)
        layers.append((x, wq, ws))
    flops = sum(2.0 * rows * N * K for _, N, K in DSV3_LAYERS)

    def one_pass():
        for x, wq, ws in layers:
            if kind == "reference":
                torch.ops.sgl_cpu_ref.fp8_scaled_mm_cpu(x, wq, ws, [128, 128], None, torch.bfloat16, True)
            else:
                from oracle import block_fp8_oracle as O
                O.block_fp8_linear(x.float().numpy(), wq.view(torch.uint8).numpy(), ws.numpy())

    for _ in range(warmup):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return kind, cores, dt, flops


def _rand_fp8_weight(shape, g):
    """Random e4m3 codes without NaN patterns (exponent-and-mantissa field below 0x78) and random signs."""
    import torch
    q = torch.randint(0, 0x78, shape, generator=g, dtype=torch.uint8)
    return (q | (torch.randint(0, 2, shape, generator=g, dtype=torch.uint8) << 7)).view(torch.float8_e4m3fn)


def cpu_config0():
    """BASELINE config 0 on the host cores: one block-FP8 linear, M = 64, N = K = 4096, through the reference's
    fp8_scaled_mm_cpu (or the oracle port where that library is not usable)."""
    import torch
    try:
        kind = _load_ref_cpu()
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        g = torch.Generator().manual_seed(0)
        M, N, K = 64, 4096, 4096
        x = torch.randn(M, K, generator=g).bfloat16()
        wq = _rand_fp8_weight((N, K), g)
        ws = torch.rand(N // 128, K // 128, generator=g) * 1e-3 + 1e-4
        if kind == "reference":
            wp = torch.ops.sgl_cpu_ref.convert_weight_packed(wq)
            fn = lambda: torch.ops.sgl_cpu_ref.fp8_scaled_mm_cpu(x, wp, ws, [128, 128], None, torch.bfloat16, True)
        else:
            from oracle import block_fp8_oracle as O
            xn, wn, sn = x.float().numpy(), wq.view(torch.uint8).numpy(), ws.numpy()
            fn = lambda: O.block_fp8_linear(xn, wn, sn)
        for _ in range(3):
            fn()
        iters = 50 if kind == "reference" else 2
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        dt = (time.perf_counter() - t0) / iters
        return {"workload": "BASELINE config 0: M=64, N=K=4096 block-FP8 linear", "kind": kind, "cores": cores,
                "ms": dt * 1e3, "tflops": 2.0 * M * N * K / dt / 1e12}
    except Exception as e:  # a reported extra: never breaks the line
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


def cpu_moe_baseline():
    """The reference's CPU MoE (sgl-kernel fused_experts_cpu, FP8 weights dequantised on the fly = W8A16, AMX) on the
    host cores for the MoE layers of BASELINE configs 3 and 4 at reduced token counts.  Config 3's 256 experts are 32
    distinct random experts repeated eight times (the kernel reads every expert's own copy; 11 GB of codes)."""
    import torch
    out = {}
    try:
        if _load_ref_cpu() != "reference":
            return {"unavailable": "oracle/_ref/libsgl_cpu_ref.so is not usable on this host (needs AVX512-BF16 + AMX)"}
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        ops = torch.ops.sgl_cpu_ref
        for name, E, H, I, topk, T, distinct in (("config3_T512", 256, 7168, 2048, 8, 512, 32),
                                                 ("config4_T1024", 128, 2048, 768, 8, 1024, 128)):
            g = torch.Generator().manual_seed(3)
            w13 = ops.convert_weight_packed(_rand_fp8_weight((distinct, 2 * I, H), g)).repeat(E // distinct, 1, 1)
            w2 = ops.convert_weight_packed(_rand_fp8_weight((distinct, H, I), g)).repeat(E // distinct, 1, 1)
            w13s = torch.rand(E, 2 * I // 128, H // 128, generator=g) * 1e-3 + 1e-4
            w2s = torch.rand(E, H // 128, I // 128, generator=g) * 1e-3 + 1e-4
            x = torch.randn(T, H, generator=g).bfloat16()
            tw, ti = torch.topk(torch.softmax(torch.randn(T, E, generator=g), -1), topk)
            ti = ti.to(torch.int32)
            tw = tw.float().contiguous()
            fn = lambda: ops.fused_experts_cpu(x, w13, w2, tw, ti, False, False, True, w13s, w2s, [128, 128], None, None, True)
            fn()
            t0 = time.perf_counter()
            iters = 3
            for _ in range(iters):
                fn()
            dt = (time.perf_counter() - t0) / iters
            out[name] = {"ms": dt * 1e3, "tokens_per_s": T / dt, "tflops": 6.0 * T * topk * H * I / dt / 1e12}
            del w13, w2
        return {"kernel": "sgl-kernel fused_experts_cpu, use_fp8_w8a16 (the CPU path does not quantise activations)",
                "kind": "reference", "cores": cores, "routed_experts_only": True, "results": out}
    except Exception as e:
        out["unavailable"] = f"{type(e).__name__}: {e}"[:200]
        return out


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = CPU_SAMPLE_ROWS
    kind, cores, dt, flops = cpu_reference_pass(rows, args.steps, args.warmup)
    v = flops / dt / 1e12
    sample = f"{rows} of {M_TOKENS} token rows through all six layers per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations x fp8 weights (W8A16), f32 accumulate",
        "data": "synthetic", "config": _config(),
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "sgl-kernel fp8_scaled_mm_cpu (AMX brgemm) on the host cores; the CPU path does not quantise activations",
    }
    gpu_ref = reference_gpu_kernel(args)
    if gpu_ref is not None:
        line["reference_gpu_kernel"] = gpu_ref
    line["config0"] = cpu_config0()
    line["moe_cpu_baseline"] = cpu_moe_baseline()
    print(json.dumps(line), flush=True)


def reference_gpu_kernel(args):
    """Extra, rank 0 only: the reference's own CUDA block-FP8 GEMM (oracle/_ref/libsgl_gpu_ref.so, its
    fp8_blockwise_gemm_kernel.cu compiled unmodified for sm_100a) timed on this box's GPU over the layers of the
    workload it accepts (it wants N to be a multiple of 128, which leaves out N = 2112), M = 4096, inputs resident,
    the layers run back to back so that the weights (583 MB) do not stay in L2.  Not part of `value`."""
    lib = os.path.join(ROOT, "oracle", "_ref", "libsgl_gpu_ref.so")
    try:
        import torch
        if not (os.path.exists(lib) and torch.cuda.is_available()):
            return None
        torch.ops.load_library(lib)
        mm = torch.ops.sgl_gpu_ref.fp8_blockwise_scaled_mm
        dev = torch.device("cuda", 0)
        gen = torch.Generator(device=dev).manual_seed(1234)
        M = M_TOKENS
        layers = []
        for name, N, K in DSV3_LAYERS:
            if N % 128:
                continue
            wq, ws = make_block_fp8_weight(N, K, dev, gen)
            x = torch.randn(M, K, device=dev, generator=gen)
            g = x.view(M, K // 128, 128)
            xs = (g.abs().amax(-1).clamp_min(1e-10) / 448.0)
            xq = (g / xs.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn).view(M, K)
            layers.append((name, N, K, xq, xs.t().contiguous().t(), wq.t(), ws.t()))
        per = {}
        def step(record=None):
            for name, N, K, xq, xs, wt, wst in layers:
                if record is not None:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                mm(xq, wt, xs, wst, torch.bfloat16)
                if record is not None:
                    e1.record()
                    record.append((name, 2.0 * M * N * K, e0, e1))
        for _ in range(max(3, args.warmup)):
            step()
        torch.cuda.synchronize()
        rec = []
        for _ in range(args.steps):
            step(rec)
        torch.cuda.synchronize()
        for name, fl, e0, e1 in rec:
            d = per.setdefault(name, [0.0, 0.0])
            d[0] += e0.elapsed_time(e1)
            d[1] += fl
        tot_ms = sum(d[0] for d in per.values())
        tot_fl = sum(d[1] for d in per.values())
        return {"kernel": "sgl-kernel fp8_blockwise_scaled_mm (CUTLASS sm100 blockwise, 128x128x128 tiles)",
                "M": M, "unit": "TFLOP/s", "gemm_tflops": tot_fl / (tot_ms / 1e3) / 1e12,
                "per_layer_tflops": {n: d[1] / (d[0] / 1e3) / 1e12 for n, d in per.items()},
                "compare_with": "roofline.per_layer_tflops of the default arm (same shapes, same timing)"}
    except Exception as e:  # the comparator is optional: never let it break the reference arm
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


CPU_SAMPLE_ROWS = 1024  # token rows of the workload that the CPU legs run per step (scaled by FLOP)


def _config():
    return {
        "workload": "BASELINE config 1: DeepSeek-V3 dense block-FP8 layers "
                    "(N,K) in {(2112,7168),(24576,1536),(32768,512),(7168,16384),(36864,7168),(7168,18432)} at M=4096",
        "M": M_TOKENS, "block": [128, 128], "group": 128,
        "M_sample": f"the CPU legs (cpu_baseline, --impl reference) run {CPU_SAMPLE_ROWS} of the {M_TOKENS} rows per step",
        "l2": "per-step working set (583 MB weights + activations + outputs) exceeds the 126 MB L2; no flush",
    }


# ------------------------------------------------------------------------------------------------
# GPU side
# ------------------------------------------------------------------------------------------------


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.idx = device_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in out.strip().splitlines():
            f = [c.strip() for c in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def _smi_device_id(local_index: int) -> str:
    """nvidia-smi id of CUDA device `local_index` (honours CUDA_VISIBLE_DEVICES, indices or UUIDs)."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v.strip() for v in vis.split(",") if v.strip()]
        if local_index < len(ids):
            return ids[local_index]
    return str(local_index)


def make_block_fp8_weight(N, K, device, gen, std=0.02, experts=None):
    """N(0,std) weights quantised per 128x128 block on the device (scale = block amax / 448)."""
    import torch
    lead = () if experts is None else (experts,)
    nb, kb = (N + 127) // 128, (K + 127) // 128
    w = torch.zeros(*lead, nb * 128, kb * 128, device=device)
    w[..., :N, :K] = torch.randn(*lead, N, K, device=device, generator=gen) * std
    blk = w.view(*lead, nb, 128, kb, 128)
    s = blk.abs().amax(dim=(-3, -1), keepdim=True) / torch.full((), 448.0, device=device)
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = (blk / s).clamp(-448, 448).to(torch.float8_e4m3fn).view(*lead, nb * 128, kb * 128)[..., :N, :K].contiguous()
    return q, s.view(*lead, nb, kb).contiguous()


def measure_fp8_peak(dev):
    """Dense FP8 tensor throughput of this GPU as the vendor library reaches it: torch._scaled_mm (cuBLASLt), per-tensor
    scales, 8192^3, bf16 out; best of a burst of 10 and the mean of the burst.  None when the call is not available."""
    import torch
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()  # column-major second operand
        one = torch.ones((), device=dev)
        f = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
        for e0, e1 in ev:
            e0.record()
            f()
            e1.record()
        torch.cuda.synchronize()
        ms = [e0.elapsed_time(e1) for e0, e1 in ev]
        fl = 2.0 * n ** 3
        return {"best": fl / min(ms) / 1e9, "mean": fl / (sum(ms) / len(ms)) / 1e9}
    except Exception:
        return None


def run_main(args, dist_ctx):
    import torch
    from sglang_b200 import ops
    from sglang_b200._lib import lib as _lib
    from sglang_b200.srt.layers.linear import ColumnParallelLinear
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config

    rank, world, dev = dist_ctx
    peaks = _peaks()
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    cfg = Fp8Config(weight_block_size=[128, 128])
    M = args.m_tokens
    layers = []
    for name, N, K in DSV3_LAYERS:
        if args.layers and name not in args.layers.split(","):
            continue
        lin = ColumnParallelLinear(K, N, quant_config=cfg, device=dev)  # tp group of 1 here: full weights
        wq, ws = make_block_fp8_weight(N, K, dev, gen)
        lin.weight.data.copy_(wq)
        lin.weight_scale_inv.data.copy_(ws)
        del wq, ws
        x_host = torch.randn(M, K, generator=torch.Generator().manual_seed(rank * 100 + len(layers))).bfloat16().pin_memory()
        x_dev = x_host.to(dev)
        y_host = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
        layers.append(dict(name=name, N=N, K=K, lin=lin, x_host=x_host, x_dev=x_dev, y_host=y_host))
    torch.cuda.empty_cache()
    flops_step = sum(2.0 * M * l["N"] * l["K"] for l in layers)
    stream = torch.cuda.current_stream()

    gemm_ev = []

    def step_resident(record=False):
        for l in layers:
            xq, xs = ops.per_token_group_quant_fp8(l["x_dev"], 128)
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            y = ops.w8a8_block_fp8_matmul(xq, l["lin"].weight, xs, l["lin"].weight_scale_inv, [128, 128], torch.bfloat16)
            if record:
                e1.record(stream)
                gemm_ev.append((e0, e1, 2.0 * M * l["N"] * l["K"], l["name"]))
        return y

    # End to end: host tensors in, host tensors out, through the public layer call.  Three streams, as a serving
    # loop would run it: the input copy of layer i+1 and the output copy of layer i-1 travel (PCIe is full duplex)
    # while layer i computes.  Device buffers are per layer; events order their reuse from one step to the next.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    for l in layers:
        l["x_stage"] = torch.empty_like(l["x_dev"])
        l["ev_in"], l["ev_done"], l["ev_out"] = (torch.cuda.Event() for _ in range(3))

    def step_e2e():
        for l in layers:
            with torch.cuda.stream(s_in):
                s_in.wait_event(l["ev_done"])  # the previous step's GEMM has consumed the staging buffer
                l["x_stage"].copy_(l["x_host"], non_blocking=True)
                l["ev_in"].record(s_in)
            stream.wait_event(l["ev_in"])
            y, _ = l["lin"](l["x_stage"])  # Fp8LinearMethod.apply: quantise + block GEMM
            l["ev_done"].record(stream)
            y.record_stream(s_out)
            with torch.cuda.stream(s_out):
                s_out.wait_event(l["ev_done"])
                l["y_host"].copy_(y, non_blocking=True)
                l["ev_out"].record(s_out)
        for l in layers:  # the step ends when its last output byte is on the host
            stream.wait_event(l["ev_out"])

    def timed(fn, steps, warmup, **kw):
        for _ in range(warmup):
            fn()
        _barrier(world)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn(**kw)
        e1.record(stream)
        torch.cuda.synchronize()
        _barrier(world)
        return _max_over_ranks(e0.elapsed_time(e1) / 1e3, world, dev)

    sampler = ClockSampler(_smi_device_id(dev.index))
    sampler.start()
    t_res = timed(step_resident, args.steps, args.warmup, record=True)
    clocks = sampler.stop()
    t_e2e = timed(step_e2e, args.steps, max(args.warmup, 3))
    assert ops.gemm_status() == 0, "a GEMM pipeline wait expired during the benchmark"

    # dominant kernel: the block-scaled GEMM.  Per-launch durations from the events recorded in the timed region.
    gemm_ms = sum(a.elapsed_time(b) for a, b, _, _ in gemm_ev)
    gemm_flops = sum(f for _, _, f, _ in gemm_ev)
    achieved = gemm_flops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else 0.0
    per_layer = {}
    for a, b, f, n in gemm_ev:
        d = per_layer.setdefault(n, [0.0, 0.0])
        d[0] += a.elapsed_time(b)
        d[1] += f
    # One denominator everywhere (this line and the per-M sweep): the FP8 rate the vendor library reaches on THIS GPU in
    # THIS run (cuBLASLt per-tensor FP8, 8192^3, burst); where that call is unavailable, twice the measured burst bf16
    # rate of MEASURED_PEAKS.json.  The other two yard-sticks are printed beside the fraction.
    fp8 = measure_fp8_peak(dev)
    peak = fp8["best"] if fp8 else 2.0 * peaks["bf16"]
    peaks["fp8_measured"] = peak
    value = world * flops_step * args.steps / t_res / 1e12
    e2e = world * flops_step * args.steps / t_e2e / 1e12
    h2d = sum(l["x_host"].numel() * 2 for l in layers)
    d2h = sum(l["y_host"].numel() * 2 for l in layers)
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t_res / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3, f32 accumulate, bf16 out", "data": "synthetic",
        "config": _config(), "clocks": clocks,
        "e2e": {"value": e2e, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": t_e2e / args.steps * 1e3,
                "api": "ColumnParallelLinear.forward -> Fp8LinearMethod.apply on pinned host tensors; input / compute / output streams"},
        # per layer: the quantizer, the GEMM, and the partial-sum reduction where the GEMM splits tiles along K
        "gpu_launches": args.steps * sum(2 + (1 if _lib.sglb200_gemm_workspace_bytes(M, l["N"], l["K"]) > 0 else 0)
                                         for l in layers),
        "roofline": {
            "kernel": "fp8_blockscale_gemm_kernel<false>", "bound": "tensor", "achieved": achieved, "peak": peak,
            "unit": "TFLOP/s", "frac": achieved / peak if peak else None, "traffic": _gemm_traffic(M, layers),
            "peak_source": ("torch._scaled_mm (cuBLASLt) per-tensor FP8 8192^3 timed in this run on this GPU, best of 10"
                            if fp8 else f"2 x bf16_tflops of MEASURED_PEAKS.json ({peaks['source']}); torch._scaled_mm unavailable"),
            "fp8_library_mean_of_burst": fp8["mean"] if fp8 else None,
            "frac_of_2x_burst_bf16": achieved / (2.0 * peaks["bf16"]),
            "frac_of_2x_sustained_bf16": achieved / (2.0 * peaks["bf16_sustained"]),
            "frac_of_nominal_fp8_4500": achieved / FP8_NOMINAL_TFLOPS,
            "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of the six GEMM launches of this workload in "
                              "one ncu capture (a constant of this file, not measured in this run); null for other workloads",
            "per_layer_tflops": {n: v[1] / (v[0] / 1e3) / 1e12 for n, v in per_layer.items()},
        },
    }
    return line, layers


# DRAM bytes (read + write) of the GEMM launches of one step of the default workload, from one ncu capture of
# `bench.py --steps 1 --warmup 1 --sections main --cpu-baseline 0` (dram__bytes_read.sum + dram__bytes_write.sum
# of the first six fp8_blockscale_gemm_kernel launches).  Algorithmic bytes
# of the same six launches: 1 706 MB (weights 583, activations 210, outputs 906, scales 7).
_GEMM_DRAM_BYTES_PER_STEP_M4096 = {"fused_qkv_a": 49.2e6, "q_b": 187.5e6, "kv_b": 226.1e6, "o_proj": 503.1e6,
                                   "gate_up": 577.2e6, "down": 689.9e6}


def _gemm_traffic(M, layers):
    """Average DRAM bytes per GEMM launch, or None when the run is not the captured workload."""
    names = [l["name"] for l in layers]
    if M != M_TOKENS or any(n not in _GEMM_DRAM_BYTES_PER_STEP_M4096 for n in names):
        return None
    return sum(_GEMM_DRAM_BYTES_PER_STEP_M4096[n] for n in names) / len(names)


def _barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def _max_over_ranks(seconds, world, dev):
    if world == 1:
        return seconds
    import torch
    import torch.distributed as dist
    t = torch.tensor([seconds], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--sections", default="main,moe,tp,sweep,hbm",
                    help="main is always run; moe = moe3 (config 3) + moe4 (config 4, skewed), tp, sweep, hbm")
    ap.add_argument("--cpu-baseline", type=int, default=1)
    ap.add_argument("--layers", default="", help="comma-separated subset of layer names (profiler captures only)")
    ap.add_argument("--m-tokens", type=int, default=M_TOKENS, help="smaller values are for profiler captures only")
    ap.add_argument("--moe-experts", type=int, default=0, help="config-3 MoE section with this many experts "
                                                                "(profiler captures only; 0 = the 256 of the config)")
    ap.add_argument("--moe-tokens", type=int, default=0, help="config-3 MoE section at this one token count "
                                                               "(profiler captures only; 0 = the sizes of the config)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from sglang_b200._lib import check, lib
    check(lib.sglb200_check_device(local))
    sections = set(args.sections.split(","))

    cpu = None
    if rank == 0 and world == 1 and args.cpu_baseline:
        rows = CPU_SAMPLE_ROWS
        kind, cores, dt, flops = cpu_reference_pass(rows, 3, 1)
        cpu = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind,
               "sample": f"{rows} of {M_TOKENS} token rows through all six layers, 3 timed passes after 1 warm-up"}

    cpu_extra = {}
    if rank == 0 and world == 1 and args.cpu_baseline:
        cpu_extra = {"config0_cpu": cpu_config0(), "moe_cpu_baseline": cpu_moe_baseline()}
    line, layers = run_main(args, (rank, world, dev))
    if cpu is not None:
        line["cpu_baseline"] = cpu
    line.update(cpu_extra)
    del layers
    torch.cuda.empty_cache()
    extra = {}
    try:
        import bench_sections as bs  # optional extra sections live beside this file
        pk = _peaks()
        pk["fp8_measured"] = line["roofline"]["peak"]
        extra = bs.run(sections, args, (rank, world, dev), pk)
    except ImportError:
        pass
    line.update(extra)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
