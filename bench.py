"""Benchmark of the MX quantize-dequantize hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: MXFP8 (E4M3 elements, E8M0 scale, block 32) fake-quantization of one bf16 tensor [65536, 8192]
(Student-t(3) * 0.02, seeded), the largest shape of the quantizer sweep; 1 GiB in, 1 GiB out, so inputs exceed
the 126 MB L2 and no flush is needed between steps.  A step is one pass over that tensor.  With N > 1 every rank
processes its own tensor of that shape (row shards of an N-times taller tensor; blocks are independent, so there
is no collective) and the reported value is the aggregate ("weak" scaling).

  value   algorithmic GB/s (numel * (2 + 2) bytes per pass) with inputs resident in HBM, CUDA-event timed
  e2e     the same metric through the public API with pinned HOST buffers: host->device copy, quantize,
          device->host copy of the result inside the timed region (chunked over two streams)
  roofline  the fake-quant kernel against the measured HBM copy bandwidth
  cpu_baseline  MASE's own CPU quantizer (staged by oracle/stage_reference.py into oracle/_ref, kind "reference") or,
          where that is absent, the CPU port in oracle/ (kind "port"), on a bounded sample of the same tensor, rank 0
  extra   other formats / shapes of the sweep, the MX Linear forward, the mixed-precision decoder layer and the
          tensor-parallel Linear stack, measured outside the timed region.  The MX-Linear half of the metric is also
          nested in the contract's objects: roofline["mx_linear"], cpu_baseline["mx_linear"], roofline["peaks"].

`--impl reference` times the CPU implementation on the host cores instead (bounded sample per step).
"""

from __future__ import annotations

import argparse
import copy
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, COLS = 65536, 8192
BLOCK, EXP_BITS, FRAC_BITS = 32, 4, 3
BYTES_PER_ELEM = 4  # bf16 read + bf16 write
CPU_SAMPLE_ROWS = 2048
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per element (read + write) of the fake-quant kernel from an ncu capture of a smaller tensor of the
# same kernel (profiles/); None until measured.  Scales linearly with the element count.
NCU_DRAM_BYTES_PER_ELEM = 3.65


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_bf16_tflops() -> tuple[float, float, str]:
    """(burst, sustained, source) of the dense bf16 library GEMM from MEASURED_PEAKS.json, else the fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            d = json.load(fh)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


def measure_fp8_peak(device) -> dict:
    """FP8-rate tensor-core peak measured the way MEASURED_PEAKS.json measures bf16: the library FP8 GEMM
    (`torch._scaled_mm`, E4M3 x E4M3, per-tensor scales, bf16 output) at 8192^3, best of 10 launches (burst) and
    back to back for ~2 s (sustained).  Measurement only: nothing on the product path calls it."""
    n = 8192
    try:
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()  # column-major second operand
        one = torch.ones((), device=device, dtype=torch.float32)
        run = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        flops = 2.0 * n * n * n
        best = float("inf")
        for _ in range(10):
            s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_.record()
            run()
            e_.record()
            torch.cuda.synchronize()
            best = min(best, s_.elapsed_time(e_) / 1e3)
        reps = max(10, int(2.0 / best))
        s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_.record()
        for _ in range(reps):
            run()
        e_.record()
        torch.cuda.synchronize()
        sustained = flops * reps / (s_.elapsed_time(e_) / 1e3) / 1e12
        del a, b
        return {"fp8_tflops": flops / best / 1e12, "fp8_tflops_sustained": sustained,
                "how": f"torch._scaled_mm E4M3 x E4M3 (per-tensor scale, bf16 out) {n}^3: best of 10 (burst); {reps} "
                       "back to back (sustained); CUDA events"}
    except Exception as exc:  # library without an FP8 GEMM: the 2 x bf16 stand-in is used and labelled
        return {"fp8_tflops": None, "fp8_tflops_sustained": None, "how": f"unavailable: {type(exc).__name__}: {exc}"[:200]}


def tensor_peaks(device) -> dict:
    """Denominators of the tensor-bound rooflines: measured FP8-rate peak (this run), 2 x measured bf16, nominal."""
    bf16, bf16_sus, src = measured_bf16_tflops()
    pk = measure_fp8_peak(device)
    pk.update({"bf16_tflops": bf16, "bf16_tflops_sustained": bf16_sus, "bf16_source": src + " cuBLAS bf16 8192^3",
               "fp8_nominal_tflops": 4500.0, "bf16_nominal_tflops": 2250.0})
    if pk["fp8_tflops"]:
        pk["fp8_used"], pk["fp8_used_source"] = pk["fp8_tflops"], "measured library FP8 GEMM, burst (this run)"
    else:
        pk["fp8_used"], pk["fp8_used_source"] = 2.0 * bf16, f"2 x {src} bf16 burst (no FP8 library GEMM measured)"
    return pk


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed regions run (read-only)."""

    def __init__(self, device):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            try:  # the CUDA ordinal is not the NVML index when CUDA_VISIBLE_DEVICES is set: look up by UUID
                uuid = "GPU-" + str(torch.cuda.get_device_properties(device).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device.index or 0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "note": "NVML unavailable"}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def dist_env():
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    return rank, world, local


def cpu_quantizers():
    """The CPU implementation that is timed beside the GPU numbers: MASE's own `chop.nn.quantizers` when it has been
    staged into oracle/_ref (kind "reference"), else the restatement in oracle/mx_oracle.py (kind "port").
    Returns ({"mxfp": f(x, block, E, F), "mxint": f(x, block, bits)}, kind); both quantize along the last dim."""
    try:
        from oracle import stage_reference

        q = stage_reference.import_staged_quantizers()
        return {"mxfp": lambda x, block, e, f: q.mxfp_quantizer(x, block, e, f),
                "mxint": lambda x, block, bits: q.mxint_quantizer(x, block, bits),
                "mxfp_search": lambda x, block, e, f: q.mxfp_quantizer(x, block, e, f, -1, 8, True),
                "mxint_search": lambda x, block, bits: q.mxint_quantizer(x, block, bits, -1, 8, True)}, "reference"
    except Exception:
        from oracle import mx_oracle as O

        return {"mxfp": lambda x, block, e, f: O.mxfp_fake(x, block, e, f),
                "mxint": lambda x, block, bits: O.mxint_fake(x, block, bits)}, "port"


def cpu_quantizer_time(rows: int, repeats: int = 1) -> tuple[float, int, str]:
    """Seconds for the CPU implementation to fake-quantize `rows` rows of the workload; uses every host thread."""
    from mase_b200 import synthetic

    qs, kind = cpu_quantizers()
    fake = qs["mxfp"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = synthetic.student_t3(rows, COLS, seed=1)
    fake(x[:64], BLOCK, EXP_BITS, FRAC_BITS)  # warm-up
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fake(x, BLOCK, EXP_BITS, FRAC_BITS)
        best = min(best, time.perf_counter() - t0)
    return best, torch.get_num_threads(), kind


def cpu_linear_time(x: torch.Tensor, wq: torch.Tensor, e: int = 4, f: int = 3) -> tuple[float, str]:
    """Seconds for the CPU forward of an MX Linear on the rows of `x` the way MASE runs it
    (chop/nn/quantized/modules/linear.py:877-895): MXFP-quantize x along K, then `F.linear` in x.dtype against the
    weight that was quantized at load time."""
    qs, kind = cpu_quantizers()
    fake = qs["mxfp"]
    torch.set_num_threads(os.cpu_count() or 1)
    torch.nn.functional.linear(fake(x[:8], 32, e, f), wq)  # warm-up
    t0 = time.perf_counter()
    torch.nn.functional.linear(fake(x, 32, e, f), wq)
    return time.perf_counter() - t0, kind


def run_reference(args) -> None:
    """The CPU implementation of the path on the host cores; rank 0 only."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from mase_b200 import synthetic

    qs, kind = cpu_quantizers()
    fake = qs["mxfp"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = synthetic.student_t3(CPU_SAMPLE_ROWS, COLS, seed=1)
    for _ in range(args.warmup):
        fake(x[:256], BLOCK, EXP_BITS, FRAC_BITS)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fake(x, BLOCK, EXP_BITS, FRAC_BITS)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = CPU_SAMPLE_ROWS * COLS * BYTES_PER_ELEM / dt / 1e9
    sample = f"{CPU_SAMPLE_ROWS} of {ROWS} rows per step (one GPU's tensor; not multiplied by the number of GPUs)"
    print(json.dumps({
        "impl": "reference", "metric": "mx_quant_dequant_GBps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(n_gpus: int) -> dict:
    return {"workload": f"MXFP8-E4M3 block-32 fake-quant of bf16 [{ROWS},{COLS}] per GPU, Student-t(3)*0.02",
            "rows_per_gpu": ROWS, "cols": COLS, "block": BLOCK, "element": "E4M3", "scale": "E8M0",
            "sharding": f"rows x{n_gpus}, no collective", "l2": "inputs (1 GiB) exceed L2, no flush"}


def time_region(fn, steps: int, world: int, device) -> float:
    """Seconds for `steps` calls of fn, CUDA-event timed between barriers, max over ranks."""
    import torch.distributed as dist

    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sec = torch.tensor([start.elapsed_time(end) / 1e3], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(sec, op=dist.ReduceOp.MAX)
    return float(sec.item())


def quick_gbs(fn, bytes_per_call: int, calls: int = 10) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(calls):
        fn()
    e.record()
    torch.cuda.synchronize()
    return bytes_per_call * calls / (s.elapsed_time(e) / 1e3) / 1e9


def extras(device, x, peaks: dict) -> dict:
    """Other rows of the sweep, measured after the timed region (not part of `value`)."""
    import mase_b200 as mb
    from mase_b200 import synthetic

    out = {}
    n = x.numel()
    out["mxint8_bf16_65536x8192_GBps"] = quick_gbs(lambda: mb.mxint_quantizer(x, 32, 8), n * 4)
    out["bfp_w8_b32_bf16_65536x8192_GBps"] = quick_gbs(lambda: mb.block_fp_quantizer(x, 8, 8, 127, [1, 32], True), n * 4)
    out["bfp_w7_b16_bf16_65536x8192_GBps"] = quick_gbs(lambda: mb.block_fp_quantizer(x, 7, 8, 127, [1, 16], True), n * 4)
    out["mxfp4_e2m1_bf16_65536x8192_GBps"] = quick_gbs(lambda: mb.mxfp_quantizer(x, 32, 2, 1), n * 4)
    meta = mb.MXFPMeta(32, 8, 4, 3, True, "rn")
    out["mxfp8_pack_codes_bf16_65536x8192_GBps"] = quick_gbs(
        lambda: mb.extract_mxfp_components(x.view(-1), meta), int(n * (2 + 1 + 1 / 32)))
    from mase_b200 import gemm
    out["mxfp8_tensor_core_operands_bf16_65536x8192_GBps"] = quick_gbs(
        lambda: gemm.pack_mx_operand(x, 4, 3), int(n * (2 + 1 + 1 / 32)))
    out["mxint8_codes_bf16_65536x8192_GBps"] = quick_gbs(
        lambda: mb.mxint_codes(x.view(-1), 32, 8), int(n * (2 + 1 + 1 / 32)))
    # MXINT8 of fp32 [4096,4096] (N(0,1) with outliers): rotate 8 tensors (512 MB) so that HBM, not L2, is measured
    xs = [synthetic.normal_with_outliers(4096, 4096, seed=0).to(device) for _ in range(1)]
    xs = xs + [xs[0].clone() for _ in range(7)]
    state = {"i": 0}

    def f32_step():
        mb.mxint_quantizer(xs[state["i"] % 8], 32, 8)
        state["i"] += 1

    out["mxint8_fp32_4096x4096_GBps"] = quick_gbs(f32_step, 4096 * 4096 * 8, calls=16)
    del xs
    for shape in ((1, 4096), (128, 4096), (4096, 4096)):
        xx = synthetic.student_t3(*shape, seed=1).to(device)
        g = quick_gbs(lambda: mb.mxfp_quantizer(xx, 32, 4, 3), xx.numel() * 4, calls=50)
        out[f"mxfp8_bf16_{shape[0]}x{shape[1]}_us"] = xx.numel() * 4 / g / 1e3
    out["linear_mxfp8_4096x4096"] = linear_extras(device, peaks)
    out["decoder_layer_mixed_precision"] = decoder_layer_extras(device, peaks)
    for name, fn in (("calibration", lambda: calibration_extras(device)),
                     ("attention_block_mxfp8", lambda: attention_extras(device, peaks))):
        try:
            out[name] = fn()
        except Exception as exc:  # off the timed path: report instead of losing the line
            out[name] = {"error": repr(exc)}
    return out


def calibration_extras(device) -> dict:
    """Calibration-time work on one 4096 x 4096 weight: the clipping search of both formats (one kernel each) and a
    GPTQ sweep with the MXINT4 search inside, each with the CPU implementation timed on a bounded slice (the
    reference's own quantizers when staged, else the port; GPTQ always the port, on a 1024 x 1024 layer)."""
    import mase_b200 as mb
    from mase_b200 import gptq
    from oracle import mx_oracle as O

    out = {}
    g = torch.Generator().manual_seed(3)
    w = torch.randn(4096, 4096, generator=g) * 0.02
    w[torch.rand(4096, 4096, generator=g) < 0.01] *= 20
    wd = w.to(device).bfloat16()
    qs, kind = cpu_quantizers()
    torch.set_num_threads(os.cpu_count() or 1)
    int_meta, fp_meta = mb.MXIntMeta(32, 8, 4), mb.MXFPMeta(32, 8, 2, 1, True, "rn")
    rows = 256
    for name, gpu_fn, cpu_fn in (
            ("mxint4", lambda: mb.mxint_quantizer_sim(wd, 1, int_meta, quantile_search=True),
             (lambda x: qs["mxint_search"](x, 32, 4)) if "mxint_search" in qs else (lambda x: O.mxint_clip_search(x, 32, 4, 1))),
            ("mxfp4_e2m1", lambda: mb.mxfp_quantizer_sim(wd, 1, fp_meta, quantile_search=True),
             (lambda x: qs["mxfp_search"](x, 32, 2, 1)) if "mxfp_search" in qs else (lambda x: O.mxfp_clip_search(x, 32, 2, 1, 1)))):
        gbs = quick_gbs(gpu_fn, wd.numel() * 4)
        xs = w[:rows].bfloat16()
        cpu_fn(xs[:8])
        t0 = time.perf_counter()
        cpu_fn(xs)
        cpu_s = (time.perf_counter() - t0) * (4096 / rows)
        out[f"{name}_clip_search_bf16_4096x4096"] = {
            "us": wd.numel() * 4 / gbs / 1e3, "GBps": gbs,
            "cpu_baseline": {"value": cpu_s * 1e6, "unit": "us (scaled from the sample)", "kind": kind,
                             "cores": torch.get_num_threads(), "sample": f"{rows} of 4096 rows"}}

    def gptq_layer(n: int, tokens: int):
        lin = torch.nn.Linear(n, n, bias=False, device=device)
        lin.weight.data.copy_(w[:n, :n])
        acts = torch.randn(4, tokens // 4, n, generator=g) * (0.5 + 2 * torch.rand(n, generator=g))
        acts_d = acts.to(device)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        solver = gptq.GPTQ(lin)
        for i in range(4):
            solver.add_batch(acts_d[i : i + 1])
        q = solver.fasterquant(None, "mxint", {"weight_block_size": 32, "weight_width": 4}, quant_search=True)
        torch.cuda.synchronize()
        return time.perf_counter() - t0, acts, q

    gptq_layer(256, 512)  # warm-up: kernels, the solver library
    t_big = min(gptq_layer(4096, 8192)[0] for _ in range(2))  # host-driven (128 sweep steps): best of two
    t_small, acts, q = gptq_layer(1024, 2048)
    ws = w[:1024, :1024].clone()
    t0 = time.perf_counter()
    q_ref = O.gptq_quantize(ws, O.gptq_hessian([acts[i : i + 1] for i in range(4)]),
                            lambda W1: O.mxint_clip_search(W1, 32, 4, 1)[0], 32)
    t_cpu = time.perf_counter() - t0
    out["gptq_mxint4_search"] = {
        "layer_4096x4096_8192_tokens_ms": t_big * 1e3, "layer_1024x1024_2048_tokens_ms": t_small * 1e3,
        "weights_equal_to_cpu_port_1024": float((q.cpu() == q_ref).float().mean()),
        "cpu_baseline": {"value": t_cpu * 1e3, "unit": "ms", "kind": "port", "cores": torch.get_num_threads(),
                         "sample": "the 1024 x 1024 layer, 2048 tokens"}}
    return out


def attention_extras(device, peaks: dict) -> dict:
    """The quantized attention block (MXFP8 queries and probabilities, minifloat rotary tables and softmax input) at
    hidden 4096, 32 heads, 8 x 512 tokens, bf16, and its two batched products alone; the CPU restatement of the same
    block timed on one sequence."""
    from mase_b200 import attention, gemm
    from oracle import mx_oracle as O

    fp = {"data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    mini = {"data_in_exponent_width": 5, "data_in_frac_width": 10}
    qc = {"qk_matmul": fp, "av_matmul": fp, "rope": mini, "softmax": mini, "kv_cache": fp}
    B, S, H, D = 8, 512, 32, 128
    g = torch.Generator().manual_seed(5)
    block = attention.AttentionMXFP(None, 0, qc, hidden_size=H * D, num_heads=H, num_kv_heads=H, device=device,
                                    dtype=torch.bfloat16)
    for prm in block.parameters():
        prm.data.copy_((torch.randn(prm.shape, generator=g) * 0.02).to(device))
    hidden = torch.randn(B, S, H * D, generator=g).bfloat16()
    pos = torch.arange(S, dtype=torch.float32)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.cat([pos[:, None] * inv[None], pos[:, None] * inv[None]], dim=-1)
    cos, sin = ang.cos()[None].expand(B, S, D).bfloat16(), ang.sin()[None].expand(B, S, D).bfloat16()
    mask = torch.zeros(B, 1, S, S, dtype=torch.bfloat16).masked_fill(
        torch.ones(S, S, dtype=torch.bool).triu(1)[None, None], torch.finfo(torch.bfloat16).min)
    hd, cd, sd, md = hidden.to(device), cos.to(device), sin.to(device), mask.to(device)
    with torch.no_grad():
        t_block = 1.0 / quick_gbs(lambda: block(hd, (cd, sd), md), 1, calls=5) / 1e9
        q = torch.randn(B * H, S, D, device=device).bfloat16()
        k = torch.randn(B * H, S, D, device=device).bfloat16()
        p = torch.rand(B * H, S, S, device=device).bfloat16()
        vt = torch.randn(B * H, D, S, device=device).bfloat16()
        t_qk = 1.0 / quick_gbs(lambda: gemm.batched_product(q, k), 1, calls=10) / 1e9
        t_pv = 1.0 / quick_gbs(lambda: gemm.batched_product(p, vt), 1, calls=10) / 1e9
    flops = 2.0 * B * H * S * S * D
    # the same block with its projections swapped for MXINT8 layers (what the quantize pass does by name): every
    # kernel of the forward is then this package's
    import mase_b200 as mb

    int_cfg = {"weight_block_size": 32, "weight_width": 8, "data_in_block_size": 32, "data_in_width": 8}
    quant_block = attention.AttentionMXFP.from_attention(block, qc)
    for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
        lin = getattr(quant_block, name)
        q_lin = mb.LinearMXInt(lin.in_features, lin.out_features, bias=False, device=device, dtype=torch.bfloat16, config=int_cfg)
        q_lin.load_state_dict({"weight": lin.weight.data}, strict=False)
        setattr(quant_block, name, q_lin)
    with torch.no_grad():
        t_quant_block = 1.0 / quick_gbs(lambda: quant_block(hd, (cd, sd), md), 1, calls=5) / 1e9
    del quant_block
    w = {n: prm.detach().cpu() for n, prm in block.named_parameters()}
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    O.attention_mx(hidden[:1], w, cos[:1], sin[:1], mask[:1], "mxfp", qc, H, H, False)
    t_cpu = time.perf_counter() - t0
    hbm, hbm_kind = measured_peaks()
    # bytes each product has to move: both operands once, the result once (bf16)
    qk_bytes = 2.0 * B * H * (S * D + S * D + S * S)
    pv_bytes = 2.0 * B * H * (S * S + D * S + S * D)
    return {"block_ms": t_block * 1e3, "block_with_mxint8_projections_ms": t_quant_block * 1e3,
            "qk_batched_us": t_qk * 1e6, "pv_batched_us": t_pv * 1e6,
            "qk_TFLOPs": flops / t_qk / 1e12, "pv_TFLOPs": flops / t_pv / 1e12,
            "roofline": {"bound": "hbm", "unit": "GB/s", "peak": hbm, "peak_source": f"{hbm_kind} copy bandwidth",
                         "qk_achieved": qk_bytes / t_qk / 1e9, "qk_frac": qk_bytes / t_qk / 1e9 / hbm,
                         "pv_achieved": pv_bytes / t_pv / 1e9, "pv_frac": pv_bytes / t_pv / 1e9 / hbm,
                         "algorithmic_bytes": {"qk": qk_bytes, "pv": pv_bytes},
                         "timed": "256 products of 512 x 512 x 128 (Q K^T) and 512 x 128 x 512 (P V) per launch; 200 MB "
                                  "per launch, more than L2"},
            "cpu_baseline": {"value": t_cpu * B * 1e3, "unit": "ms (scaled from the sample)", "kind": "port",
                             "cores": torch.get_num_threads(), "sample": "1 of 8 sequences"}}


def decoder_layer_extras(device, peaks: dict, steps: int = 10) -> dict:
    """Llama-style decoder layer, hidden 4096, 32 heads, FFN 11008, batch 8 x sequence 512 (4096 tokens), bf16:
    q/k/v/o MXINT8 weights and activations (exact bf16 tensor-core GEMM of the quantized values), gate/up/down MXFP4
    weights x MXFP8 activations (block-scaled GEMM); norms, RoPE, attention and SiLU unquantized."""
    import mase_b200 as mb
    from mase_b200 import gemm, synthetic

    layer = synthetic.quantize_decoder_layer(
        synthetic.DecoderLayer().to(device),
        lambda k, n: mb.LinearMXInt(k, n, bias=False, device=device, dtype=torch.bfloat16,
                                    config=dict(synthetic.MXINT8_LINEAR)),
        lambda k, n: mb.LinearMXFP(k, n, bias=False, device=device, dtype=torch.bfloat16,
                                   config=dict(synthetic.MXFP4W_MXFP8A_LINEAR)))
    g = torch.Generator().manual_seed(3)
    tokens = 8 * 512
    x = torch.randn(8, 512, 4096, generator=g).bfloat16()
    xd = x.to(device)
    with torch.no_grad():
        t = 1.0 / quick_gbs(lambda: layer(xd), 1, calls=steps) / 1e9
    gemm.check_status(device)
    flops = layer.linear_flops(tokens)
    flops_int = 2.0 * tokens * 4 * layer.hidden * layer.hidden   # q/k/v/o on the bf16 kind
    flops_ffn = flops - flops_int                                 # gate/up/down at the FP8 rate
    t_ideal = flops_int / (peaks["bf16_tflops"] * 1e12) + flops_ffn / (peaks["fp8_used"] * 1e12)
    # CPU: the seven projections of the layer the way MASE runs them (quantize the input, F.linear in bf16) on a
    # sample of the tokens; norms, RoPE and attention are left out on both sides of this ratio
    qs, kind = cpu_quantizers()
    sample = 64
    xs = x.view(-1, 4096)[:sample]
    hs = torch.randn(sample, layer.ffn, generator=g).bfloat16()
    weights = {n: getattr(layer, n).weight.data.cpu() for n in synthetic.DecoderLayer.ATTENTION + synthetic.DecoderLayer.FFN}
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    for n in synthetic.DecoderLayer.ATTENTION:
        torch.nn.functional.linear(qs["mxint"](xs, 32, 8), weights[n])
    for n in ("gate_proj", "up_proj"):
        torch.nn.functional.linear(qs["mxfp"](xs, 32, 4, 3), weights[n])
    torch.nn.functional.linear(qs["mxfp"](hs, 32, 4, 3), weights["down_proj"])
    t_cpu = time.perf_counter() - t0
    return {"ms_per_forward": t * 1e3, "linear_TFLOPs": flops / t / 1e12, "tokens": tokens, "linear_flops": flops,
            "roofline": {"bound": "tensor", "achieved": flops / t / 1e12, "peak": flops / t_ideal / 1e12,
                         "unit": "TFLOP/s", "frac": t_ideal / t,
                         "peak_source": "Linear FLOPs at their rates: q/k/v/o at the measured bf16 peak, gate/up/down at "
                                        + peaks["fp8_used_source"] + "; attention, norms and RoPE count as overhead"},
            "cpu_baseline": {"value": layer.linear_flops(sample) / t_cpu / 1e12, "unit": "TFLOP/s",
                             "cores": torch.get_num_threads(), "kind": kind,
                             "sample": f"the 7 projections (quantize input + bf16 F.linear) on {sample} of {tokens} tokens"}}


def linear_extras(device, peaks: dict) -> dict:
    """MXFP8 Linear forward 4096 -> 4096 (bf16, no bias): activation quantization + block-scaled tcgen05 GEMM.
    Each M carries its roofline (HBM-bound up to M = 128, tensor-bound above) and the CPU forward timed beside it."""
    import mase_b200 as mb
    from mase_b200 import gemm, synthetic

    K = N = 4096
    cfg = {"weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    hbm, hbm_kind = measured_peaks()
    out = {}
    layer = None
    for M in (1, 16, 128, 2048, 8192):
        x, w = synthetic.linear_operands(M, K, N, seed=2)
        xh = x
        x = x.to(device)
        if layer is None:
            layer = mb.LinearMXFP(K, N, bias=False, device=device, dtype=torch.bfloat16, config=cfg)
            layer.load_state_dict({"weight": w.to(device)}, strict=False)
            wq_cpu = layer.weight.data.cpu()
            copies = [layer]
        flops = 2.0 * M * N * K
        calls = 20 if M >= 2048 else 50
        t_fwd = 1.0 / quick_gbs(lambda: layer(x), 1, calls=calls) / 1e9   # seconds per call
        xp = gemm.pack_mx_operand(x, 4, 3)
        wp = layer._packed_weight()
        t_gemm = 1.0 / quick_gbs(lambda: gemm.mx_gemm(xp, wp, None, torch.bfloat16, static_b=True), 1, calls=calls) / 1e9
        xq = mb.mxfp_quantizer(x, 32, 4, 3)
        t_dense = 1.0 / quick_gbs(lambda: gemm.linear_forward(xq, layer.weight, None), 1, calls=calls) / 1e9
        # the same forward replayed from a CUDA graph: device time without the per-call host work.  Small problems are
        # captured sixteen to a graph, each on its own copy of the layer (16 x 17 MB of packed weights > L2), so that the
        # replay's launch cost does not hide a kernel of a few microseconds and the weights stream from HBM every time.
        reps = 16 if M <= 128 else 1
        if reps > 1 and len(copies) == 1:
            copies.extend(copy.deepcopy(layer) for _ in range(reps - 1))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for r in range(reps):
                copies[r](x)
        t_graph = 1.0 / quick_gbs(graph.replay, 1, calls=calls) / 1e9 / reps
        del graph
        if reps > 1:
            wps = [c._packed_weight() for c in copies]
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for r in range(reps):
                    gemm.mx_gemm(xp, wps[r], None, torch.bfloat16, static_b=True)  # a layer's weight: packed at load
            t_gemm = min(t_gemm, 1.0 / quick_gbs(graph.replay, 1, calls=calls) / 1e9 / reps)
            del graph
        if M <= 128:
            algo = N * K * (1 + 1 / 32) + M * K * 2 + M * N * 2
            roof = {"bound": "hbm", "achieved": algo / t_graph / 1e9, "peak": hbm, "unit": "GB/s",
                    "frac": algo / t_graph / 1e9 / hbm, "gemm_only_frac": algo / t_gemm / 1e9 / hbm,
                    "peak_source": f"{hbm_kind} copy bandwidth", "algorithmic_bytes": algo,
                    "timed": "whole forward (activation pack + GEMM), sixteen layers with their own weights to a CUDA "
                             "graph: 280 MB of weights per replay, more than L2"}
        else:
            ach = flops / t_graph / 1e12
            roof = {"bound": "tensor", "achieved": ach, "peak": peaks["fp8_used"], "unit": "TFLOP/s",
                    "frac": ach / peaks["fp8_used"], "gemm_only_frac": flops / t_gemm / 1e12 / peaks["fp8_used"],
                    "peak_source": peaks["fp8_used_source"],
                    "frac_of_2x_measured_bf16": ach / (2 * peaks["bf16_tflops"]),
                    "frac_of_nominal_4500": ach / peaks["fp8_nominal_tflops"],
                    "timed": "whole forward (activation pack + GEMM) replayed from a CUDA graph"}
        sample = min(M, 256)
        t_cpu, kind = cpu_linear_time(xh[:sample], wq_cpu)
        out[f"M{M}"] = {"forward_us": t_fwd * 1e6, "forward_TFLOPs": flops / t_fwd / 1e12,
                        "forward_cuda_graph_us": t_graph * 1e6, "forward_cuda_graph_TFLOPs": flops / t_graph / 1e12,
                        "gemm_only_us": t_gemm * 1e6, "gemm_only_TFLOPs": flops / t_gemm / 1e12,
                        "bf16_gemm_of_fake_quant_us": t_dense * 1e6, "bf16_gemm_TFLOPs": flops / t_dense / 1e12,
                        "roofline": roof,
                        "cpu_baseline": {"value": 2.0 * sample * N * K / t_cpu / 1e12, "unit": "TFLOP/s",
                                         "cores": torch.get_num_threads(), "kind": kind,
                                         "sample": f"{sample} of {M} rows: MXFP8-quantize x, F.linear in bf16"}}
    gemm.check_status()
    return out


def oracle_quantize_weight(w: torch.Tensor, e: int, f: int, rows_per_chunk: int = 2048) -> torch.Tensor:
    """MXFP fake-quantization of a [N, K] weight along K with the CPU oracle, in row chunks (bounded host memory)."""
    from oracle import mx_oracle as O

    return torch.cat([O.mxfp_fake(w[r:r + rows_per_chunk], 32, e, f, 1) for r in range(0, w.shape[0], rows_per_chunk)])


def tp_stack_extras(device, rank: int, world: int, peaks: dict, reduce_mode: str = "fused", comm_sms: int = 16) -> dict:
    """Tensor-parallel Linear stack at the 70B shape: hidden 8192, FFN 28672, 4 gated-MLP layers, M = 8192 tokens,
    MXFP4 (E2M1) weights / MXFP8 (E4M3) activations, gate/up column parallel, down row parallel with an fp32
    reduction.  Strong scaling (total work fixed); every rank runs it.  Outside the timed region rank 0 recomputes a
    few output rows of the first layer on the CPU with the oracle (weights regenerated from the seed and quantized by
    the oracle) and reports the largest deviation, so the multi-GPU result is checked in the run that times it."""
    import torch.distributed as dist

    import mase_b200 as mb
    from mase_b200 import gemm, tp as tpmod

    hidden, ffn, layers, M = 8192, 28672, 4, 8192
    cfg = {"weight_block_size": 32, "weight_exponent_width": 2, "weight_frac_width": 1,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    tp = tpmod.TPGroup(rank, world, None)

    def build_stack(mode: str):
        gen = torch.Generator(device=device).manual_seed(4)
        stack = []
        for _ in range(layers):
            # every rank draws the same full weights (same seed) and keeps its shards
            ws = [(torch.randn(n, k, generator=gen, device=device) * 0.02).to(torch.bfloat16)
                  for (n, k) in ((ffn, hidden), (ffn, hidden), (hidden, ffn))]
            stack.append(tpmod.build_tp_gated_mlp(mb.LinearMXFP, ws[0], ws[1], ws[2], cfg, tp, device=device, reduce=mode))
            del ws
        return stack, torch.randn(M, hidden, generator=gen, device=device).to(torch.bfloat16)

    def time_stack(stack, x0):
        res = {}
        for micro in ((1,) if world == 1 else (1, 2)):
            def step():
                return tpmod.run_mlp_stack(stack, x0, micro_batches=micro, comm_sms=comm_sms)

            for _ in range(2):
                step()
            steps = 3
            res[micro] = time_region(step, steps, world, device) / steps
        gemm.check_status()
        return res

    stack, x0 = build_stack(reduce_mode)
    fallback_note = None
    by_mode = {}
    if reduce_mode == "fused" and world > 1:
        # the fused reduction needs symmetric memory and peer access between all ranks: try one step, and let every
        # rank fall back to the collective route together if any of them could not run it
        ok, why = 1, ""
        try:
            tpmod.run_mlp_stack(stack, x0)
            gemm.check_status()
        except Exception as exc:  # noqa: BLE001 - reported in the JSON line
            ok, why = 0, f"{type(exc).__name__}: {exc}"[:200]
        flag = torch.tensor([ok], device=device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            reduce_mode = "scatter_gather"
            fallback_note = "fused reduction unavailable on this run" + (f" ({why})" if why else "")
        else:
            by_mode["fused"] = time_stack(stack, x0)
        # The peer-store route and the collective route are both measured: small stores over NVLink favour the fused
        # route on few GPUs and the collective on many.  The faster one is the reported configuration.
        del stack
        torch.cuda.empty_cache()
        stack, x0 = build_stack("scatter_gather")
        by_mode["scatter_gather"] = time_stack(stack, x0)
        if "fused" in by_mode and min(by_mode["fused"].values()) <= min(by_mode["scatter_gather"].values()):
            del stack
            torch.cuda.empty_cache()
            reduce_mode = "fused"
            stack, x0 = build_stack("fused")
        else:
            reduce_mode = "scatter_gather"
        results = by_mode[reduce_mode]
    else:
        results = time_stack(stack, x0)
        by_mode[reduce_mode] = results
    micro, sec_step = min(results.items(), key=lambda kv: kv[1])
    flops = layers * 3 * 2.0 * M * hidden * ffn

    # ---- parity of layer 1 against the oracle (all ranks run the layer; rank 0 checks) ----
    y1 = stack[0](x0)
    gemm.check_status()
    parity = cpu = None
    weights_ok = None
    if rank == 0:
        from oracle import mx_oracle as O

        # Layer 1 on four rows, unsharded: activations quantized by the CPU oracle; the three full weights are
        # regenerated from the seed and fake-quantized on the device, with 64 rows of each checked bit for bit against
        # the oracle (quantizing all 700 M weight elements on the host would take minutes); the reference products run
        # in fp32 (torch.matmul as the checker, outside every timed region).
        rows = torch.tensor([0, 1171, 4097, M - 1])
        g1 = torch.Generator(device=device).manual_seed(4)
        wq = []
        weights_ok = True
        for (n, k) in ((ffn, hidden), (ffn, hidden), (hidden, ffn)):
            w = (torch.randn(n, k, generator=g1, device=device) * 0.02).to(torch.bfloat16)
            q = mb.mxfp_quantizer(w, 32, 2, 1, 1)
            idx = torch.arange(0, n, max(1, n // 64), device=device)
            weights_ok &= torch.equal(q[idx].cpu().view(torch.int16), O.mxfp_fake(w[idx].cpu(), 32, 2, 1, 1).view(torch.int16))
            wq.append(q)
            del w
        xs = x0[rows.to(device)].cpu()
        xq = O.mxfp_fake(xs, 32, 4, 3).to(device).float()
        gate = (xq @ wq[0].float().t()).bfloat16()
        up = (xq @ wq[1].float().t()).bfloat16()
        h = (torch.nn.functional.silu(gate) * up).cpu()
        ref = (O.mxfp_fake(h, 32, 4, 3).to(device).float() @ wq[2].float().t()).cpu()
        got = y1[rows.to(device)].float().cpu()
        parity = float((got - ref).abs().max() / ref.abs().max())
        # CPU baseline: one layer the way MASE's modules run it (quantize, F.linear in bf16) on a sample of the rows
        qs, kind = cpu_quantizers()
        sample = 64
        xc = x0[:sample].cpu()
        wc = [q.cpu() for q in wq]
        del wq
        torch.set_num_threads(os.cpu_count() or 1)
        t0 = time.perf_counter()
        xq16 = qs["mxfp"](xc, 32, 4, 3)
        hc = torch.nn.functional.silu(torch.nn.functional.linear(xq16, wc[0])) * torch.nn.functional.linear(xq16, wc[1])
        torch.nn.functional.linear(qs["mxfp"](hc, 32, 4, 3), wc[2])
        t_cpu = time.perf_counter() - t0
        cpu = {"value": 3 * 2.0 * sample * hidden * ffn / t_cpu / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
               "kind": kind, "sample": f"one layer (gate, up, SiLU*mul, down) on {sample} of {M} rows, unsharded"}
        del wc
    del stack, y1
    torch.cuda.empty_cache()
    ach = flops / sec_step / 1e12
    return {"config": "4 x (gate+up: 8192->2x28672 column; down: 28672->8192 row + fp32 reduction), M=8192, W E2M1 / A E4M3",
            "ms_per_step": sec_step * 1e3, "TFLOPs_aggregate": ach, "n_gpus": world,
            "scaling": "strong", "micro_batches": micro,
            "ms_per_step_by_micro_batches": {str(k): v * 1e3 for k, v in results.items()},
            "ms_per_step_by_reduction": {m: {str(k): v * 1e3 for k, v in r.items()} for m, r in by_mode.items()},
            "reduction": "fused: GEMM epilogue stores fp32 tiles into the owning GPU's memory (peer stores over NVLink), "
                         "bounded peer barrier, reduce + bf16 all-gather kernel over peer stores; no collective library "
                         "on the data path" if reduce_mode == "fused"
                         else "fp32 reduce-scatter + bf16 all-gather (NCCL) on a side stream",
            "reduction_note": fallback_note,
            "parity_max_rel_err": parity,
            "parity_check": "layer 1, rows 0/1171/4097/8191: activations quantized by the CPU oracle, weights quantized on "
                            "the device with 64 rows of each checked bit for bit against the oracle, fp32 reference "
                            "products, bf16 roundings of gate, up and SiLU*mul as torch does them",
            "parity_weight_rows_match_oracle": weights_ok,
            "roofline": {"bound": "tensor", "achieved": ach, "peak": world * peaks["fp8_used"], "unit": "TFLOP/s",
                         "frac": ach / (world * peaks["fp8_used"]),
                         "peak_source": f"{world} x " + peaks["fp8_used_source"]},
            "cpu_baseline": cpu}


def run_ours(args) -> None:
    import torch.distributed as dist

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MX kernels have no CPU fallback")
    device = torch.device(f"cuda:{local}")
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    import mase_b200 as mb
    from mase_b200 import synthetic

    global ROWS
    ROWS = args.rows
    x = synthetic.device_student_t3(ROWS, COLS, seed=1 + rank, device=device)
    n = x.numel()
    step_bytes = n * BYTES_PER_ELEM
    state = {}

    def step():
        state["y"] = mb.mxfp_quantizer(x, BLOCK, EXP_BITS, FRAC_BITS)

    sampler = ClockSampler(device)
    for _ in range(max(args.warmup, 3)):
        step()
    sampler.start()
    sec = time_region(step, args.steps, world, device)
    value = world * step_bytes * args.steps / sec / 1e9
    kernel_gbs = step_bytes * args.steps / sec / 1e9  # one kernel launch per step, on the timed stream

    if args.kernel_only:  # profiling aid: only the device-resident timed region
        if rank == 0:
            print(json.dumps({"metric": "mx_quant_dequant_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
                              "rows": ROWS, "steps": args.steps, "ms_per_step": sec / args.steps * 1e3}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end through the public API with host buffers -----------------------------------------
    chunks = 16
    rows_c = ROWS // chunks
    hx = torch.empty((ROWS, COLS), dtype=torch.bfloat16).pin_memory()
    hy = torch.empty((ROWS, COLS), dtype=torch.bfloat16).pin_memory()
    hx.copy_(x)
    n_streams = 2  # one chunk uploading while the other downloads (four streams measured slower: 87 vs 93 GB/s)
    streams = [torch.cuda.Stream(device=device) for _ in range(n_streams)]
    dbuf = [torch.empty((rows_c, COLS), dtype=torch.bfloat16, device=device) for _ in range(n_streams)]

    def e2e_step():
        cur = torch.cuda.current_stream()
        for s in streams:
            s.wait_stream(cur)
        for c in range(chunks):
            s = streams[c % n_streams]
            with torch.cuda.stream(s):
                dbuf[c % n_streams].copy_(hx[c * rows_c:(c + 1) * rows_c], non_blocking=True)
                yq = mb.mxfp_quantizer(dbuf[c % n_streams], BLOCK, EXP_BITS, FRAC_BITS)
                hy[c * rows_c:(c + 1) * rows_c].copy_(yq, non_blocking=True)
                yq.record_stream(s)
        for s in streams:
            cur.wait_stream(s)

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    e2e_sec = time_region(e2e_step, e2e_steps, world, device)
    e2e_value = world * step_bytes * e2e_steps / e2e_sec / 1e9
    ok = torch.equal(hy[:rows_c].view(torch.int16), state["y"][:rows_c].cpu().view(torch.int16))
    from oracle import mx_oracle as O  # checker only, outside every timed region

    probe = torch.arange(0, ROWS, max(1, ROWS // 16))[:16]
    ok_oracle = torch.equal(hy[probe].view(torch.int16), O.mxfp_fake(hx[probe], BLOCK, EXP_BITS, FRAC_BITS).view(torch.int16))
    clocks = sampler.stop()
    del hx, hy, dbuf
    tp_extra = None
    if not args.no_extra:
        state.clear()
        del x
        torch.cuda.empty_cache()
        peaks = tensor_peaks(device)
        tp_extra = tp_stack_extras(device, rank, world, peaks, args.tp_reduce, args.comm_sms)
        x = synthetic.device_student_t3(ROWS, COLS, seed=1 + rank, device=device)

    if rank == 0:
        peak, peak_kind = measured_peaks()
        roof = {"bound": "hbm", "achieved": kernel_gbs, "peak": peak, "unit": "GB/s", "frac": kernel_gbs / peak,
                "peak_source": f"{peak_kind} copy bandwidth", "kernel": "mxq::mxfp_kernel<bf16,bf16,fake,E4M3>",
                "algorithmic_bytes_per_launch": step_bytes,
                "traffic": None if NCU_DRAM_BYTES_PER_ELEM is None else NCU_DRAM_BYTES_PER_ELEM * n}
        cpu_sec, cores, cpu_kind = cpu_quantizer_time(CPU_SAMPLE_ROWS)
        cpu = {"value": CPU_SAMPLE_ROWS * COLS * BYTES_PER_ELEM / cpu_sec / 1e9, "unit": "GB/s", "cores": cores,
               "kind": cpu_kind, "sample": f"{CPU_SAMPLE_ROWS} of {ROWS} rows, one pass"}
        extra = extras(device, x, peaks) if not args.no_extra else {}
        if tp_extra is not None:
            extra["tp_linear_stack_70b_shape"] = tp_extra
        if extra:
            # the MX-Linear half of the metric, inside the objects of the bench contract
            lin = extra["linear_mxfp8_4096x4096"]
            roof["peaks"] = peaks
            roof["mx_linear"] = {m: v["roofline"] for m, v in lin.items()}
            roof["decoder_layer"] = extra["decoder_layer_mixed_precision"]["roofline"]
            roof["tp_linear_stack"] = dict(tp_extra["roofline"], ms_per_step=tp_extra["ms_per_step"],
                                           parity_max_rel_err=tp_extra["parity_max_rel_err"])
            cpu["mx_linear"] = {m: v["cpu_baseline"] for m, v in lin.items()}
            cpu["decoder_layer"] = extra["decoder_layer_mixed_precision"]["cpu_baseline"]
            cpu["tp_linear_stack"] = tp_extra["cpu_baseline"]
        print(json.dumps({
            "metric": "mx_quant_dequant_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": n * 2, "d2h_bytes_per_step": n * 2,
                    "steps": e2e_steps, "result_matches_device_path": bool(ok),
                    "result_rows_match_cpu_oracle": bool(ok_oracle)},
            "gpu_launches": args.steps, "roofline": roof, "cpu_baseline": cpu, "clocks": clocks, "extra": extra,
        }))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_linear(args) -> None:
    """`--workload linear`: MX Linear forward 4096 -> 4096 at M = --m (single GPU), one JSON line.  Used for the
    tensor-core roofline and for profiler captures of the GEMM and activation-pack kernels.  `--wfmt e2m1` stores
    the weight as nibble-packed MXFP4 (activations stay MXFP8)."""
    import mase_b200 as mb
    from mase_b200 import gemm, synthetic

    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    M, K, N = args.m, 4096, 4096
    we, wf = (2, 1) if args.wfmt == "e2m1" else (4, 3)
    cfg = {"weight_block_size": 32, "weight_exponent_width": we, "weight_frac_width": wf,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    x, w = synthetic.linear_operands(M, K, N, seed=2)
    x = x.to(device)
    layer = mb.LinearMXFP(K, N, bias=False, device=device, dtype=torch.bfloat16, config=cfg)
    layer.load_state_dict({"weight": w.to(device)}, strict=False)
    for _ in range(max(args.warmup, 3)):
        layer(x)
    sec = time_region(lambda: layer(x), args.steps, 1, device)
    xp = gemm.pack_mx_operand(x, 4, 3)
    wp = layer._packed_weight()
    sec_gemm = time_region(lambda: gemm.mx_gemm(xp, wp, None, torch.bfloat16), args.steps, 1, device)
    gemm.check_status()
    flops = 2.0 * M * N * K
    bf16_peak, _, src = measured_bf16_tflops()
    peak = 2.0 * bf16_peak
    ach = flops * args.steps / sec_gemm / 1e12
    print(json.dumps({
        "metric": "mx_linear_forward_TFLOPs", "value": flops * args.steps / sec / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": sec / args.steps * 1e3,
        "higher_is_better": True, "dtype": f"mxfp8 activations x {args.wfmt} weights, E8M0 scales, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"LinearMXFP 4096->4096 forward, M={M}, bf16 in/out, W {args.wfmt} / A e4m3, block 32"},
        "gpu_launches": 2 * args.steps,  # activation pack + GEMM
        "roofline": {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                     "peak_source": f"2 x {src} bf16 cuBLAS burst (the default run measures the library FP8 GEMM instead)",
                     "kernel": "mxq::gemm::umma_gemm_pair_kernel (cta_group::2, 256x256 tiles)" if M > 128
                     else "mxq::gemm::umma_gemm_swap_kernel (weight as the 128-row operand, K split over a cluster)",
                     "traffic": None},
        "gemm_only_ms": sec_gemm / args.steps * 1e3,
    }))


def run_decoder(args) -> None:
    """`--workload decoder`: the mixed-precision decoder layer alone (single GPU), one JSON line; for launch lists."""
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    peaks = {"bf16_tflops": measured_bf16_tflops()[0]}
    peaks["fp8_used"], peaks["fp8_used_source"] = 2.0 * peaks["bf16_tflops"], "2 x measured bf16 (no FP8 GEMM measured in this mode)"
    out = decoder_layer_extras(device, peaks, steps=args.steps)
    print(json.dumps({"metric": "decoder_layer_linear_TFLOPs", "value": out["linear_TFLOPs"], "unit": "TFLOP/s", "n_gpus": 1,
                      "steps": args.steps, "ms_per_step": out["ms_per_forward"], "higher_is_better": True,
                      "config": {"workload": "Llama-style decoder layer, hidden 4096, FFN 11008, 8 x 512 tokens, MXINT8 "
                                             "attention projections, MXFP4-weight / MXFP8-activation FFN"},
                      "roofline": out["roofline"], "cpu_baseline": out["cpu_baseline"]}))


def run_search(args) -> None:
    """`--workload search`: the clipping search of both formats on a bf16 [4096, 4096] weight (single GPU), one JSON
    line; for profiler captures of the search kernels."""
    import mase_b200 as mb

    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    g = torch.Generator().manual_seed(3)
    w = torch.randn(4096, 4096, generator=g) * 0.02
    w[torch.rand(4096, 4096, generator=g) < 0.01] *= 20
    wd = w.to(device).bfloat16()
    int_meta, fp_meta = mb.MXIntMeta(32, 8, 4), mb.MXFPMeta(32, 8, 2, 1, True, "rn")

    def step():
        mb.mxint_quantizer_sim(wd, 1, int_meta, quantile_search=True)
        mb.mxfp_quantizer_sim(wd, 1, fp_meta, quantile_search=True)

    for _ in range(max(args.warmup, 1)):
        step()
    sec = time_region(step, args.steps, 1, device)
    print(json.dumps({"metric": "clip_search_pair_ms", "value": sec / args.steps * 1e3, "unit": "ms", "n_gpus": 1,
                      "steps": args.steps, "higher_is_better": False,
                      "config": {"workload": "MXINT4 + MXFP4 (E2M1) clipping search of a bf16 [4096, 4096] weight, block 32"}}))


def run_attention(args) -> None:
    """`--workload attention`: the quantized attention block alone (single GPU), one JSON line; for launch lists and
    profiler captures of the batched products, the rotary and the softmax kernels."""
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    out = attention_extras(device, {"bf16_tflops": measured_bf16_tflops()[0]})
    print(json.dumps({"metric": "attention_block_ms", "value": out["block_ms"], "unit": "ms", "n_gpus": 1,
                      "steps": args.steps, "higher_is_better": False,
                      "config": {"workload": "MXFP8 attention block, hidden 4096, 32 heads of 128, 8 x 512 tokens, bf16"},
                      "roofline": out["roofline"], "cpu_baseline": out["cpu_baseline"], "extra": out}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the untimed extra measurements")
    ap.add_argument("--rows", type=int, default=ROWS, help="rows of the [rows, 8192] tensor (default: the full workload)")
    ap.add_argument("--kernel-only", action="store_true", help="only the device-resident timed region (for profilers)")
    ap.add_argument("--workload", default="quant", choices=["quant", "linear", "decoder", "search", "attention"],
                    help="quant: the headline quantizer benchmark; linear: MX Linear forward; decoder: the mixed-precision "
                         "decoder layer (both profiling aids)")
    ap.add_argument("--m", type=int, default=8192, help="tokens for --workload linear")
    ap.add_argument("--tp-reduce", default="fused", choices=["fused", "scatter_gather", "all_reduce"],
                    help="reduction of the row-parallel layers of the tensor-parallel extra; with 'fused' the collective "
                         "route is timed as well and the faster one is reported")
    ap.add_argument("--comm-sms", type=int, default=16,
                    help="SMs the GEMMs leave to the reduction's kernels when micro-batches overlap (tensor-parallel extra)")
    ap.add_argument("--wfmt", default="e4m3", choices=["e4m3", "e2m1"], help="weight format for --workload linear")
    args = ap.parse_args()
    if args.workload == "linear" and args.impl == "ours":
        run_linear(args)
        return
    if args.workload == "search" and args.impl == "ours":
        return run_search(args)
    if args.workload == "attention" and args.impl == "ours":
        return run_attention(args)
    if args.workload == "decoder" and args.impl == "ours":
        run_decoder(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
