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
  cpu_baseline  the CPU port of MASE's algorithm (oracle/) on a bounded sample of the same tensor, rank 0 only
  extra   other formats / shapes of the sweep and the MX Linear forward, measured outside the timed region

`--impl reference` times the CPU port on the host cores instead (bounded sample per step).
"""

from __future__ import annotations

import argparse
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


def cpu_port_time(rows: int, repeats: int = 1) -> tuple[float, int]:
    """Seconds for the CPU port to fake-quantize `rows` rows of the workload; uses every host thread."""
    from mase_b200 import synthetic
    from oracle import mx_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = synthetic.student_t3(rows, COLS, seed=1)
    O.mxfp_fake(x[:64], BLOCK, EXP_BITS, FRAC_BITS)  # warm-up
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.mxfp_fake(x, BLOCK, EXP_BITS, FRAC_BITS)
        best = min(best, time.perf_counter() - t0)
    return best, torch.get_num_threads()


def run_reference(args) -> None:
    """The CPU implementation of the path on the host cores; rank 0 only."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from mase_b200 import synthetic
    from oracle import mx_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = synthetic.student_t3(CPU_SAMPLE_ROWS, COLS, seed=1)
    for _ in range(args.warmup):
        O.mxfp_fake(x[:256], BLOCK, EXP_BITS, FRAC_BITS)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.mxfp_fake(x, BLOCK, EXP_BITS, FRAC_BITS)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = CPU_SAMPLE_ROWS * COLS * BYTES_PER_ELEM / dt / 1e9
    sample = f"{CPU_SAMPLE_ROWS} of {ROWS} rows per step"
    print(json.dumps({
        "impl": "reference", "metric": "mx_quant_dequant_GBps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
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


def extras(device, x) -> dict:
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
    out["linear_mxfp8_4096x4096"] = linear_extras(device)
    out["decoder_layer_mixed_precision"] = decoder_layer_extras(device)
    return out


def decoder_layer_extras(device) -> dict:
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
    x = torch.randn(8, 512, 4096, generator=g).bfloat16().to(device)
    with torch.no_grad():
        t = 1.0 / quick_gbs(lambda: layer(x), 1, calls=10) / 1e9
    gemm.check_status(device)
    flops = layer.linear_flops(8 * 512)
    return {"ms_per_forward": t * 1e3, "linear_TFLOPs": flops / t / 1e12, "tokens": 8 * 512,
            "linear_flops": flops}


def linear_extras(device) -> dict:
    """MXFP8 Linear forward 4096 -> 4096 (bf16, no bias): activation quantization + block-scaled tcgen05 GEMM."""
    import mase_b200 as mb
    from mase_b200 import gemm, synthetic

    K = N = 4096
    cfg = {"weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    out = {}
    layer = None
    for M in (1, 16, 128, 2048, 8192):
        x, w = synthetic.linear_operands(M, K, N, seed=2)
        x = x.to(device)
        if layer is None:
            layer = mb.LinearMXFP(K, N, bias=False, device=device, dtype=torch.bfloat16, config=cfg)
            layer.load_state_dict({"weight": w.to(device)}, strict=False)
        flops = 2.0 * M * N * K
        calls = 20 if M >= 2048 else 50
        t_fwd = 1.0 / quick_gbs(lambda: layer(x), 1, calls=calls) / 1e9   # seconds per call
        xp = gemm.pack_mx_operand(x, 4, 3)
        wp = layer._packed_weight()
        t_gemm = 1.0 / quick_gbs(lambda: gemm.mx_gemm(xp, wp, None, torch.bfloat16), 1, calls=calls) / 1e9
        xq = mb.mxfp_quantizer(x, 32, 4, 3)
        t_dense = 1.0 / quick_gbs(lambda: gemm.linear_forward(xq, layer.weight, None), 1, calls=calls) / 1e9
        # the same forward replayed from a CUDA graph: device time without the per-call host work
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            layer(x)
        t_graph = 1.0 / quick_gbs(graph.replay, 1, calls=calls) / 1e9
        del graph
        out[f"M{M}"] = {"forward_us": t_fwd * 1e6, "forward_TFLOPs": flops / t_fwd / 1e12,
                        "forward_cuda_graph_us": t_graph * 1e6, "forward_cuda_graph_TFLOPs": flops / t_graph / 1e12,
                        "gemm_only_us": t_gemm * 1e6, "gemm_only_TFLOPs": flops / t_gemm / 1e12,
                        "bf16_gemm_of_fake_quant_us": t_dense * 1e6, "bf16_gemm_TFLOPs": flops / t_dense / 1e12}
    gemm.check_status()
    return out


def tp_stack_extras(device, rank: int, world: int) -> dict:
    """Tensor-parallel Linear stack at the 70B shape: hidden 8192, FFN 28672, 4 gated-MLP layers, M = 8192 tokens,
    MXFP4 (E2M1) weights / MXFP8 (E4M3) activations, gate/up column parallel, down row parallel with an fp32
    all-reduce.  Strong scaling (total work fixed); every rank runs it."""
    import torch.distributed as dist

    import mase_b200 as mb
    from mase_b200 import gemm, tp as tpmod

    hidden, ffn, layers, M = 8192, 28672, 4, 8192
    cfg = {"weight_block_size": 32, "weight_exponent_width": 2, "weight_frac_width": 1,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    tp = tpmod.TPGroup(rank, world, None)
    gen = torch.Generator(device=device).manual_seed(4)
    stack = []
    for _ in range(layers):
        mods = []
        for (n, k, mode) in ((ffn, hidden, "column"), (ffn, hidden, "column"), (hidden, ffn, "row")):
            # every rank draws the same full weight (same seed) and keeps its shard
            w = (torch.randn(n, k, generator=gen, device=device) * 0.02).to(torch.bfloat16)
            kw = {"reduce": "scatter_gather"} if mode == "row" else {}
            mods.append(tpmod.build_tp_linear(mb.LinearMXFP, w, None, cfg, mode, tp, device=device, **kw))
            del w
        stack.append(tpmod.TPGatedMLP(*mods))
    x0 = torch.randn(M, hidden, generator=gen, device=device).to(torch.bfloat16)

    results = {}
    for micro in ((1,) if world == 1 else (1, 2)):
        def step():
            return tpmod.run_mlp_stack(stack, x0, micro_batches=micro)

        for _ in range(2):
            step()
        steps = 3
        results[micro] = time_region(step, steps, world, device) / steps
    gemm.check_status()
    micro, sec_step = min(results.items(), key=lambda kv: kv[1])
    flops = layers * 3 * 2.0 * M * hidden * ffn
    del stack
    torch.cuda.empty_cache()
    return {"config": "4 x (gate, up: 8192->28672 column; down: 28672->8192 row + all-reduce), M=8192, W E2M1 / A E4M3",
            "ms_per_step": sec_step * 1e3, "TFLOPs_aggregate": flops / sec_step / 1e12, "n_gpus": world,
            "scaling": "strong", "micro_batches": micro,
            "ms_per_step_by_micro_batches": {str(k): v * 1e3 for k, v in results.items()},
            "reduction": "fp32 reduce-scatter + bf16 all-gather on a side stream"}


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
    clocks = sampler.stop()
    del hx, hy, dbuf
    tp_extra = None
    if not args.no_extra:
        state.clear()
        del x
        torch.cuda.empty_cache()
        tp_extra = tp_stack_extras(device, rank, world)
        x = synthetic.device_student_t3(ROWS, COLS, seed=1 + rank, device=device)

    if rank == 0:
        peak, peak_kind = measured_peaks()
        roof = {"bound": "hbm", "achieved": kernel_gbs, "peak": peak, "unit": "GB/s", "frac": kernel_gbs / peak,
                "peak_source": f"{peak_kind} copy bandwidth", "kernel": "mxq::mxfp_kernel<bf16,bf16,fake,E4M3>",
                "algorithmic_bytes_per_launch": step_bytes,
                "traffic": None if NCU_DRAM_BYTES_PER_ELEM is None else NCU_DRAM_BYTES_PER_ELEM * n}
        cpu_sec, cores = cpu_port_time(CPU_SAMPLE_ROWS)
        cpu = {"value": CPU_SAMPLE_ROWS * COLS * BYTES_PER_ELEM / cpu_sec / 1e9, "unit": "GB/s", "cores": cores,
               "kind": "port", "sample": f"{CPU_SAMPLE_ROWS} of {ROWS} rows, one pass"}
        extra = extras(device, x) if not args.no_extra else {}
        if tp_extra is not None:
            extra["tp_linear_stack_70b_shape"] = tp_extra
        print(json.dumps({
            "metric": "mx_quant_dequant_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": n * 2, "d2h_bytes_per_step": n * 2,
                    "steps": e2e_steps, "result_matches_device_path": bool(ok)},
            "gpu_launches": args.steps, "roofline": roof, "cpu_baseline": cpu, "clocks": clocks, "extra": extra,
        }))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_linear(args) -> None:
    """`--workload linear`: MXFP8 Linear forward 4096 -> 4096 at M = --m (single GPU), one JSON line.  Used for the
    tensor-core roofline and for profiler captures of the GEMM and activation-pack kernels."""
    import mase_b200 as mb
    from mase_b200 import gemm, synthetic

    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    M, K, N = args.m, 4096, 4096
    cfg = {"weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3,
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
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            bf16_peak, src = float(json.load(fh)["bf16_tflops"]), "2 x measured bf16 cuBLAS burst"
    except Exception:
        bf16_peak, src = 1590.0, "2 x fallback bf16"
    peak = 2.0 * bf16_peak
    ach = flops * args.steps / sec_gemm / 1e12
    print(json.dumps({
        "metric": "mx_linear_forward_TFLOPs", "value": flops * args.steps / sec / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": sec / args.steps * 1e3,
        "higher_is_better": True, "dtype": "mxfp8 (E4M3 x E4M3, E8M0 scales), fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"LinearMXFP 4096->4096 forward, M={M}, bf16 in/out, W and A MXFP8 block 32"},
        "gpu_launches": 2 * args.steps,  # activation pack + GEMM
        "roofline": {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                     "peak_source": src + " (no block-scaled FP8 entry in MEASURED_PEAKS.json; nominal 4500)",
                     "kernel": "mxq::gemm::umma_gemm_pair_kernel (cta_group::2, 256x256 tiles)" if M >= 1024
                     else "mxq::gemm::umma_gemm_kernel<mxf8,64>", "traffic": None},
        "gemm_only_ms": sec_gemm / args.steps * 1e3,
    }))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the untimed extra measurements")
    ap.add_argument("--rows", type=int, default=ROWS, help="rows of the [rows, 8192] tensor (default: the full workload)")
    ap.add_argument("--kernel-only", action="store_true", help="only the device-resident timed region (for profilers)")
    ap.add_argument("--workload", default="quant", choices=["quant", "linear"],
                    help="quant: the headline quantizer benchmark; linear: MXFP8 Linear forward (profiling aid)")
    ap.add_argument("--m", type=int, default=8192, help="tokens for --workload linear")
    args = ap.parse_args()
    if args.workload == "linear" and args.impl == "ours":
        run_linear(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
