#!/usr/bin/env python
"""Benchmark of the biased, key-masked attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2]

One "step" is one attention call over one batch of seeded synthetic input.  At N = 1 the
workload is grid / triangle self-attention over pair rows at N = 768 (q, k, v bf16
[768, 4, 768, 32], fp32 bias [4, 768, 768], row-wise key mask); for N > 1 every rank owns a
block of 768 more pair rows of the same problem (rows are independent, so there is no
data-path collective; bias and mask are broadcast once, untimed) and the line reports
``"scaling": "weak"``.  Rank 0 prints ONE JSON line.

``--impl reference`` times the CPU restatement of the reference operator (oracle/, all host
threads) on a bounded row sample of the same workload; the reference's own libxsmm build is not
available on this machine.
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
sys.path.insert(0, ROOT)

METRIC = "biased_attention_tflops"
UNIT = "TFLOP/s"
NOMINAL_BF16_TFLOPS = 2250.0


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16_tflops": p["bf16_tflops"], "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, b in names.items():
                    if bits & b:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# --------------------------------------------------------------------------- CPU arm
def time_cpu_port(inp, shape, target_s: float, max_rows: int):
    """Times the C restatement on a row sample sized for about ``target_s`` seconds."""
    from oracle import attention_oracle as O
    B1, B2, S, D = shape

    def run(rows):
        t0 = time.time()
        O.ref_semantics(inp["q"][:rows], inp["k"][:rows], inp["v"][:rows], inp["mask"][:rows],
                        inp["bias"])
        return time.time() - t0

    probe_rows = min(2, max_rows)
    run(probe_rows)                       # warm: builds / loads the library, touches memory
    t = run(probe_rows)
    rows = int(max(probe_rows, min(max_rows, target_s / max(t, 1e-4) * probe_rows)))
    secs = run(rows)
    flops = O.attention_flops(rows, B2, S, S, D)
    return {"value": flops / secs / 1e12, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
            "sample": f"{rows} of {B1} pair rows, one call, {secs:.2f} s", "rows": rows, "secs": secs}


def reference_arm(args, world, rank):
    if rank != 0:
        return
    from oracle import attention_oracle as O
    name = args.workload
    c = O.CONFIGS[name]
    shape = (c["B1"], c["B2"], c["S"], c["D"])
    sample_rows = min(c["B1"], 16)
    inp = O.make_inputs(name, rows=sample_rows)
    if c.get("fp8"):   # the reference has no fp8 path: time its bf16 operator on de-quantised inputs
        inp["q"] = (inp["q"].float() * inp["q_scale"].view(1, -1, 1, 1)).to(torch.bfloat16)
        inp["k"] = (inp["k"].float() * inp["k_scale"].view(1, -1, 1, 1)).to(torch.bfloat16)
    # size one step for roughly (120 s / steps) of CPU work
    budget = max(1.0, min(10.0, 120.0 / max(1, args.steps + args.warmup)))
    first = time_cpu_port(inp, shape, budget, sample_rows)
    rows = first["rows"]
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.time()
        O.ref_semantics(inp["q"][:rows], inp["k"][:rows], inp["v"][:rows], inp["mask"][:rows], inp["bias"])
        if i >= args.warmup:
            times.append(time.time() - t0)
    ms = 1e3 * sum(times) / len(times)
    flops = O.attention_flops(rows, c["B2"], c["S"], c["S"], c["D"])
    value = flops / (ms / 1e3) / 1e12
    sample = f"{rows} of {c['B1']} pair rows per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(name, c, world, sample_rows=rows),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the reference operator (oracle/ref_semantics.c, pthreads); "
                "the reference's libxsmm build is unavailable on this machine",
    }
    print(json.dumps(line), flush=True)


def workload_config(name, c, world, sample_rows=None):
    cfg = {
        "workload": f"{name}: biased key-masked attention, q/k/v [{c['B1']},{c['B2']},{c['S']},{c['D']}]"
                    f" {'fp8-e4m3 q/k' if c.get('fp8') else 'bf16'}, bias {str(c['bias_dtype']).split('.')[-1]}"
                    f" [{c['B2']},{c['S']},{c['S']}], mask {c['mask']}",
        "rows_per_gpu": c["B1"], "heads": c["B2"], "seq_len": c["S"], "head_dim": c["D"],
        "parallelism": f"rows{world}" if world > 1 else "single",
        "cache": "inputs larger than L2 (no flush)" if name in ("cfg2", "cfg5") else "L2 flushed between steps",
    }
    if sample_rows is not None:
        cfg["cpu_sample_rows"] = sample_rows
    return cfg


# --------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2",
                    choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "grid_block", "pair_bias"])
    ap.add_argument("--rows", type=int, default=0, help="override pair rows per GPU (debugging)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only warm-up + timed steps with a bf16 bias (for ncu captures): no e2e, no CPU leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, world, rank)
        return

    import torch.distributed as dist
    from af3_kernels_b200 import _capi, dot_product_attention_cpp
    from af3_kernels_b200.dpa import dot_product_attention, dot_product_attention_host, read_status
    from oracle import attention_oracle as O   # input generators, flop model and the CPU baseline leg only

    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl ours needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    name = args.workload
    if name in ("grid_block", "pair_bias"):
        if rank == 0:
            (grid_block_line if name == "grid_block" else pair_bias_line)(args, dev)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    c = dict(O.CONFIGS[name])
    if args.rows:
        c["B1"] = args.rows
    B1, B2, S, D = c["B1"], c["B2"], c["S"], c["D"]
    fp8 = bool(c.get("fp8"))

    # ---- inputs: every rank owns B1 pair rows; bias (and the mask pattern) come from rank 0
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    qf = torch.randn(B1, B2, S, D, generator=g, device=dev)
    kf = torch.randn(B1, B2, S, D, generator=g, device=dev)
    v = torch.randn(B1, B2, S, D, generator=g, device=dev).to(torch.bfloat16)
    if fp8:
        q, q_scale = O.quantize_e4m3_per_head(qf)
        k, k_scale = O.quantize_e4m3_per_head(kf)
    else:
        q, k, q_scale, k_scale = qf.to(torch.bfloat16), kf.to(torch.bfloat16), None, None
    del qf, kf
    gb = torch.Generator(device=dev).manual_seed(0)
    bias = (torch.randn(B2, S, S, generator=gb, device=dev) * c["bias_std"]).to(c["bias_dtype"])
    if c["mask"].startswith("tail"):
        mask = torch.ones(B1, S, dtype=torch.bool, device=dev)
        mask[:, S - int(c["mask"][4:]):] = False
    else:
        mask = torch.rand(B1, S, generator=g, device=dev) >= 0.05
    if world > 1:
        dist.broadcast(bias, src=0)
        if fp8:
            dist.broadcast(q_scale, src=0)
            dist.broadcast(k_scale, src=0)
    kw = dict(q_scale=q_scale, k_scale=k_scale) if fp8 else {}

    flush = None
    if name not in ("cfg2", "cfg5"):   # small workloads fit in L2: flush it between steps
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def step():
        if flush is not None:
            flush.zero_()
        return dot_product_attention_cpp(q, k, v, mask, bias, **kw)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    lib = _capi.load()
    if args.kernel_only:
        bias = bias.to(torch.bfloat16)
    for _ in range(args.warmup):
        step()
    launches_per_step = lib.af3k_last_launch_count()
    sync_all()
    sampler = ClockSampler(local_rank)
    sampler.start()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(args.steps)]
    for e0, e1 in evs:
        if flush is not None:
            flush.zero_()
        e0.record()
        dot_product_attention_cpp(q, k, v, mask, bias, **kw)
        e1.record()
    sync_all()
    clocks = sampler.stop()
    step_ms = [e0.elapsed_time(e1) for e0, e1 in evs]
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    ms_per_step = total_ms.item() / args.steps
    status = read_status(dev)

    flops_rank = O.attention_flops(B1, B2, S, S, D)
    value = world * flops_rank / (ms_per_step / 1e3) / 1e12

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
                              "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
                              "kernel_only": True, "config": workload_config(name, c, world),
                              "device_status": status}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- end to end through the reference-facing operator with HOST buffers (every rank)
    host = {n: t.cpu().pin_memory() for n, t in (("q", q), ("k", k), ("v", v), ("bias", bias), ("mask", mask))}
    out_host = torch.empty((B1, B2, S, D), dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = out_host.numel() * out_host.element_size()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        # the operator's host-tensor path: row blocks pipelined over three streams (H2D, kernel, D2H)
        dot_product_attention_host(host["q"], host["k"], host["v"], host["mask"], host["bias"], out=out_host,
                                   device=dev, **kw)

    e2e_step()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    sync_all()
    e2e_total = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_total, op=dist.ReduceOp.MAX)
    e2e_ms = e2e_total.item() / e2e_steps
    e2e = {"value": world * flops_rank / (e2e_ms / 1e3) / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
           "steps": e2e_steps}

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel: the attention kernel alone (bias already bf16, so the
    # staging pre-pass does not run), CUDA events around each launch on the launching stream
    peaks = load_peaks()
    bias16 = bias.to(torch.bfloat16)
    for _ in range(3):
        dot_product_attention(q, k, v, mask, bias16, **kw)
    torch.cuda.synchronize()
    kevs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            for _ in range(min(args.steps, 50))]
    for e0, e1 in kevs:
        if flush is not None:
            flush.zero_()
        e0.record()
        dot_product_attention(q, k, v, mask, bias16, **kw)
        e1.record()
    torch.cuda.synchronize()
    kernel_ms = sum(e0.elapsed_time(e1) for e0, e1 in kevs) / len(kevs)
    achieved = flops_rank / (kernel_ms / 1e3) / 1e12
    alg_bytes = O.attention_bytes(B1, B2, S, S, D, qk_bytes=1 if fp8 else 2, bias_bytes=2)
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
        "frac": achieved / peaks["bf16_tflops"], "peak_source": peaks["source"] + " (bf16 burst)",
        "kernel": "attention_kernel", "kernel_ms": kernel_ms,
        "flops_per_launch": flops_rank, "algorithmic_bytes_per_launch": alg_bytes,
        "frac_of_nominal_2250": achieved / NOMINAL_BF16_TFLOPS,
        "hbm_gbs_achieved": alg_bytes / (kernel_ms / 1e3) / 1e9,
        "traffic": TRAFFIC_BYTES.get(name),
    }

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:
        cpu_in = {n: host[n] for n in ("q", "k", "v", "bias", "mask")}
        if fp8:
            cpu_in["q"] = (host["q"].float() * q_scale.cpu().view(1, -1, 1, 1)).to(torch.bfloat16)
            cpu_in["k"] = (host["k"].float() * k_scale.cpu().view(1, -1, 1, 1)).to(torch.bfloat16)
        cb = time_cpu_port(cpu_in, (B1, B2, S, D), target_s=12.0, max_rows=B1)
        cpu_baseline = {kk: cb[kk] for kk in ("value", "unit", "cores", "kind", "sample")}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8+bf16" if fp8 else "bf16",
        "data": "synthetic (seeded normal q/k/v/bias, Bernoulli or tail key mask)",
        "config": workload_config(name, c, world),
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        "device_status": status,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def grid_block_line(args, dev):
    """Extra workload (not the headline line): the whole grid self-attention module at N = 768,
    c_pair = 128, 4 heads - LayerNorm, bias and q/k/v/gate projections (cuBLAS), the attention
    kernel, gating and output projection - on a device-resident pair representation."""
    import af3_kernels_b200 as A
    N, C, H = (args.rows or 768), 128, 4
    torch.manual_seed(0)
    m = A.GridSelfAttentionCpp(C, H).to(dev).to(torch.bfloat16).eval()
    pair = torch.randn(N, N, C, device=dev, dtype=torch.bfloat16)
    mask = torch.rand(N, N, device=dev) >= 0.05
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            m(pair, mask)
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(args.steps)]
        for e0, e1 in evs:
            e0.record()
            m(pair, mask)
            e1.record()
        torch.cuda.synchronize()
    ms = sum(e0.elapsed_time(e1) for e0, e1 in evs) / len(evs)
    attn_flops = 4.0 * N * H * N * N * (C // H)
    gemm_flops = 2.0 * N * N * C * (5 * C + H)
    print(json.dumps({"metric": "grid_block_tflops", "value": (attn_flops + gemm_flops) / (ms / 1e3) / 1e12,
                      "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
                      "ms_per_step": ms, "attention_flops": attn_flops, "projection_flops": gemm_flops,
                      "config": {"workload": f"GridSelfAttentionCpp forward, pair [{N},{N},{C}] bf16, {H} heads"},
                      "dtype": "bf16", "data": "synthetic"}), flush=True)


def pair_bias_line(args, dev):
    """Extra workload (not the headline line): the fused pair-bias producer (LayerNorm + bias
    projection + permute) on a device-resident pair [N, N, 128] bf16, N = 768, 4 heads.  HBM-bound:
    algorithmic bytes = pair read + normalised pair written (2 bytes per element each) + bias."""
    import ctypes
    from af3_kernels_b200 import _capi
    N, C, H = (args.rows or 768), 128, 4
    g = torch.Generator(device=dev).manual_seed(0)
    pair = torch.randn(N, N, C, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    ln_w = torch.ones(C, device=dev)
    ln_b = torch.zeros(C, device=dev)
    w = torch.randn(H, C, generator=g, device=dev) * 0.1
    pitch = (N + 7) // 8 * 8
    # three sets of buffers in rotation so that a launch does not find its input in L2; the C entry
    # point is called directly (the Python wrapper's allocations would be timed otherwise)
    sets = [(pair.clone(), torch.empty_like(pair), torch.empty((H, N, pitch), dtype=torch.bfloat16, device=dev))
            for _ in range(3)]
    lib = _capi.load()
    stream = torch.cuda.current_stream().cuda_stream

    def launch(i):
        src, normed, bias = sets[i % 3]
        _capi.check(lib.af3k_pair_bias(src.data_ptr(), _capi.AF3K_BF16, N, N, C, H, ln_w.data_ptr(),
                                       ln_b.data_ptr(), w.data_ptr(), ctypes.c_float(1e-5),
                                       normed.data_ptr(), bias.data_ptr(), pitch, stream))

    for i in range(max(args.warmup, 3)):
        launch(i)
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for i, (e0, e1) in enumerate(evs):
        e0.record()
        launch(i)
        e1.record()
    torch.cuda.synchronize()
    ms = sum(e0.elapsed_time(e1) for e0, e1 in evs) / len(evs)
    alg_bytes = 2.0 * N * N * C * 2 + 2.0 * H * N * ((N + 7) // 8 * 8)
    peaks = load_peaks()
    gbs = alg_bytes / (ms / 1e3) / 1e9
    print(json.dumps({"metric": "pair_bias_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "ms_per_step": ms,
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                   "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
                                   "kernel": "pair_bias_kernel_t", "algorithmic_bytes_per_launch": alg_bytes,
                                   "traffic": None},
                      "config": {"workload": f"pair-bias producer, pair [{N},{N},{C}] bf16 -> normed bf16 + bias [{H},{N},{N}] bf16",
                                 "cache": "three buffer sets in rotation (920 MB > L2)"},
                      "dtype": "f32", "data": "synthetic"}), flush=True)


# DRAM bytes per launch of attention_kernel from one ncu capture (dram__bytes_read.sum +
# dram__bytes_write.sum), scaled to the full launch by pair rows; see profiles/.
TRAFFIC_BYTES = {"cfg2": 552.8e6}   # 4 x (118.18 + 20.01) MB captured on 192 of 768 pair rows

if __name__ == "__main__":
    main()
