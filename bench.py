#!/usr/bin/env python
"""Benchmark of the hot path: one dense contraction per step on each GPU.

Default workload (N=1): the 8192^3 bf16 GEMM with fp32 accumulation, the configuration
the headline TFLOP/s figure is quoted on. With N>1 ranks (launched by torchrun, one rank per
GPU) every rank multiplies the shared A by its own 8192-column slab of B: the N-column
sharding of the GEMM with the per-GPU work held fixed (weak scaling); no collective is on
the data path, NCCL is used only for the barrier and the max-over-ranks time.

`value`   : operands already resident in HBM, kernels timed with CUDA events on the launching stream.
`e2e`     : the same contraction through the C-ABI entry with pinned HOST buffers, so every step
            pays the host->device copy of A and B and the device->host copy of C.
`--impl reference` times the CPU restatement of the reference specification (oracle/) on the
host cores instead; it is the only arm that touches oracle/ besides the cpu_baseline sample.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, dims)
    "gemm_bf16_8192": ("gemm", dict(M=8192, N=8192, K=8192, dtype="bf16")),
    "gemm_bf16_4096": ("gemm", dict(M=4096, N=4096, K=4096, dtype="bf16")),
    "gemm_bf16_16384": ("gemm", dict(M=16384, N=16384, K=16384, dtype="bf16")),
    "gemm_i8_8192": ("gemm", dict(M=8192, N=8192, K=8192, dtype="i8")),
    "gemm_i8_4096": ("gemm", dict(M=4096, N=4096, K=4096, dtype="i8")),
    "gemm_i8_16384": ("gemm", dict(M=16384, N=16384, K=16384, dtype="i8")),
    "sgemm_1024": ("gemm", dict(M=1024, N=1024, K=1024, dtype="f32")),
    "conv_cfg2": ("conv", dict(N=64, CI=256, CO=256, KY=3, KX=3, OY=14, OX=14)),
    "ttm_cfg3": ("ttm", dict(L=256, I=512, J=512, K=256)),
    "mttkrp_cfg3": ("mttkrp", dict(L=512, I=512, K=512, R=64)),
    "capsule_cfg4": ("capsule", dict(N=1, NN=32, CI=32, CII=32, CO=32, KY=3, KX=3, OY=16, OX=16, s=1)),
    # the GER design's A10 constants with its 32 x 32 outer loops: 10240 x 16384 elements
    "ger_a10": ("ger", dict(KKK=16, III=10, II=32, KK=32, K=32, I=32)),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm=d["hbm_gbs"], burst=d["bf16_tflops"], sustained=d["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, burst=1590.0, sustained=1400.0, src="fallback")


def flops_bytes(kind, w):
    """Algorithmic FLOPs and bytes (inputs once + output once) of one step."""
    if kind == "gemm":
        es = {"bf16": 2, "f16": 2, "i8": 1, "f32": 4}[w["dtype"]]
        return 2.0 * w["M"] * w["N"] * w["K"], es * (w["M"] * w["K"] + w["K"] * w["N"]) + 4 * w["M"] * w["N"]
    if kind == "conv":
        IY, IX = w["OY"] + w["KY"] - 1, w["OX"] + w["KX"] - 1
        f = 2.0 * w["N"] * w["CO"] * w["OY"] * w["OX"] * w["CI"] * w["KY"] * w["KX"]
        b = 4 * (w["N"] * w["CI"] * IY * IX + w["CI"] * w["CO"] * w["KY"] * w["KX"] + w["N"] * w["CO"] * w["OY"] * w["OX"])
        return f, b
    if kind == "ttm":
        f = 2.0 * w["I"] * w["J"] * w["K"] * w["L"]
        return f, 4 * (w["L"] * w["I"] * w["J"] + w["L"] * w["K"] + w["I"] * w["J"] * w["K"])
    if kind == "mttkrp":
        f = 2.0 * w["I"] * w["L"] * w["K"] * w["R"] + 2.0 * w["I"] * w["K"] * w["R"]
        return f, 4 * (w["L"] * w["I"] * w["K"] + w["L"] * w["R"] + w["K"] * w["R"] + w["I"] * w["R"])
    if kind == "ger":
        ti, tk = w["III"] * w["II"] * w["I"], w["KKK"] * w["KK"] * w["K"]
        return 2.0 * ti * tk, 4 * (2 * ti * tk + ti + tk)
    if kind == "capsule":
        s = w["s"]
        IY, IX = s * w["OY"] + w["KY"] - s, s * w["OX"] + w["KX"] - s
        NT = w["N"] * w["NN"]
        f = 2.0 * NT * w["CO"] * 16 * w["OY"] * w["OX"] * w["CI"] * 4 * w["KY"] * w["KX"]
        b = 4 * (16 * w["CI"] * IY * IX * NT + 16 * w["CI"] * w["CO"] * w["KY"] * w["KX"] + w["CO"] * 16 * w["OY"] * w["OX"] * NT)
        return f, b
    raise ValueError(kind)


# ----------------------------------------------------------------------------------- inputs
def make_inputs(kind, w, seed, rank):
    """Seeded synthetic host arrays (numpy) in the reference layouts, plus output shape/dtype."""
    import numpy as np
    from tests import oracle_lib as O  # generators only (Philox keyed by seed/tensor id)
    if kind == "gemm":
        M, N, K, dt = w["M"], w["N"], w["K"], w["dtype"]
        if dt == "i8":
            return [O.int8(seed, 1, (M, K)), O.int8(seed, 2 + rank, (K, N))], (M, N), np.int32, [dt, dt]
        A, B = O.uniform(seed, 1, (M, K)), O.uniform(seed, 2 + rank, (K, N))
        if dt == "bf16":
            return [O.to_bf16(A), O.to_bf16(B)], (M, N), np.float32, [dt, dt]
        return [A, B], (M, N), np.float32, [dt, dt]
    if kind == "conv":
        IY, IX = w["OY"] + w["KY"] - 1, w["OX"] + w["KX"] - 1
        I2 = np.zeros((IX, IY, w["N"] * w["CI"]), np.float32)
        I2[1:-1, 1:-1, :] = O.uniform(seed, 1 + rank, (IX - 2, IY - 2, w["N"] * w["CI"]))  # "pad 1": zero border
        K2 = O.normal(seed, 2, (w["CI"] * w["KY"], w["CO"] * w["KX"]), (1.0 / (w["KY"] * w["KX"] * w["CI"])) ** 0.5)
        return [I2.reshape(IX * IY, -1), K2], (w["OY"] * w["OX"], w["CO"] * w["N"]), np.float32, ["f32", "f32"]
    if kind == "ttm":
        return ([O.uniform(seed, 1 + rank, (w["J"], w["I"], w["L"])), O.uniform(seed, 2, (w["K"], w["L"]))],
                (w["K"], w["J"], w["I"]), np.float32, ["f32", "f32"])
    if kind == "mttkrp":
        return ([O.uniform(seed, 1 + rank, (w["K"], w["I"], w["L"])), O.uniform(seed, 2, (w["R"], w["K"])),
                 O.uniform(seed, 3, (w["R"], w["L"]))], (w["R"], w["I"]), np.float32, ["f32"] * 3)
    if kind == "ger":
        ti, tk = w["III"] * w["II"] * w["I"], w["KKK"] * w["KK"] * w["K"]
        return ([O.uniform(seed, 1 + rank, (ti, tk)), O.uniform(seed, 2, (ti,)), O.uniform(seed, 3, (tk,))],
                (w["I"], w["K"], w["KK"], w["II"], w["III"], w["KKK"]), np.float32, ["f32"] * 3)
    if kind == "capsule":
        s = w["s"]
        IY, IX = s * w["OY"] + w["KY"] - s, s * w["OX"] + w["KX"] - s
        P2 = O.normal(seed, 1 + rank, (IY * IX * w["N"], w["CI"] * 16 * w["NN"]), 0.1)
        W2 = O.normal(seed, 2, (w["CI"] * w["KY"] * w["KX"] * 4, w["CO"] * 4), 0.1)
        return [P2, W2], (w["OY"] * w["OX"] * w["N"], w["CO"] * 16 * w["NN"]), np.float32, ["f32", "f32"]
    raise ValueError(kind)


def make_desc(kind, w):
    import t2sp_b200
    if kind == "conv":
        d = t2sp_b200.ConvDesc()
        d.CI, d.CO, d.KY, d.KX, d.OY, d.OX = w["CI"], w["CO"], w["KY"], w["KX"], w["OY"], w["OX"]
        return d
    if kind == "capsule":
        d = t2sp_b200.CapsuleDesc()
        d.CI, d.CII, d.CO, d.KY, d.KX, d.OY, d.OX = w["CI"], w["CII"], w["CO"], w["KY"], w["KX"], w["OY"], w["OX"]
        d.MY = d.MX = d.MK = 4
        d.NN, d.stride = w["NN"], w["s"]
        return d
    return None


def call_op(kind, bufs, out, desc):
    import t2sp_b200
    if kind == "gemm":
        return t2sp_b200.gemm(bufs[0], bufs[1], out, desc)
    if kind == "conv":
        return t2sp_b200.conv(bufs[0], bufs[1], out, desc)
    if kind == "capsule":
        return t2sp_b200.capsule(bufs[0], bufs[1], out, desc)
    if kind == "ttm":
        return t2sp_b200.ttm(bufs[0], bufs[1], out, desc)
    if kind == "ger":
        return t2sp_b200.ger(bufs[0], bufs[1], bufs[2], out)
    return t2sp_b200.mttkrp(bufs[0], bufs[1], bufs[2], out, desc)


# ----------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons through NVML from a background thread
    while the timed region runs (read-only queries; nothing about the GPU is changed)."""

    def __init__(self, gpu_index, period_s=0.005):
        import threading
        self.samples, self.reason_bits, self.sm_max, self.err = [], 0, None, None
        self._stop = threading.Event()
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = gpu_index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if gpu_index < len(ids) and ids[gpu_index].isdigit():
                    phys = int(ids[gpu_index])
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # NVML missing: report that instead of inventing numbers
            self.err = f"NVML unavailable: {e}"
            self.nv = None
        self.period = period_s
        self.thread = threading.Thread(target=self._run, daemon=True)
        if self.nv is not None:
            self.thread.start()

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            except Exception as e:
                self.err = str(e)
                break
            time.sleep(self.period)

    def stop(self):
        self._stop.set()
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.err]}
        self.thread.join(timeout=2)
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        reasons = sorted(k for k, bit in names.items() if self.reason_bits & bit)
        sm = self.samples
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.sm_max, "reasons": reasons,
                "samples": len(sm)}


# ----------------------------------------------------------------------------------- CPU arms
def cpu_sample(kind, w, budget_s=12.0):
    """Times the CPU oracle on a bounded sample of the workload; returns (flop/s, description, threads)."""
    import numpy as np
    from tests import oracle_lib as O
    threads = int(O.load().oracle_threads())
    if kind == "gemm" and w["dtype"] in ("bf16", "i8"):
        M, N, K = w["M"], w["N"], w["K"]
        arrs, _, _, _ = make_inputs(kind, dict(w, M=min(M, 2048)), 0, 0)
        A, B = arrs
        rows = 32
        while True:
            t0 = time.perf_counter()
            if w["dtype"] == "bf16":
                O.gemm_h16(A[:rows], B, 0)
            else:
                O.gemm_i8(A[:rows], B)
            dt = time.perf_counter() - t0
            if dt * 4 > budget_s or rows * 2 > A.shape[0]:
                break
            rows *= 2 if dt * 8 > budget_s else 4
            rows = min(rows, A.shape[0])
        return 2.0 * rows * N * K / dt, f"{rows} of {M} output rows (all {N} columns, K={K}), {dt:.2f} s", threads
    arrs, _, _, _ = make_inputs(kind, w, 0, 0)
    f, _ = flops_bytes(kind, w)
    t0 = time.perf_counter()
    if kind == "gemm":
        O.gemm_f32(arrs[0], arrs[1])
    elif kind == "conv":
        O.conv_f32(arrs[0], arrs[1], w["N"], w["CI"], w["CO"], w["KY"], w["KX"], w["OY"], w["OX"])
    elif kind == "ttm":
        O.ttm_f32(arrs[0], arrs[1])
    elif kind == "mttkrp":
        O.mttkrp_f32(arrs[0], arrs[1], arrs[2])
    elif kind == "ger":
        O.ger_f32(arrs[0], arrs[1], arrs[2], w["KKK"], w["III"], w["II"], w["KK"], w["K"], w["I"])
    else:
        O.capsule_f32(arrs[0], arrs[1], w["N"], w["NN"], w["CI"], w["CII"], w["CO"], w["KY"], w["KX"], w["OY"], w["OX"],
                      4, 4, 4, w["s"])
    dt = time.perf_counter() - t0
    return f / dt, f"whole workload once, {dt:.2f} s", threads


def run_reference(args, kind, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t_begin = time.perf_counter()
    vals = []
    desc = ""
    threads = 1
    budget = max(2.0, min(12.0, 60.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        v, desc, threads = cpu_sample(kind, w, budget_s=budget)
        if i >= args.warmup:
            vals.append(v)
    tf = statistics.mean(vals) / 1e12
    f, _ = flops_bytes(kind, w)
    line = {
        "impl": "reference", "metric": "throughput", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": f / (tf * 1e12) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.get("dtype", "f32"),
        "data": "synthetic", "config": {"workload": name, **{k: v for k, v in w.items()}},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": "per step: " + desc},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference specification (oracle/); the reference's own Halide x86 path "
                "needs LLVM/clang, which this image lacks; ms_per_step is extrapolated from the sample to the whole workload",
        "wall_s": time.perf_counter() - t_begin,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm_bf16_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    kind, w = WORKLOADS[args.workload]
    if args.impl == "reference":
        return run_reference(args, kind, w, args.workload)
    args.warmup = max(args.warmup, 3)

    import numpy as np
    import torch
    import t2sp_b200
    from t2sp_b200 import Buffer, build
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank == 0:
        build.build()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: t2sp_b200 has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
    L = t2sp_b200.lib()
    L.t2sp_b200_set_device(local_rank)
    stream = torch.cuda.current_stream()
    L.t2sp_b200_set_stream(ctypes.c_void_p(stream.cuda_stream))

    arrs, out_shape, out_dtype, dts = make_inputs(kind, w, seed=0, rank=rank)
    desc = make_desc(kind, w)
    flops, abytes = flops_bytes(kind, w)

    # ---- resident arm: device tensors wrapped as halide buffers
    dev_in = [torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda() for a in arrs]
    dev_out = torch.empty(out_shape, dtype=torch.int32 if out_dtype == np.int32 else torch.float32, device="cuda")
    bufs = []
    for a, t, dt in zip(arrs, dev_in, dts):
        b = Buffer(tuple(reversed(a.shape)), dt)
        t2sp_b200.wrap_device(b, t.data_ptr())
        bufs.append(b)
    ob = Buffer(tuple(reversed(out_shape)), "i32" if out_dtype == np.int32 else "f32")
    t2sp_b200.wrap_device(ob, dev_out.data_ptr())
    L.t2sp_b200_set_async(1)

    def sync_all():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        rc = call_op(kind, bufs, ob, desc)
        if rc != 0:
            raise SystemExit(f"hot path failed with halide error {rc}")
    rc = L.t2sp_b200_sync()
    if rc != 0:
        raise SystemExit(f"hot path failed with halide error {rc}")
    sync_all()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = L.t2sp_b200_kernel_launches()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    evs[0].record(stream)
    for i in range(args.steps):
        call_op(kind, bufs, ob, desc)
        evs[i + 1].record(stream)
    sync_all()
    clocks = sampler.stop() if sampler else None
    launches = int(L.t2sp_b200_kernel_launches() - launches0)
    rc = L.t2sp_b200_sync()
    if rc != 0:
        raise SystemExit(f"hot path failed with halide error {rc}")
    total_ms = evs[0].elapsed_time(evs[-1])
    step_ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    if dist is not None:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    L.t2sp_b200_set_async(0)
    ms_per_step = total_ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12

    # ---- end-to-end arm: pinned host buffers through the synchronous C-ABI call
    e2e = None
    if not args.no_e2e:
        pin_in = []
        for a in arrs:
            t = torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).pin_memory()
            pin_in.append(t)
        pin_out = torch.empty(out_shape, dtype=torch.int32 if out_dtype == np.int32 else torch.float32).pin_memory()
        hb = [Buffer(tuple(reversed(a.shape)), dt, host=t.data_ptr(), keepalive=t) for a, t, dt in zip(arrs, pin_in, dts)]
        hob = Buffer(tuple(reversed(out_shape)), "i32" if out_dtype == np.int32 else "f32", host=pin_out.data_ptr(),
                     keepalive=pin_out)
        e2e_steps = max(1, min(args.steps, 10))
        for _ in range(2):
            rc = call_op(kind, hb, hob, desc)
            if rc != 0:
                raise SystemExit(f"end-to-end call failed with halide error {rc}")
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            call_op(kind, hb, hob, desc)
        e1.record(stream)
        sync_all()
        e2e_ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([e2e_ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e = {"value": world * flops / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(sum(a.nbytes for a in arrs)),
               "d2h_bytes_per_step": int(np.prod(out_shape)) * 4, "steps": e2e_steps,
               "ms_per_step": e2e_ms / e2e_steps}

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    pk = peaks()
    kernel_ms = statistics.mean(step_ms)
    # fp32 contractions run as 3xTF32: their tensor ceiling is the bf16 peak / 2 / 3. The bound is
    # whichever of (bytes / HBM bandwidth) and (FLOPs / tensor ceiling) is the longer time.
    t_hbm = abytes / (pk["hbm"] * 1e9)
    t_tensor = flops / (pk["burst"] * {"bf16": 1.0, "f16": 1.0, "i8": 2.0, "f32": 1.0 / 6.0}[w.get("dtype", "f32")] * 1e12)
    hbm_bound = t_hbm > t_tensor
    if hbm_bound:
        achieved, peak, unit = abytes / (kernel_ms * 1e-3) / 1e9, pk["hbm"], "GB/s"
        peak_note = f"{pk['src']} HBM copy bandwidth"
    else:
        long_run = total_ms > 1000.0
        bf16_peak = pk["sustained"] if long_run else pk["burst"]
        dt = w.get("dtype", "f32")
        scale = {"bf16": 1.0, "f16": 1.0, "i8": 2.0, "f32": 1.0 / 6.0}[dt]
        achieved, peak, unit = flops / (kernel_ms * 1e-3) / 1e12, bf16_peak * scale, "TFLOP/s"
        peak_note = (f"{pk['src']} cuBLAS bf16 {'sustained' if long_run else 'burst'} {bf16_peak} TFLOP/s"
                     + {1.0: "", 2.0: " x2 (int8 rate)", 1.0 / 6.0: " /2 (tf32 rate) /3 (three MMAs per product)"}[scale])
    traffic = KNOWN_TRAFFIC.get(args.workload)
    line = {
        "metric": "throughput", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": w.get("dtype", "f32"), "data": "synthetic",
        "config": {"workload": args.workload, **w, "sharding": "N-column slab per GPU (A replicated)" if kind == "gemm" else "independent batch/slab per GPU",
                   "l2": "inputs+output larger than L2" if abytes > 126e6 else "operands fit in L2 (working set smaller than 126 MB)"},
        "e2e": e2e, "gpu_launches": launches,
        "roofline": {"bound": "hbm" if hbm_bound else "tensor", "achieved": achieved, "peak": peak, "unit": unit,
                     "frac": achieved / peak, "traffic": traffic, "peak_source": peak_note,
                     "kernel_ms": kernel_ms, "algorithmic_flops": flops, "algorithmic_bytes": abytes},
        "clocks": clocks,
    }
    if not args.no_cpu_baseline and world == 1:
        v, sample, threads = cpu_sample(kind, w)
        line["cpu_baseline"] = {"value": v / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample}
    print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (None where no capture has been taken).
KNOWN_TRAFFIC = {
    # profiles/gemm_bf16_8192_pair_dram_traffic.md: mean of two launches of the 512 x 256 pair kernel
    # (837695488 + 237744128 and 849618944 + 235083520 bytes read + written)
    "gemm_bf16_8192": 1059237248,
    # small-case captures (one launch each): profiles/gemm_bf16_i8_4096_pair_kernels_full.md and
    # profiles/fp32_3xtf32_kernels_conv_ttm_mttkrp_capsule_sgemm_full.md
    "gemm_bf16_4096": 94957312 + 32456192,
    "gemm_i8_4096": 35462400 + 18725376,
    "conv_cfg2": 19220480 + 142336,
    "ttm_cfg3": 268876800 + 218153984,
    "mttkrp_cfg3": 537606400 + 3475456,
    "capsule_cfg4": 21994496 + 7168,
    "sgemm_1024": 8471808,
    # profiles/ger_a10_rows_kernel_full.md
    "ger_a10": 671217664 + 620295680,
}

if __name__ == "__main__":
    main()
