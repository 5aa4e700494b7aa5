#!/usr/bin/env python
"""Benchmark of the hot path: one dense contraction per step.

Default workload: the 8192^3 bf16 GEMM with fp32 accumulation, the configuration the headline
TFLOP/s figure is quoted on. With N>1 ranks (launched by torchrun, one rank per GPU) the SAME
problem is split: rank g computes columns [g N/G, (g+1) N/G) of C from all of A and its columns of
B through the library's sharded entry (strong scaling; operands are placed before the timed
region); no collective is on the data path, NCCL carries the barrier, the max-over-ranks time and,
timed separately as `gather_ms`, the all-gather that puts all of C on every GPU.

`value`   : operands already resident in HBM, kernels timed with CUDA events on the launching stream.
`e2e`     : the same contraction through the C-ABI entry with HOST buffers (pinned; `pageable` beside it),
            so every step pays the host->device copy of A and B and the device->host copy of C.
`sustained`, `workloads`: the headline launch repeated for more than two seconds, and the other
            configurations device-timed for `steps` launches each (single GPU).
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
    # what one of 8 GPUs computes of the 8192^3 problem when it is sharded by N-column slabs
    "gemm_bf16_slab8": ("gemm", dict(M=8192, N=1024, K=8192, dtype="bf16")),
    "gemm_bf16_16384": ("gemm", dict(M=16384, N=16384, K=16384, dtype="bf16")),
    "gemm_i8_8192": ("gemm", dict(M=8192, N=8192, K=8192, dtype="i8")),
    "gemm_i8_4096": ("gemm", dict(M=4096, N=4096, K=4096, dtype="i8")),
    "gemm_i8_16384": ("gemm", dict(M=16384, N=16384, K=16384, dtype="i8")),
    "sgemm_1024": ("gemm", dict(M=1024, N=1024, K=1024, dtype="f32")),
    "sgemm_4096": ("gemm", dict(M=4096, N=4096, K=4096, dtype="f32")),
    "sgemm_8192": ("gemm", dict(M=8192, N=8192, K=8192, dtype="f32")),
    "conv_cfg2": ("conv", dict(N=64, CI=256, CO=256, KY=3, KX=3, OY=14, OX=14)),
    "ttm_cfg3": ("ttm", dict(L=256, I=512, J=512, K=256)),
    "mttkrp_cfg3": ("mttkrp", dict(L=512, I=512, K=512, R=64)),
    "sgemm_n128": ("gemm", dict(M=32768, N=128, K=1152, dtype="f32")),  # the GEMM shape of capsule_cfg4
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
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w.get("dtype", "f32"),
        "data": "synthetic", "config": {"workload": name, **{k: v for k, v in w.items()}},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": "per step: " + desc},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference specification (oracle/); the reference's own Halide x86 path "
                "needs LLVM/clang, which this image lacks; ms_per_step is extrapolated from the sample to the whole workload",
        "wall_s": time.perf_counter() - t_begin,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------- GPU arm
SIDE_WORKLOADS = ["sgemm_1024", "conv_cfg2", "ttm_cfg3", "mttkrp_cfg3", "capsule_cfg4", "gemm_bf16_4096",
                  "gemm_bf16_16384", "gemm_i8_8192"]
RATE = {"bf16": 1.0, "f16": 1.0, "i8": 2.0, "f32": 1.0 / 6.0}  # tensor ceiling relative to the bf16 peak
# fp32 workloads that run on the pair kernel with the A operand in tensor memory (many row tiles over one B): per 32
# contraction values four TF32 MMAs (hi * hi) and four bf16 MMAs (the cross terms) where a bf16 GEMM issues two, so the
# ceiling is a quarter of the bf16 peak instead of the sixth of three TF32 passes
BF16_CROSS_TERMS = {"conv_cfg2", "ttm_cfg3", "capsule_cfg4", "sgemm_n128", "sgemm_4096", "sgemm_8192"}


class Resident:
    """One workload with its operands resident in HBM, wrapped as halide buffers; call() enqueues one step
    (this rank's shard of it when world > 1) on the library's stream."""

    def __init__(self, name, rank, world, device_generated=False):
        import numpy as np
        import torch
        import t2sp_b200
        from t2sp_b200 import Buffer
        self.name, self.rank, self.world = name, rank, world
        self.kind, self.w = WORKLOADS[name]
        kind, w = self.kind, self.w
        self.desc = make_desc(kind, w)
        self.flops, self.abytes = flops_bytes(kind, w)
        if device_generated and kind == "gemm" and w["dtype"] in ("bf16", "i8"):
            # large operands are drawn on the device (same distributions, torch's seeded generator)
            g = torch.Generator(device="cuda")
            g.manual_seed(1234)
            M, N, K = w["M"], w["N"], w["K"]
            if w["dtype"] == "bf16":
                mk = lambda r, c: (torch.rand((r, c), generator=g, device="cuda") * 2 - 1).to(torch.bfloat16)
                out_t = torch.float32
            else:
                mk = lambda r, c: torch.randint(-127, 128, (r, c), generator=g, device="cuda", dtype=torch.int8)
                out_t = torch.int32
            self.dev_in = [mk(M, K), mk(K, N)]
            self.shapes, self.dts, self.out_shape, self.out_dt = [(M, K), (K, N)], [w["dtype"]] * 2, (M, N), out_t
            self.host_in = None
        else:
            arrs, out_shape, out_dtype, dts = make_inputs(kind, w, seed=0, rank=0)
            self.host_in = arrs
            self.dev_in = [torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda() for a in arrs]
            self.shapes, self.dts, self.out_shape = [a.shape for a in arrs], dts, out_shape
            self.out_dt = torch.int32 if out_dtype == np.int32 else torch.float32
        self.dev_out = torch.empty(self.out_shape, dtype=self.out_dt, device="cuda")
        self.bufs = []
        for shp, t, dt in zip(self.shapes, self.dev_in, self.dts):
            b = Buffer(tuple(reversed(shp)), dt)
            t2sp_b200.wrap_device(b, t.data_ptr())
            self.bufs.append(b)
        self.ob = Buffer(tuple(reversed(self.out_shape)), "i32" if self.out_dt == torch.int32 else "f32")
        t2sp_b200.wrap_device(self.ob, self.dev_out.data_ptr())

    def call(self):
        if self.world == 1:
            return call_op(self.kind, self.bufs, self.ob, self.desc)
        from t2sp_b200 import shard
        k, b, r, n = self.kind, self.bufs, self.rank, self.world
        if k == "gemm":
            return shard.gemm_shard(b[0], b[1], self.ob, r, n)
        if k == "conv":
            return shard.conv_shard(b[0], b[1], self.ob, self.desc, r, n)
        if k == "capsule":
            return shard.capsule_shard(b[0], b[1], self.ob, self.desc, r, n)
        if k == "ttm":
            return shard.ttm_shard(b[0], b[1], self.ob, r, n)
        if k == "mttkrp":
            return shard.mttkrp_shard(b[0], b[1], b[2], self.ob, r, n)
        raise SystemExit(f"workload kind {k} does not shard")

    SHARDING = {"gemm": "one problem, N-column slabs of B and C per GPU, A replicated, placement outside the timed region",
                "conv": "one problem, batch items per GPU, weights replicated",
                "capsule": "one problem, batch items per GPU, weights replicated",
                "ttm": "one problem, j slabs per GPU, b replicated",
                "mttkrp": "one problem, k ranges (the contraction) per GPU; partial results are not summed inside the timed region",
                "ger": "not sharded"}


def roofline_of(name, kernel_ms, long_run=False):
    """Which roofline bounds the workload (the longer of bytes / HBM bandwidth and FLOPs / tensor ceiling) and
    how close kernel_ms comes to it."""
    kind, w = WORKLOADS[name]
    flops, abytes = flops_bytes(kind, w)
    pk = peaks()
    scale = 0.25 if name in BF16_CROSS_TERMS else RATE[w.get("dtype", "f32")]
    t_hbm = abytes / (pk["hbm"] * 1e9)
    t_tensor = flops / (pk["burst"] * scale * 1e12)
    if t_hbm > t_tensor:
        achieved, peak, unit, bound = abytes / (kernel_ms * 1e-3) / 1e9, pk["hbm"], "GB/s", "hbm"
        note = f"{pk['src']} HBM copy bandwidth"
    else:
        bf16_peak = pk["sustained"] if long_run else pk["burst"]
        achieved, peak, unit, bound = flops / (kernel_ms * 1e-3) / 1e12, bf16_peak * scale, "TFLOP/s", "tensor"
        note = (f"{pk['src']} cuBLAS bf16 {'sustained' if long_run else 'burst'} {bf16_peak} TFLOP/s"
                + {1.0: "", 2.0: " x2 (int8 rate)", 1.0 / 6.0: " /2 (tf32 rate) /3 (three MMAs per product)",
                   0.25: " /4 (one TF32 pass = two bf16 passes, plus two bf16 passes for the cross terms)"}[scale])
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
            "traffic": KNOWN_TRAFFIC.get(name), "peak_source": note, "kernel_ms": kernel_ms,
            "algorithmic_flops": flops, "algorithmic_bytes": abytes}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm_bf16_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the sustained run, the other workloads and the gather timing")
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
    stream = torch.cuda.Stream()  # the library launches on this stream; the timing events are recorded on it
    torch.cuda.set_stream(stream)
    L.t2sp_b200_set_stream(ctypes.c_void_p(stream.cuda_stream))
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # twice the 126 MB L2

    def sync_all():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def check(rc, what="hot path"):
        if rc != 0:
            raise SystemExit(f"{what} failed with halide error {rc}")

    def timed_region(job, steps, warmup):
        """W warm-up steps, then exactly `steps` steps between two events, barrier + synchronize on both
        sides; returns (total ms as the max over ranks, per-step ms of this rank, launches)."""
        L.t2sp_b200_set_async(1)
        for _ in range(warmup):
            check(job.call())
        check(L.t2sp_b200_sync())
        sync_all()
        n0 = L.t2sp_b200_kernel_launches()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        evs[0].record(stream)
        for i in range(steps):
            job.call()
            evs[i + 1].record(stream)
        sync_all()
        launches = int(L.t2sp_b200_kernel_launches() - n0)
        check(L.t2sp_b200_sync())
        L.t2sp_b200_set_async(0)
        total = max_over_ranks(evs[0].elapsed_time(evs[-1]))
        return total, [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)], launches

    def flushed_steps(job, steps, warmup):
        """Per-step device times with L2 flushed (a 256 MB write) between steps; for working sets that fit L2."""
        L.t2sp_b200_set_async(1)
        for _ in range(warmup):
            check(job.call())
        check(L.t2sp_b200_sync())
        pairs = []
        for _ in range(steps):
            flush_buf.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            job.call()
            e1.record(stream)
            pairs.append((e0, e1))
        torch.cuda.synchronize()
        check(L.t2sp_b200_sync())
        L.t2sp_b200_set_async(0)
        return [a.elapsed_time(b) for a, b in pairs]

    # ---- headline: operands resident in HBM
    job = Resident(args.workload, rank, world)
    flops, abytes = job.flops, job.abytes
    sampler = ClockSampler(local_rank) if rank == 0 else None
    total_ms, step_ms, launches = timed_region(job, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    ms_per_step = total_ms / args.steps
    value = flops / (ms_per_step * 1e-3) / 1e12  # one problem whatever the number of GPUs

    extras = {}
    if not args.no_extras:
        # ---- the same launch back to back for more than two seconds: the power-capped regime
        n_sus = int(min(20000, max(50, 2200.0 / max(ms_per_step, 1e-3))))
        sus_total, _, _ = timed_region(job, n_sus, 1)
        sus_ms = sus_total / n_sus
        sus_tf = flops / (sus_ms * 1e-3) / 1e12
        pk = peaks()
        extras["sustained"] = {"steps": n_sus, "ms_per_step": sus_ms, "value": sus_tf, "unit": "TFLOP/s",
                               "region_s": sus_total * 1e-3,
                               "frac": (sus_tf / world / (pk["sustained"] * RATE[w.get("dtype", "f32")])) if kind == "gemm" else None,
                               "peak_source": f"{pk['src']} cuBLAS bf16 sustained {pk['sustained']} TFLOP/s"}
        # ---- what the caller pays to have all of C on every GPU afterwards: NCCL all-gather of the column slabs
        if world > 1 and kind == "gemm":
            from t2sp_b200 import shard
            comm = shard.Comm(rank, world, shard.torch_id_exchange(dist, torch.device("cuda", local_rank)))
            L.t2sp_b200_set_async(1)
            for _ in range(2):
                check(comm.gather_columns(job.ob), "gather_columns")
            sync_all()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record(stream)
            for _ in range(5):
                comm.gather_columns(job.ob)
            g1.record(stream)
            sync_all()
            L.t2sp_b200_set_async(0)
            extras["gather_ms"] = max_over_ranks(g0.elapsed_time(g1) / 5)
            extras["gather_bytes_received_per_gpu"] = int(4 * w["M"] * (w["N"] - w["N"] // world))
            comm.destroy()

    # ---- end-to-end arm: host buffers through the synchronous C-ABI call (single GPU, or each rank its shard)
    e2e = None
    if not args.no_e2e:
        arrs = job.host_in
        out_shape = job.out_shape
        out_np = np.int32 if job.out_dt == torch.int32 else np.float32

        def host_job(pinned):
            class J:
                pass
            j = J()
            if pinned:
                tin = [torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).pin_memory() for a in arrs]
                tout = torch.empty(out_shape, dtype=job.out_dt).pin_memory()
                hb = [Buffer(tuple(reversed(a.shape)), dt, host=t.data_ptr(), keepalive=t) for a, t, dt in zip(arrs, tin, job.dts)]
                hob = Buffer(tuple(reversed(out_shape)), "i32" if out_np == np.int32 else "f32", host=tout.data_ptr(), keepalive=tout)
            else:
                hb = [Buffer.from_numpy(a, dtype=dt) for a, dt in zip(arrs, job.dts)]  # plain malloc'ed (pageable) memory
                hob = Buffer.from_numpy(np.empty(out_shape, out_np))
            h = Resident.__new__(Resident)
            h.kind, h.desc, h.rank, h.world, h.bufs, h.ob = kind, job.desc, rank, world, hb, hob
            return h

        def time_host(pinned, steps):
            h = host_job(pinned)
            for _ in range(2):
                check(h.call(), "end-to-end call")
            sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                h.call()
            e1.record(stream)
            sync_all()
            return max_over_ranks(e0.elapsed_time(e1)) / steps

        in_bytes = int(sum(a.nbytes for a in arrs))
        out_bytes = int(np.prod(out_shape)) * 4
        e2e_steps = max(1, min(args.steps, 10))
        ms_pin = time_host(True, e2e_steps)
        e2e = {"value": flops / (ms_pin * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": in_bytes,
               "d2h_bytes_per_step": out_bytes, "steps": e2e_steps, "ms_per_step": ms_pin, "host_memory": "pinned"}
        if not args.no_extras:
            ms_page = time_host(False, max(1, min(args.steps, 3)))
            e2e["pageable"] = {"value": flops / (ms_page * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_page,
                               "note": "the same call on plain malloc'ed host arrays, as Halide::Runtime::Buffer allocates them"}

    # ---- the other configurations, device-timed (single GPU): ~steps launches each, L2 flushed between steps
    # where the working set fits L2
    side = []
    if not args.no_extras and world == 1 and args.workload == "gemm_bf16_8192":
        del job
        torch.cuda.empty_cache()
        for name in SIDE_WORKLOADS:
            sj = Resident(name, 0, 1, device_generated=True)
            fits_l2 = sj.abytes <= 126e6
            if fits_l2:
                t = flushed_steps(sj, args.steps, 3)
            else:
                _, t, _ = timed_region(sj, args.steps, 3)
            r = roofline_of(name, statistics.mean(t))
            side.append({"workload": name, "ms_per_step": statistics.mean(t), "ms_min": min(t), "steps": args.steps,
                         "achieved": r["achieved"], "peak": r["peak"], "unit": r["unit"], "frac": r["frac"], "bound": r["bound"],
                         "peak_source": r["peak_source"], "l2": "flushed between steps" if fits_l2 else "inputs larger than L2"})
            del sj
            torch.cuda.empty_cache()

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    kernel_ms = statistics.mean(step_ms)
    roof = roofline_of(args.workload, kernel_ms, long_run=total_ms > 1000.0)
    if world > 1:
        # per GPU: its share of the work against one GPU's peak (every rank's launch does 1/world of the FLOPs)
        roof["achieved"] /= world
        roof["frac"] /= world
        roof["note"] = "per GPU: this rank's share of the problem over its own kernel time"
    line = {
        "metric": "throughput", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None, "dtype": w.get("dtype", "f32"), "data": "synthetic",
        "config": {"workload": args.workload, **w},
        "sharding": Resident.SHARDING[kind] if world > 1 else "single GPU",
        "l2": "inputs+output larger than L2, no flush" if abytes / world > 126e6 else "operands fit in L2 (working set smaller than 126 MB), no flush in the headline region",
        "e2e": e2e, "gpu_launches": launches, "roofline": roof, "clocks": clocks,
        "step_ms_min_max": [min(step_ms), max(step_ms)],
    }
    line.update(extras)
    if side:
        line["workloads"] = side
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
    # profiles/fp32_x3tm_kernel_ttm_conv_full.md
    "conv_cfg2": 21600256 + 485888,
    "ttm_cfg3": 269131520 + 217162752,
    # profiles/mttkrp_cfg3_mttkrp2_kernel_full.md
    "mttkrp_cfg3": 537191168 + 4868352,
    "capsule_cfg4": 22507008 + 11008,
    "sgemm_1024": 8471808,
    # profiles/ger_a10_rows_kernel_full.md
    "ger_a10": 671217664 + 620295680,
}

if __name__ == "__main__":
    main()
