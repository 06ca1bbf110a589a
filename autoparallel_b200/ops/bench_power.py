"""Sustained GEMM throughput, SM clock and power of this framework's tcgen05 GEMM against the library GEMM.

    python -m autoparallel_b200.ops.bench_power [--seconds 3] [--zeros]

A B200 under its 1 kW cap is energy-bound on dense GEMMs: what a kernel sustains is set by its energy per FLOP,
not by its per-clock efficiency, and the data matter (operand toggling is most of the tensor-core power; zeros run
at the maximum clock).  Each case loops one GEMM form for a few seconds with operands rotated through three sets
(larger than L2 together), samples clock and power through NVML while it runs, and prints TFLOP/s, the median clock,
the mean power and pJ/FLOP of the second half of the loop.  Reading the settings only: nothing is set or reset.
"""
from __future__ import annotations

import argparse
import statistics
import threading
import time

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seconds", type=float, default=3.0)
    ap.add_argument("--zeros", action="store_true", help="operands of zeros instead of N(0, 0.05): the data-independent power")
    args = ap.parse_args()
    import pynvml

    from . import cuda_impl

    cuda_impl.ensure_loaded()
    C = cuda_impl.extension()
    pynvml.nvmlInit()
    h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
    st = cuda_impl.status_buffer(torch.device("cuda"))
    bf = torch.bfloat16

    def sample(stop, out):
        while not stop.is_set():
            out.append((pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM), pynvml.nvmlDeviceGetPowerUsage(h) / 1e3))
            time.sleep(0.05)

    def run(label, fns, flops):
        for f in fns:
            f()
        torch.cuda.synchronize()
        stop, out = threading.Event(), []
        th = threading.Thread(target=sample, args=(stop, out))
        th.start()
        t0, n = time.time(), 0
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        while time.time() - t0 < args.seconds:
            for _ in range(8):
                for f in fns:
                    f()
            n += 8 * len(fns)
            torch.cuda.synchronize()
        e.record()
        torch.cuda.synchronize()
        stop.set()
        th.join()
        half = out[len(out) // 2:] or [(0, 0.0)]
        clk, pw = statistics.median(x[0] for x in half), statistics.mean(x[1] for x in half)
        tf = flops * n / s.elapsed_time(e) / 1e9
        print(f"{label:46s} {tf:7.1f} TF/s  {clk:5.0f} MHz  {pw:6.1f} W  {pw / max(tf, 1e-9):5.3f} pJ/FLOP", flush=True)
        time.sleep(1.0)

    def R(*shape):
        if args.zeros:
            return torch.zeros(*shape, device="cuda", dtype=bf)
        return (torch.randn(*shape, device="cuda", dtype=torch.float32) * 0.05).to(bf)

    T, D, F, NB = 8192, 4096, 14336, 3
    xs, w1, dys = [R(T, D) for _ in range(NB)], [R(F, D) for _ in range(NB)], [R(T, F) for _ in range(NB)]
    y = [torch.empty(T, F, device="cuda", dtype=bf) for _ in range(NB)]
    dx = [torch.empty(T, D, device="cuda", dtype=bf) for _ in range(NB)]
    dw32 = [torch.empty(F, D, device="cuda", dtype=torch.float32) for _ in range(NB)]
    dw16 = [torch.empty(F, D, device="cuda", dtype=bf) for _ in range(NB)]
    fl = 2.0 * T * D * F
    rng = range(NB)
    run("library NT forward [8192x14336x4096]", [(lambda i=i: torch.matmul(xs[i], w1[i].t(), out=y[i])) for i in rng], fl)
    run("own     NT forward", [(lambda i=i: C.gemm(xs[i], w1[i], y[i], False, False, st)) for i in rng], fl)
    run("library NN dgrad   [8192x4096x14336]", [(lambda i=i: torch.matmul(dys[i], w1[i], out=dx[i])) for i in rng], fl)
    run("own     NN dgrad", [(lambda i=i: C.gemm(dys[i], w1[i], dx[i], False, True, st)) for i in rng], fl)
    run("library TN wgrad bf16 out [14336x4096x8192]", [(lambda i=i: torch.matmul(dys[i].t(), xs[i], out=dw16[i])) for i in rng], fl)
    run("own     TN wgrad bf16 out", [(lambda i=i: C.gemm(dys[i], xs[i], dw16[i], True, True, st)) for i in rng], fl)
    run("own     TN wgrad fp32 out", [(lambda i=i: C.gemm(dys[i], xs[i], dw32[i], True, True, st)) for i in rng], fl)
    wk = [R(1024, D) for _ in rng]
    ok = [torch.empty(T, 1024, device="cuda", dtype=bf) for _ in rng]
    run("library NT [8192x1024x4096]", [(lambda i=i: torch.matmul(xs[i], wk[i].t(), out=ok[i])) for i in rng], 2.0 * T * 1024 * D)
    run("own     NT [8192x1024x4096]", [(lambda i=i: C.gemm(xs[i], wk[i], ok[i], False, False, st)) for i in rng], 2.0 * T * 1024 * D)
    cuda_impl.check_status()


if __name__ == "__main__":
    main()
