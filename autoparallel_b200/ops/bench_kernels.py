"""Per-kernel timing against the machine's measured roofline.

``python -m autoparallel_b200.ops.bench_kernels [--json out.json]`` times each sm_100a kernel at
the Llama-3 8B shapes with CUDA events (3 warm-ups, inputs rotated through a pool larger than the
126 MB L2 so every timed launch reads cold data) and prints achieved TFLOP/s or GB/s next to the
fraction of the measured peak (``MEASURED_PEAKS.json`` beside the repo root if present, else
6.65 TB/s and 1.59 PFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        m = json.load(open(p))
        return m["hbm_gbs"], m["bf16_tflops"], m.get("bf16_tflops_sustained", m["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def time_fn(make_args, fn, iters=10, pool=4):
    """(median, best) milliseconds per call.  The calls of one round - one per argument set, so consecutive calls touch
    different memory (the sets together exceed L2 for the large cases) - are captured in a CUDA graph and replayed:
    what is timed is device time, not the host's cost of dispatching a short kernel."""
    argsets = [make_args() for _ in range(pool)]
    for i in range(3):
        fn(*argsets[i % pool])
    torch.cuda.synchronize()
    graph = None
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for a in argsets:
                fn(*a)
        graph = g
    except Exception:
        torch.cuda.synchronize()
        graph = None
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for i, (s, e) in enumerate(evs):
        s.record()
        if graph is not None:
            graph.replay()
        else:
            for a in argsets:
                fn(*a)
        e.record()
    torch.cuda.synchronize()
    ts = sorted(s.elapsed_time(e) / pool for s, e in evs)
    return ts[len(ts) // 2], ts[0]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", default=None, choices=["gemm_nt", "gemm_tn", "rms_norm_bwd", "xent_bwd", "grouped_mm", "attention", "moe_dispatch"],
                    help="run a single small case (what a profiler capture is taken on)")
    ap.add_argument("--pair", default=None, choices=["on", "off"], help="force the CTA-pair (cta_group::2) GEMM kernel on or off")
    ap.add_argument("--gemm-only", action="store_true", help="stop after the GEMM rows")
    ap.add_argument("--skip-gemm", action="store_true", help="bandwidth-bound kernels only (a short run for profiler captures)")
    args = ap.parse_args()
    from autoparallel_b200.ops import cuda_impl, library as L

    cuda_impl.ensure_loaded()
    if args.pair is not None:
        cuda_impl.extension().gemm_set_pair_mode(args.pair == "on")
    hbm, tf_burst, tf_sus, src = _peaks()
    dev = "cuda"
    bf = torch.bfloat16
    rows = []

    def rec(name, ms, best, flops=None, nbytes=None):
        r = {"kernel": name, "ms_median": ms, "ms_best": best}
        if flops:
            r["tflops"] = flops / best / 1e9
            r["frac_of_burst_gemm_peak"] = r["tflops"] / tf_burst
        if nbytes:
            r["gbs"] = nbytes / best / 1e6
            r["frac_of_copy_peak"] = r["gbs"] / hbm
        rows.append(r)
        extra = f"{r.get('tflops', 0):8.1f} TF/s ({r.get('frac_of_burst_gemm_peak', 0):.2f} of {src} burst)" if flops else \
            f"{r.get('gbs', 0):8.1f} GB/s ({r.get('frac_of_copy_peak', 0):.2f} of {src} copy)"
        print(f"{name:44s} {best:8.3f} ms  {extra}", flush=True)

    M = 8192
    if args.only:
        # one kernel, inputs larger than the 126 MB L2 but well under a GB, a handful of launches
        if args.only in ("gemm_nt", "gemm_tn"):
            ta = args.only == "gemm_tn"
            mk = (lambda: (torch.randn(4096, M, device=dev, dtype=bf), torch.randn(4096, 4096, device=dev, dtype=bf))) if ta else \
                (lambda: (torch.randn(M, 4096, device=dev, dtype=bf), torch.randn(4096, 4096, device=dev, dtype=bf)))
            ms, best = time_fn(mk, lambda a, b: L.ops.gemm(a, b, ta, not ta, bf), iters=3, pool=2)
            rec(f"{args.only} 8192x4096x4096", ms, best, flops=2.0 * M * 4096 * 4096)
        elif args.only == "attention":
            # causal, 8192 tokens, 32 query / 8 key-value heads of 128: the library kernel, or this package's own forward
            # kernel when APB200_ATTENTION_FWD=own is set
            mk = lambda: (torch.randn(1, M, 32, 128, device=dev, dtype=bf), torch.randn(1, M, 8, 128, device=dev, dtype=bf),
                          torch.randn(1, M, 8, 128, device=dev, dtype=bf))
            ms, best = time_fn(mk, lambda q, k, v: L.ops.attention(q, k, v, True, 128 ** -0.5), iters=3, pool=2)
            rec(f"attention fwd causal 8192 32q/8kv ({os.environ.get('APB200_ATTENTION_FWD', 'library')})", ms, best,
                flops=4.0 * M * M * 4096 * 0.5)
        elif args.only == "moe_dispatch":
            # the dispatch of the MoE configuration on one rank: 8192 tokens, top-8 of 64 experts, capacity factor 1.25, d = 2048;
            # this package's kernels against the index-operator formulas they replace (ops/moe_ops.py)
            from autoparallel_b200.ops import moe_ops

            T_, k_, E_, d_ = 8192, 8, 64, 2048
            C_ = int(1.25 * T_ * k_ / E_)
            gi = torch.stack([torch.randperm(E_, device=dev)[:k_] for _ in range(T_)])
            x = torch.randn(T_, d_, device=dev, dtype=bf)
            w = torch.rand(T_, k_, device=dev)
            slot = torch.ops.apb200.moe_slots(gi, E_, C_, 1)
            buf = torch.ops.apb200.moe_scatter(x, slot, w, E_, C_, 1)
            moved = 2 * T_ * k_ * d_ * 2
            for name, fn, ref, nb_ in (
                    ("moe_slots", lambda: torch.ops.apb200.moe_slots(gi, E_, C_, 1), lambda: moe_ops._moe_slots(gi, E_, C_, 1), T_ * k_ * 16),
                    ("moe_scatter", lambda: torch.ops.apb200.moe_scatter(x, slot, w, E_, C_, 1), lambda: moe_ops._moe_scatter(x, slot, w, E_, C_, 1),
                     moved + E_ * C_ * d_ * 2),
                    ("moe_gather", lambda: torch.ops.apb200.moe_gather(buf, slot, w), lambda: moe_ops._moe_gather(buf, slot, w), moved)):
                ms, best = time_fn(lambda: (), fn, iters=3, pool=2)
                rec(f"{name} {T_}x{k_} E={E_} C={C_} d={d_} (kernel)", ms, best, nbytes=nb_)
                ms, best = time_fn(lambda: (), ref, iters=3, pool=2)
                rec(f"{name} (index-operator formula)", ms, best, nbytes=nb_)
        elif args.only == "grouped_mm":
            E, Me, Ne, Ke = 8, 4096, 1408, 2048  # the expert projection of the MoE configuration at half its token count
            mk = lambda: (torch.randn(E, Me, Ke, device=dev, dtype=bf) * 0.05, torch.randn(E, Ke, Ne, device=dev, dtype=bf) * 0.05)
            ms, best = time_fn(mk, lambda a, b: torch.ops.apb200.grouped_mm(a, b, False, bf), iters=3, pool=2)
            rec(f"grouped_mm {E}x{Me}x{Ne}x{Ke}", ms, best, flops=2.0 * E * Me * Ne * Ke)
        elif args.only == "rms_norm_bwd":
            mk = lambda: (torch.randn(M, 4096, device=dev, dtype=bf), torch.randn(M, 4096, device=dev, dtype=bf), torch.randn(4096, device=dev, dtype=bf), torch.rand(M, device=dev))
            ms, best = time_fn(mk, lambda dy, x, w, r: L.ops.rms_norm_bwd(dy, x, w, r), iters=3, pool=2)
            rec("rms_norm bwd 8192x4096", ms, best, nbytes=3 * M * 4096 * 2)
        else:
            V = 32064
            mk = lambda: (torch.randn(M, device=dev), torch.randn(M, V, device=dev, dtype=bf), torch.randint(0, V, (M,), device=dev), torch.rand(M, device=dev) + 10)
            ms, best = time_fn(mk, lambda g, lg, lb, lse: L.ops.cross_entropy_bwd(g, lg, lb, lse), iters=3, pool=2)
            rec("cross_entropy bwd 8192x32064", ms, best, nbytes=2 * M * V * 2)
        cuda_impl.check_status()
        return
    shapes = [(M, 4096, 4096), (M, 14336, 4096), (M, 4096, 14336), (M, 1024, 4096)]
    if not args.quick:
        shapes.append((M, 128256, 4096))
    for (m, n, k) in ([] if args.skip_gemm else shapes):
        for tag, ta, tb in (("nt", False, True), ("nn", False, False), ("tn", True, False)):
            if tag == "tn":
                mk = lambda: (torch.randn(k, m, device=dev, dtype=bf), torch.randn(k, n, device=dev, dtype=bf))
            elif tag == "nn":
                mk = lambda: (torch.randn(m, k, device=dev, dtype=bf), torch.randn(k, n, device=dev, dtype=bf))
            else:
                mk = lambda: (torch.randn(m, k, device=dev, dtype=bf), torch.randn(n, k, device=dev, dtype=bf))
            ms, best = time_fn(mk, lambda a, b: L.ops.gemm(a, b, ta, tb, bf), pool=3)
            rec(f"gemm_{tag} {m}x{n}x{k}", ms, best, flops=2.0 * m * n * k)
            if tag == "nt":
                ms, best = time_fn(mk, lambda a, b: torch.matmul(a, b.t()), pool=3)
                rec(f"  cublas_nt {m}x{n}x{k}", ms, best, flops=2.0 * m * n * k)
    cuda_impl.check_status()
    if args.gemm_only:
        return
    D = 4096
    mk = lambda: (torch.randn(M, D, device=dev, dtype=bf), torch.randn(D, device=dev, dtype=bf))
    ms, best = time_fn(mk, lambda x, w: L.ops.rms_norm(x, w, 1e-5), pool=8)
    rec("rms_norm fwd 8192x4096", ms, best, nbytes=2 * M * D * 2)
    mk = lambda: (torch.randn(M, D, device=dev, dtype=bf), torch.randn(M, D, device=dev, dtype=bf), torch.randn(D, device=dev, dtype=bf), torch.rand(M, device=dev))
    ms, best = time_fn(mk, lambda dy, x, w, r: L.ops.rms_norm_bwd(dy, x, w, r), pool=8)
    rec("rms_norm bwd 8192x4096", ms, best, nbytes=3 * M * D * 2)
    H = 14336
    mk = lambda: (torch.randn(M, H, device=dev, dtype=bf), torch.randn(M, H, device=dev, dtype=bf))
    ms, best = time_fn(mk, lambda a, b: L.ops.swiglu(a, b), pool=4)
    rec("swiglu fwd 8192x14336", ms, best, nbytes=3 * M * H * 2)
    mk = lambda: (torch.randn(M, H, device=dev, dtype=bf), torch.randn(M, H, device=dev, dtype=bf), torch.randn(M, H, device=dev, dtype=bf))
    ms, best = time_fn(mk, lambda g, a, b: L.ops.swiglu_bwd(g, a, b), pool=4)
    rec("swiglu bwd 8192x14336", ms, best, nbytes=5 * M * H * 2)
    ang = torch.randn(M, 64, device=dev)
    cs, sn = ang.cos(), ang.sin()
    mk = lambda: (torch.randn(1, M, 32, 128, device=dev, dtype=bf),)
    ms, best = time_fn(mk, lambda x: L.ops.rope(x, cs, sn, False), pool=8)
    rec("rope 1x8192x32x128", ms, best, nbytes=2 * M * 4096 * 2)
    if not args.quick:
        V = 128256
        mk = lambda: (torch.randn(M, V, device=dev, dtype=bf), torch.randint(0, V, (M,), device=dev))
        ms, best = time_fn(mk, lambda lg, lb: L.ops.cross_entropy(lg, lb), pool=2)
        rec("cross_entropy fwd 8192x128256", ms, best, nbytes=M * V * 2)
    # cross-entropy backward, casts, embedding, multi-tensor AdamW, grouped expert GEMM
    V2 = 32064
    mk = lambda: (torch.randn(M, device=dev), torch.randn(M, V2, device=dev, dtype=bf), torch.randint(0, V2, (M,), device=dev), torch.rand(M, device=dev) + 10)
    ms, best = time_fn(mk, lambda g, lg, lb, lse: L.ops.cross_entropy_bwd(g, lg, lb, lse), pool=4)
    rec("cross_entropy bwd 8192x32064", ms, best, nbytes=2 * M * V2 * 2)
    mk = lambda: (torch.randn(M, H, device=dev),)
    ms, best = time_fn(mk, lambda x: L.ops.dtype_cast(x, bf), pool=3)
    rec("cast fp32->bf16 8192x14336", ms, best, nbytes=M * H * 6)
    mk = lambda: (torch.randn(M, H, device=dev, dtype=bf),)
    ms, best = time_fn(mk, lambda x: L.ops.dtype_cast(x, torch.float32), pool=3)
    rec("cast bf16->fp32 8192x14336", ms, best, nbytes=M * H * 6)
    tab = torch.randn(128256, D, device=dev, dtype=bf)
    mk = lambda: (torch.randint(0, 128256, (1, M), device=dev),)
    ms, best = time_fn(mk, lambda ids: L.ops.embedding(tab, ids), pool=4)
    rec("embedding fwd 8192 of 128256x4096", ms, best, nbytes=2 * M * D * 2)
    from autoparallel_b200.optim import AdamW

    ps = [torch.nn.Parameter(torch.randn(H, D, device=dev)) for _ in range(4)]
    for p_ in ps:
        p_.grad = torch.randn_like(p_)
    opt = AdamW(ps, lr=1e-3, emit_bf16=True)
    opt.step()  # state and tables exist before timing
    opt.prepare_capture()
    ms, best = time_fn(lambda: (), lambda: opt.step(), pool=2)
    rec("adamw 4 x 14336x4096 fp32 (+bf16 copy)", ms, best, nbytes=4 * H * D * (16 + 12 + 2))
    if not args.quick:
        E, Me, Ne, Ke = 8, 8192, 1408, 2048
        mk = lambda: (torch.randn(E, Me, Ke, device=dev, dtype=bf) * 0.05, torch.randn(E, Ke, Ne, device=dev, dtype=bf) * 0.05)
        ms, best = time_fn(mk, lambda a, b: torch.ops.apb200.grouped_mm(a, b, False, bf), pool=3)
        rec(f"grouped_mm {E}x{Me}x{Ne}x{Ke}", ms, best, flops=2.0 * E * Me * Ne * Ke)
    mk = lambda: (torch.randn(1, M, 32, 128, device=dev, dtype=bf), torch.randn(1, M, 8, 128, device=dev, dtype=bf), torch.randn(1, M, 8, 128, device=dev, dtype=bf))
    ms, best = time_fn(mk, lambda q, k, v: L.ops.attention(q, k, v, True, 128 ** -0.5), pool=2)
    rec("attention fwd causal 8192 32q/8kv (library kernel unless APB200_ATTENTION_FWD=own)", ms, best, flops=4.0 * M * M * 4096 * 0.5)
    if args.json:
        json.dump({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf_burst, "bf16_tflops_sustained": tf_sus, "source": src}, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
