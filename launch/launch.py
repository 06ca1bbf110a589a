"""Single-node launcher and sweep runner.

    python launch/launch.py bench --gpus 8 -- --steps 10 --warmup 3
    python launch/launch.py sweep --gpus 1,2,4,8 --out results.jsonl

``bench`` starts ``bench.py`` under ``torch.distributed.run`` on 127.0.0.1 with one rank per GPU
(retries on failure, NCCL debug level and extra environment settable); ``sweep`` runs a list of
configurations (GPU counts × executors × communication back-ends × implementation arms) and
appends each JSON result line to a file.  The reference ships a cluster launcher for Meta's
internal scheduler plus TorchTitan sweep definitions (mast/mast.py, mast/sweep.py); this is the
equivalent for one NVSwitch box.
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import socket
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_bench(gpus: int, extra: list[str], env: dict | None = None, retries: int = 0, timeout: int = 3600) -> dict | None:
    cmd = [sys.executable]
    if gpus > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
                "--master-port", str(free_port())]
    cmd += [os.path.join(ROOT, "bench.py"), "--gpus", str(gpus), *extra]
    e = dict(os.environ, **(env or {}))
    for attempt in range(retries + 1):
        r = subprocess.run(cmd, capture_output=True, text=True, env=e, timeout=timeout)
        line = next((l for l in reversed(r.stdout.splitlines()) if l.startswith("{")), None)
        if r.returncode == 0 and line:
            return json.loads(line)
        sys.stderr.write(f"attempt {attempt + 1} failed (rc={r.returncode}):\n{r.stderr[-2000:]}\n")
        time.sleep(2)
    return None


SWEEP = {
    "executor": ["graph", "streams"],
    "comm": ["nccl", "symm"],
    "impl": ["ours", "reference"],
}


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    b = sub.add_parser("bench")
    b.add_argument("--gpus", type=int, default=1)
    b.add_argument("--retries", type=int, default=0)
    b.add_argument("--nccl-debug", default=None)
    b.add_argument("rest", nargs=argparse.REMAINDER)
    s = sub.add_parser("sweep")
    s.add_argument("--gpus", default="1,2,4,8")
    s.add_argument("--out", default="sweep.jsonl")
    s.add_argument("--steps", type=int, default=5)
    s.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    if a.cmd == "bench":
        extra = [x for x in a.rest if x != "--"]
        env = {"NCCL_DEBUG": a.nccl_debug} if a.nccl_debug else None
        res = run_bench(a.gpus, extra, env, a.retries)
        print(json.dumps(res))
        sys.exit(0 if res else 1)
    with open(a.out, "a") as f:
        for n in [int(x) for x in a.gpus.split(",")]:
            for ex, comm, impl in itertools.product(SWEEP["executor"], SWEEP["comm"], SWEEP["impl"]):
                if impl == "reference" and (ex, comm) != ("graph", "nccl"):
                    continue
                if n == 1 and comm == "symm":
                    continue
                extra = ["--steps", str(a.steps), "--warmup", str(a.warmup), "--impl", impl]
                if impl == "ours":
                    extra += ["--executor", ex, "--comm", comm]
                res = run_bench(n, extra)
                f.write(json.dumps({"gpus": n, "executor": ex, "comm": comm, "impl": impl, "result": res}) + "\n")
                f.flush()


if __name__ == "__main__":
    main()
