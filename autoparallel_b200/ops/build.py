"""In-tree build of the sm_100a extension (``autoparallel_b200/ops/_C*.so``).

``nvcc`` compiles each ``.cu`` for ``sm_100a`` only (no torch headers in device code, so this
takes seconds and cross-compiles on machines without a GPU); the pybind translation unit is
compiled with the host compiler against torch's headers; everything is linked into one shared
object that sits next to this file, so a source snapshot carries the built kernels with it.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_build")
NAME = "_C"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def so_path() -> str:
    return os.path.join(HERE, NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def _sources():
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    hdr = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    return cu, cpp, hdr


def _digest() -> str:
    h = hashlib.sha256()
    cu, cpp, hdr = _sources()
    for f in cu + cpp + hdr:
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    stamp = os.path.join(OBJ, "stamp")
    return os.path.exists(so_path()) and os.path.exists(stamp) and open(stamp).read() == _digest()


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and is_current():
        return so_path()
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OBJ, exist_ok=True)
    cu, cpp, _ = _sources()
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", f"-I{cuda_inc}"]
    jobs = []
    for f in cu:
        out = os.path.join(OBJ, f + ".o")
        extra = ["-Xptxas", "-v"] if verbose else []
        jobs.append(([nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, f), "-o", out], out))
    cxx = os.environ.get("CXX", "g++")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for f in cpp:
        out = os.path.join(OBJ, f + ".o")
        jobs.append((
            [cxx, "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-DTORCH_EXTENSION_NAME={NAME}",
             "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, "-c", os.path.join(CSRC, f), "-o", out],
            out,
        ))

    def run(job):
        cmd, out = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return out

    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        objs = list(ex.map(run, jobs))
    libdirs = ce.library_paths(device_type="cuda")
    link = [cxx, "-shared", *objs, "-o", so_path()]
    for d in libdirs:
        link += [f"-L{d}", f"-Wl,-rpath,{d}"]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed: {' '.join(link)}\n{r.stderr}")
    with open(os.path.join(OBJ, "stamp"), "w") as f:
        f.write(_digest())
    return so_path()


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
