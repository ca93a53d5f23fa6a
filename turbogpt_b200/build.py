"""Builds libturbogpt_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libturbogpt_b200.so"
SOURCES = ["host.cpp", "checkpoint.cpp", "elementwise.cu", "attention_simt.cu", "gemm_simt.cu", "gemm_tc.cu", "attention_tc.cu", "attention_bwd_fused.cu", "optim.cu",
           "selftest.cu", "engine.cu", "runtime.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default", "--expt-relaxed-constexpr"]


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build_library(verbose: bool = False, ptxas_info: bool = False) -> Path:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objdir = PACKAGE / "build"
    objdir.mkdir(exist_ok=True)
    headers = [*CSRC.glob("*.h"), *CSRC.glob("*.cuh"), PACKAGE.parent / "include" / "turbogpt_b200.h"]

    def compile_one(name: str):
        src, obj = CSRC / name, objdir / (name + ".o")
        if not _stale(obj, [src, *headers]) and not ptxas_info:
            return obj, ""
        cmd = [nvcc, *FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd += ["-Xptxas", "-v"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"nvcc failed for {name}:\n{r.stdout}\n{r.stderr}")
        return obj, r.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    objects = [str(o) for o, _ in results]
    if verbose or ptxas_info:
        for _, log in results:
            if log:
                print(log, file=sys.stderr)
    if _stale(LIBRARY, objects):
        staged = LIBRARY.with_name(LIBRARY.name + ".staged")  # linked aside, then moved into place in one step
        cmd = [nvcc, "-shared", "-o", str(staged), *objects, "-lcudart", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(staged, LIBRARY)
    return LIBRARY


HOST = PACKAGE / "turbogpt_dp"


def build_host() -> Path:
    """The data-parallel training host (host/train_dp.cpp) over the C ABI of the library."""
    source = PACKAGE / "host" / "train_dp.cpp"
    if _stale(HOST, [source, PACKAGE.parent / "include" / "turbogpt_b200.h", LIBRARY]):
        staged = HOST.with_name(HOST.name + ".staged")
        cmd = ["g++", "-O2", "-std=c++17", "-pthread", str(source), f"-L{PACKAGE}", "-lturbogpt_b200",
               "-Wl,-rpath,$ORIGIN", "-o", str(staged)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"host build failed:\n{r.stdout}\n{r.stderr}")
        os.replace(staged, HOST)
    return HOST


if __name__ == "__main__":
    print(build_library(verbose=True, ptxas_info="--ptxas" in sys.argv))
    print(build_host())
