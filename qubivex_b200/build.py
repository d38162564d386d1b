"""Builds libqvx_cuda.so (sm_100a) in-tree with nvcc.  `python -m qubivex_b200.build`.

Each source is compiled to an object under build/ and the objects are linked into
qubivex_b200/lib/libqvx_cuda.so with the static CUDA runtime, so the library has no
dependency the GPU box could miss.  Only attn_exact.cu is built with -fmad=false: its
arithmetic must keep the reference's operation order (no contraction).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
# The shipped library, and the experiment build of the same sources (-DQVX_EXPERIMENTS: the chunk and
# run-length rules and the bf16 remainder pass can be changed through the environment; the tests that
# show which of those move no bit, and the profiling drivers, load it).
LIB = PKG / "lib" / "libqvx_cuda.so"
LIB_EXPERIMENTS = PKG / "lib" / "libqvx_cuda_experiments.so"
# A test build: bounded waits of a few thousand polls and a hook that loses one publication, so that a
# test can watch a wait run out and the device recover (tests/test_gpu_guards.py).
LIB_SHORT_WAITS = PKG / "lib" / "libqvx_cuda_shortwaits.so"
# QVX_LIB / QVX_NVCC_EXTRA build one more variant (kernel experiments) and make it the library loaded.
if os.environ.get("QVX_LIB"):
    LIB = Path(os.environ["QVX_LIB"]).resolve()
EXTRA = os.environ.get("QVX_NVCC_EXTRA", "").split()

LINK: list[str] = ["-ldl"]  # NCCL is bound at run time (comm.cu)
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]
SOURCES = {
    "qvx_api.cu": [],
    "kv_rows.cu": [],
    "block_copy.cu": [],
    "attn_stream.cu": [],
    "attn_static.cu": [],
    "attn_exact.cu": ["-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false"],
    "attn_prelude.cu": ["-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false"],
    "comm.cu": [],
    "runtime.cpp": [],
}


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA backend cannot be built")
    return exe


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, experiments: bool = False, short_waits: bool = False) -> Path:
    """Compiles what is stale and links the library; `experiments` builds libqvx_cuda_experiments.so,
    `short_waits` libqvx_cuda_shortwaits.so."""
    lib = LIB_SHORT_WAITS if short_waits else LIB_EXPERIMENTS if experiments else LIB
    extra_flags = (["-DQVX_TEST_HOOKS", "-DQVX_WAIT_LIMIT=4096"] if short_waits else ["-DQVX_EXPERIMENTS"] if experiments else EXTRA)
    obj_dir = ROOT / "build" / ("obj-" + lib.stem)
    obj_dir.mkdir(parents=True, exist_ok=True)
    lib.parent.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + [ROOT / "include" / "qvx.h", Path(__file__)]
    jobs = []
    for name, extra in SOURCES.items():
        src = CSRC / name
        obj = obj_dir / (name.rsplit(".", 1)[0] + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc(), *ARCH, *COMMON, *extra, *extra_flags]
            if verbose:
                cmd += ["-Xptxas", "-v"]
            cmd += ["-c", str(src), "-o", str(obj)]
            jobs.append((name, cmd))

    def run(job):
        name, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return name, r

    with ThreadPoolExecutor(max_workers=min(6, max(1, len(jobs)))) as ex:
        for name, r in ex.map(run, jobs):
            if verbose or r.returncode:
                sys.stderr.write(f"--- {name}\n{r.stdout}{r.stderr}")
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {name}")
    objs = [obj_dir / (n.rsplit(".", 1)[0] + ".o") for n in SOURCES]
    if force or jobs or _stale(lib, objs):
        cmd = [nvcc(), *ARCH, "-shared", "-o", str(lib), *map(str, objs), "-cudart", "static", *LINK]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return lib


if __name__ == "__main__":
    for kw in ({}, {"experiments": True}, {"short_waits": True}):
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, **kw))
