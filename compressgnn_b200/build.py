"""In-tree build of the native libraries (no JIT cache, no torch headers).

``libcgnn_b200.so``   -- the sm_100a CUDA kernels behind the C ABI of ``include/cgnn_b200.h``
                         (``csrc/*.cu``, compiled by nvcc, one object per file, in parallel).
``libcgnn_host.so``   -- host-side graph preparation (``host/*.cpp``, g++ with OpenMP), when
                         its sources exist.

Objects are rebuilt only when their source or a header is newer.  ``python -m
compressgnn_b200.build`` builds everything.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
HOST = PKG / "host"
OBJ = PKG / "_build"
CUDA_LIB = PKG / "libcgnn_b200.so"
HOST_LIB = PKG / "libcgnn_host.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = Path(cuda_home) / "bin" / "nvcc"
    return str(exe) if exe.is_file() else "nvcc"


def _stale(target, deps):
    if not target.is_file():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print("[build]", " ".join(cmd), flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: {}\n{}".format(" ".join(cmd), proc.stdout))
    return proc.stdout


def build_cuda(verbose=False, ptxas_info=False):
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libcgnn_b200.so``."""
    OBJ.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + \
        sorted((PKG.parent / "include").glob("*.h"))
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if _stale(obj, [src] + headers):
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + \
                ["-c", str(src), "-o", str(obj)]
            jobs.append(cmd)
    logs = []
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            logs = list(pool.map(lambda c: _run(c, verbose), jobs))
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if jobs or _stale(CUDA_LIB, objs):
        _run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o",
              str(CUDA_LIB)] + [str(o) for o in objs], verbose)
    return CUDA_LIB, logs


def build_host(verbose=False):
    """Compile ``host/*.cpp`` into ``libcgnn_host.so`` (g++ -O3 -fopenmp)."""
    sources = sorted(HOST.glob("*.cpp")) if HOST.is_dir() else []
    if not sources:
        return None
    headers = sorted(HOST.glob("*.h")) + sorted(HOST.glob("*.hpp"))
    if _stale(HOST_LIB, sources + headers):
        _run(["g++", "-O3", "-std=c++17", "-fopenmp", "-shared", "-fPIC",
              "-o", str(HOST_LIB)] + [str(s) for s in sources], verbose)
    return HOST_LIB


def build_all(verbose=False):
    lib, _ = build_cuda(verbose)
    return lib, build_host(verbose)


if __name__ == "__main__":
    out = build_cuda(verbose=True, ptxas_info="--ptxas" in sys.argv)
    if "--ptxas" in sys.argv:
        print("\n".join(out[1]))
    print(out[0])
    print(build_host(verbose=True))
