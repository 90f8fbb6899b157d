"""Build the reference's own CPU code into ``oracle/_ref/`` (test infrastructure only).

Nothing here is product code.  The script compiles, with plain ``g++`` command lines and
*from the sources where they lie* in a checkout of ZhengChenCS/CompressGNN, two Python
extension modules:

``compressgnn_runtime``  (reference ``src/runtime/csrc``: ``function.cpp``,
    ``sparse/spmm.cpp``, ``sparse/cpu/spmm_cpu.cpp``, ``cluster/cluster.cpp``,
    ``cluster/cpu/cluster_cpu.cpp``) -- the CPU operators ``spmm_func`` and
    ``cluster_forward`` that the parity tests and the bench's CPU baseline call.

``compressgnn_offline``  (reference ``src/offline/csrc/function.cpp`` + ``Gorder/*.cpp``)
    -- graph preparation helpers (``filter_csr``, ``depth_filter_csr``,
    ``hybird_partition``, ``topo_partition``, norms, ...).  The reference's grammar
    compressor lives in an un-vendored git submodule, so ``bind_batch_cpu`` is satisfied
    by the no-op stub ``ref_offline_stub.cpp`` next to this file.  ``-DNDEBUG`` is needed
    because ``gen_mask.h:240`` carries an assert that can never hold.

The outputs are git-ignored shared objects; no reference source is copied.  When the
reference checkout is absent (the GPU box) the script does nothing and the prebuilt files
that travelled with the tree are used.
"""
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
# where the reference checkout is looked for: $CGNN_REFERENCE_DIR, else a directory named
# "reference" beside this repository
DEFAULT_REFERENCE = Path(os.environ.get("CGNN_REFERENCE_DIR") or HERE.parent.parent / "reference")


def _run(cmd):
    print("[oracle/_ref]", " ".join(str(c) for c in cmd), flush=True)
    subprocess.run([str(c) for c in cmd], check=True)


def _newer(target, sources):
    if not target.is_file():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def build_runtime(ref):
    import torch
    from torch.utils import cpp_extension

    csrc = ref / "src" / "runtime" / "csrc"
    sources = [csrc / "function.cpp", csrc / "sparse" / "spmm.cpp",
               csrc / "sparse" / "cpu" / "spmm_cpu.cpp", csrc / "cluster" / "cluster.cpp",
               csrc / "cluster" / "cpu" / "cluster_cpu.cpp"]
    target = OUT / "compressgnn_runtime.so"
    if _newer(target, sources):
        return target
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = ["g++", "-O3", "-fopenmp", "-std=c++17", "-shared", "-fPIC", "-Wl,-Bsymbolic",
           "-DTORCH_EXTENSION_NAME=compressgnn_runtime", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I", csrc, "-I", sysconfig.get_paths()["include"]]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += sources
    cmd += ["-L", torch_lib, f"-Wl,-rpath,{torch_lib}", "-lc10", "-ltorch", "-ltorch_cpu",
            "-ltorch_python", "-o", target]
    _run(cmd)
    return target


def build_runtime_cuda(ref):
    """The reference's runtime WITH its CUDA kernels (``-DWITH_CUDA``: ``sparse/cuda/spmm_gpu.cu``,
    ``cluster/cuda/cluster_kernel.cu`` next to the CPU files), compiled for sm_100 into
    ``oracle/_ref_cuda/compressgnn_runtime_cuda.so``.  A second checker and the GPU baseline of the
    benchmark's informational ``reference_cuda`` block; its kernels index with 32-bit products
    (``elist * col_num``, sparse/cuda/row_balance.cuh:82-128), so it is only ever run on inputs with
    rows * width below 2^31 and valid indices."""
    import torch
    from torch.utils import cpp_extension

    csrc = ref / "src" / "runtime" / "csrc"
    cpp = [csrc / "function.cpp", csrc / "sparse" / "spmm.cpp", csrc / "sparse" / "cpu" / "spmm_cpu.cpp",
           csrc / "cluster" / "cluster.cpp", csrc / "cluster" / "cpu" / "cluster_cpu.cpp"]
    cu = [csrc / "sparse" / "cuda" / "spmm_gpu.cu", csrc / "cluster" / "cuda" / "cluster_kernel.cu"]
    out_dir = HERE / "_ref_cuda"
    out_dir.mkdir(exist_ok=True)
    # its own module name, so that it can be imported beside the CPU build
    target = out_dir / "compressgnn_runtime_cuda.so"
    if _newer(target, cpp + cu):
        return target
    torch_lib = Path(torch.__file__).parent / "lib"
    defines = ["-DWITH_CUDA", "-DTORCH_EXTENSION_NAME=compressgnn_runtime_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    includes = ["-I", csrc, "-I", sysconfig.get_paths()["include"]]
    for inc in cpp_extension.include_paths(device_type="cuda"):
        includes += ["-isystem", inc]
    objects = []
    for src in cu:
        obj = out_dir / (src.stem + ".o")   # kept: compiling these against torch's headers takes minutes
        if not _newer(obj, [src]):
            _run(["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100,code=sm_100", "--expt-relaxed-constexpr",
                  "-DCUDA_HAS_FP16=1", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                  "-D__CUDA_NO_HALF2_OPERATORS__", "-Xcompiler", "-fPIC"] + defines + includes + ["-c", src, "-o", obj])
        objects.append(obj)
    cuda_lib = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "lib64"
    # -Bsymbolic: this module and the CPU build of the same sources may sit in one process; each must call
    # its own spmm_func / cluster_forward, not whichever was loaded first
    _run(["g++", "-O3", "-fopenmp", "-std=c++17", "-shared", "-fPIC", "-Wl,-Bsymbolic"] + defines + includes + cpp +
         objects + ["-L", torch_lib, f"-Wl,-rpath,{torch_lib}", "-L", cuda_lib, "-lc10", "-lc10_cuda", "-ltorch",
                    "-ltorch_cpu", "-ltorch_cuda", "-ltorch_python", "-lcudart", "-o", target])
    return target


def build_offline(ref):
    import pybind11

    csrc = ref / "src" / "offline" / "csrc"
    sources = [csrc / "function.cpp"] + sorted((csrc / "Gorder").glob("*.cpp"))
    sources.append(HERE / "ref_offline_stub.cpp")
    target = OUT / "compressgnn_offline.so"
    if _newer(target, sources):
        return target
    cmd = ["g++", "-O3", "-DNDEBUG", "-std=c++17", "-fopenmp", "-shared", "-fPIC", "-w",
           "-I", csrc, "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    cmd += sources + ["-o", target]
    _run(cmd)
    return target


def build_sample(ref):
    """The reference's host neighbour sampler (``src/sample/csrc``: one translation unit over torch's
    headers and the header-only hash map under ``third_party/parallel-hashmap``)."""
    import torch
    from torch.utils import cpp_extension

    csrc = ref / "src" / "sample" / "csrc"
    sources = [csrc / "function.cpp"]
    target = OUT / "compressgnn_sample.so"
    if _newer(target, sources + [csrc / "neighbor_sample.h", csrc / "storage_api.h"]):
        return target
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = ["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-w", "-Wl,-Bsymbolic",
           "-DTORCH_EXTENSION_NAME=compressgnn_sample", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I", csrc, "-I", sysconfig.get_paths()["include"]]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += sources
    cmd += ["-L", torch_lib, f"-Wl,-rpath,{torch_lib}", "-lc10", "-ltorch", "-ltorch_cpu",
            "-ltorch_python", "-o", target]
    _run(cmd)
    return target


def build(reference_dir=DEFAULT_REFERENCE, quiet=False, with_cuda=False):
    """Compile both modules when the reference checkout exists; return what is usable."""
    ref = Path(reference_dir)
    OUT.mkdir(exist_ok=True)
    if (ref / "src" / "runtime" / "csrc" / "function.cpp").is_file():
        build_runtime(ref)
        build_offline(ref)
        if (ref / "src" / "sample" / "csrc" / "function.cpp").is_file() and \
                (ref / "third_party" / "parallel-hashmap" / "parallel_hashmap" / "phmap.h").is_file():
            build_sample(ref)
        if with_cuda:
            build_runtime_cuda(ref)
    elif not quiet:
        print("[oracle/_ref] reference checkout not found; using prebuilt files if present")
    return {name: (OUT / f"{name}.so").is_file()
            for name in ("compressgnn_runtime", "compressgnn_offline", "compressgnn_sample")}


if __name__ == "__main__":
    paths = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(Path(paths[0]) if paths else DEFAULT_REFERENCE, with_cuda="--cuda" in sys.argv))
