"""In-tree build of the native pieces for sm_100a.

``build_native()`` compiles ``csrc/*.cu`` with nvcc into ``libflashquant_b200.so`` (the
C-ABI library, no torch dependency) next to this file.  ``build_pybind()`` compiles the
pybind11 module ``_C`` (torch tensors in, C ABI underneath) with the same nvcc.  Both skip
the work when the outputs are newer than every source.

    python -m flashquant_b200.build            # build both
    python -m flashquant_b200.build --verbose  # also print ptxas resource usage
"""

from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
BUILD = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "libflashquant_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", INCLUDE]

KERNEL_SOURCES = ["capi.cu", "compress.cu", "decompress.cu", "paged_decode.cu", "prefill.cu",
                  "rotate.cu", "host_step.cu", "cache_update.cu",
                  "decode_multi.cu", "packing.cu"]


def _sources():
    return [s for s in KERNEL_SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _newest_input() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    paths += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    paths.append(os.path.abspath(__file__))
    return max(os.path.getmtime(p) for p in paths)


def _run(cmd, verbose):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    if verbose:
        sys.stderr.write(r.stdout + r.stderr)


def build_native(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_input():
        return LIB
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src):
        obj = os.path.join(BUILD, src.replace(".cu", ".o"))
        _run([NVCC, *ARCH, *COMMON, *extra, "-c", os.path.join(CSRC, src), "-o", obj], verbose)
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, _sources()))
    _run([NVCC, *ARCH, "-shared", "-o", LIB, *objs, "-lcudart"], verbose)
    return LIB


def pybind_path() -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(HERE, "_C" + suffix)


def build_pybind(verbose: bool = False, force: bool = False) -> str:
    """Compile the pybind11 module ``flashquant_b200._C`` (needs torch headers)."""
    out = pybind_path()
    src = os.path.join(CSRC, "pybind_module.cpp")
    if not os.path.exists(src):
        raise RuntimeError("pybind_module.cpp is missing")
    build_native(verbose=verbose, force=force)
    if not force and os.path.exists(out) and os.path.getmtime(out) >= max(
            _newest_input(), os.path.getmtime(LIB)):
        return out
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths():
        inc += ["-I", p]
    inc += ["-I", sysconfig.get_paths()["include"], "-I", "/usr/local/cuda/include"]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=_C",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           "-I", INCLUDE, *inc, src, "-o", out,
           "-L", HERE, "-l:libflashquant_b200.so", "-Wl,-rpath,$ORIGIN",
           "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10", "-ltorch_cuda",
           "-lc10_cuda", "-L", "/usr/local/cuda/lib64", "-lcudart",
           f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, verbose)
    return out


if __name__ == "__main__":
    v = "--verbose" in sys.argv
    f = "--force" in sys.argv
    print(build_native(verbose=v, force=f))
    if os.path.exists(os.path.join(CSRC, "pybind_module.cpp")):
        print(build_pybind(verbose=v, force=f))
