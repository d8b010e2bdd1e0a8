"""Builds the native code in-tree for sm_100a.

``python torchex_b200/build.py`` (run as a script: importing the package needs the
libraries this builds) writes

* ``torchex_b200/lib/libtexb_scatter.so`` -- the kernels behind the plain C ABI of
  ``include/texb_scatter.h`` (nvcc; no torch dependency), and
* ``torchex_b200/lib/scatter_ext*.so`` -- the torch extension module ``scatter_ext``
  (g++ against the installed torch; ``csrc/scatter_ext_binding.cpp``), which binds that
  C ABI to tensors the way TorchEx's own ``scatter_ext`` does.

Each ``.cu`` file is compiled to its own object (in parallel, and only when it or a
header changed), then the objects are linked.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
# TEXB_LIB_DIR: another directory to build into and load from (for trying out a build with
# different -D options beside the regular one); TEXB_NVCC_EXTRA: extra nvcc options for it.
LIB_DIR = os.environ.get("TEXB_LIB_DIR") or os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libtexb_scatter.so")
HEADER = os.path.join(os.path.dirname(PKG_DIR), "include", "texb_scatter.h")
SOURCES = ["abi.cu", "segment_reduce.cu", "reduce_unit_sum.cu", "reduce_unit_sum_plain.cu", "reduce_unit_max.cu",
           "reduce_unit_sum_max.cu", "segment_small.cu", "segment_plan.cu", "segment_backward.cu", "peer_copy.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
EXT_NAME = "scatter_ext"
EXT_SOURCE = os.path.join(CSRC, "scatter_ext_binding.cpp")
EXT_PATH = os.path.join(LIB_DIR, EXT_NAME + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return nvcc


def _headers():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + [HEADER]


def _newer(target: str, deps) -> bool:
    """True when ``target`` is missing or older than one of ``deps``."""
    if not os.path.exists(target):
        return True
    built = os.path.getmtime(target)
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def is_stale() -> bool:
    deps = [os.path.join(CSRC, s) for s in SOURCES] + _headers()
    return _newer(LIB_PATH, deps)


def _run(cmd, what):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"{what} failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return proc.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every .cu file into one shared library; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = find_nvcc()
    headers = _headers()
    jobs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
        if force or _newer(obj, [path] + headers):
            cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("TEXB_NVCC_EXTRA", "").split(),
                   *(["-Xptxas", "-v"] if verbose else []), "-c", "-o", obj, path]
            jobs.append((cmd, src))
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        for log in pool.map(lambda j: _run(j[0], "nvcc " + j[1]), jobs):
            if verbose:
                sys.stderr.write(log)
    objs = [os.path.join(OBJ_DIR, s[:-3] + ".o") for s in SOURCES]
    _run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs], "link")
    return LIB_PATH


def extension_is_stale() -> bool:
    # the module links the library dynamically: only its own source and the ABI header matter
    return _newer(EXT_PATH, [EXT_SOURCE, HEADER])


def build_extension(force: bool = False) -> str:
    """Compiles the torch extension module ``scatter_ext`` and links it against the
    C-ABI library beside it (found at run time through an ``$ORIGIN`` rpath)."""
    build(force=False)
    if not force and not extension_is_stale():
        return EXT_PATH
    import torch
    from torch.utils import cpp_extension as ce
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = ce.CUDA_HOME or "/usr/local/cuda"
    cmd = [shutil.which("g++") or "g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}"]
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include"),
                                     os.path.dirname(HEADER)]:
        cmd += ["-isystem", inc]
    cmd += [EXT_SOURCE, "-o", EXT_PATH, f"-L{torch_lib}", f"-L{LIB_DIR}", "-ltexb_scatter",
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, "g++ scatter_ext")
    return EXT_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_extension(force="--force" in sys.argv))
