"""In-tree build of the native pieces (run by ``__graft_entry__.build()``).

    drivingsdk_b200/libmsda_sm100.so   the C-ABI library: hand-written CUDA for sm_100a
    drivingsdk_b200/_C.so              the torch extension that calls it

Both are plain ``nvcc`` / ``g++`` command lines so the result sits next to the
sources and travels with the tree. ``python -m drivingsdk_b200.build`` rebuilds
what is stale; ``--force`` rebuilds everything.
"""
import os
import shutil
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libmsda_sm100.so")
EXT = os.path.join(PKG, "_C.so")

CUDA_SOURCES = ["msda_capi.cu", "msda_fwd_sm100.cu", "msda_bwd_sm100.cu",
                "msda_static_scratch.cu"]
CUDA_HEADERS = ["msda_common.cuh", "msda_tile.cuh", "msda_launch.h"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def _stale(target, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, log_name):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError(f"build step failed ({log_name}): {' '.join(cmd)}")
    return proc.stdout


def build_library(force=False, verbose_ptxas=False) -> str:
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in CUDA_HEADERS] + [
        os.path.join(ROOT, "include", "msda_sm100.h")]
    if force or _stale(LIB, deps):
        flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose_ptxas else [])
        out = _run([_nvcc()] + flags + srcs + ["-o", LIB], "nvcc")
        if verbose_ptxas:
            sys.stdout.write(out)
    return LIB


def build_extension(force=False) -> str:
    src = os.path.join(CSRC, "binding.cpp")
    deps = [src, os.path.join(ROOT, "include", "msda_sm100.h"), LIB]
    if not (force or _stale(EXT, deps)):
        return EXT
    import torch
    from torch.utils import cpp_extension

    inc = []
    for p in cpp_extension.include_paths(device_type="cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_lib = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = (["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
            "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={abi}"] + inc + [src, "-o", EXT,
            f"-L{PKG}", "-lmsda_sm100", f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch", "-ltorch_python", f"-L{cuda_lib}", "-lcudart",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{cuda_lib}"])
    _run(cmd, "g++ binding")
    return EXT


def build_all(force=False):
    return build_library(force), build_extension(force)


if __name__ == "__main__":
    force = "--force" in sys.argv
    lib = build_library(force, verbose_ptxas="--ptxas" in sys.argv)
    ext = build_extension(force)
    print(lib)
    print(ext)
