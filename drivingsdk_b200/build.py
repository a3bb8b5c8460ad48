"""In-tree build of the native pieces (run by ``__graft_entry__.build()``).

    drivingsdk_b200/libmsda_sm100.so   the C-ABI library: hand-written CUDA for sm_100a
    drivingsdk_b200/libmsda_sm100_dbg.so  the same sources with -DMSDA_DEBUG_BOUNDS: every row
                                       offset the MSDA kernels compute is checked before use
                                       (what the tests run in place of a memory checker)
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
DEBUG_LIB = os.path.join(PKG, "libmsda_sm100_dbg.so")
EXT = os.path.join(PKG, "_C.so")

CUDA_SOURCES = ["msda_capi.cu", "msda_fwd_sm100.cu", "msda_bwd_sm100.cu", "gka_fwd_sm100.cu",
                "gka_bwd_sm100.cu", "msda_fused_fwd_sm100.cu", "msda_fused_bwd_sm100.cu", "da_sm100.cu",
                "msda_static_scratch.cu", "hw_probe_sm100.cu", "resnet_ops_sm100.cu", "dcn_sm100.cu",
                "gemm_simt_sm100.cu", "gemm_tc_sm100.cu"]
CUDA_HEADERS = ["msda_common.cuh", "msda_tile.cuh", "msda_launch.h", "msda_fwd_kernel.cuh",
                "msda_bwd_kernel.cuh", "gemm_sm100.h"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]
OBJ_DIR = os.path.join(PKG, "build")


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


def build_library(force=False, verbose_ptxas=False, debug_bounds=False) -> str:
    """nvcc each .cu to an object (in parallel: the kernel files hold many template
    instantiations), then link the shared library. ``debug_bounds`` builds the
    bounds-checking variant next to the normal one."""
    from concurrent.futures import ThreadPoolExecutor
    target = DEBUG_LIB if debug_bounds else LIB
    obj_dir = OBJ_DIR + ("_dbg" if debug_bounds else "")
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in CUDA_HEADERS] + [
        os.path.join(ROOT, "include", "msda_sm100.h"),
        os.path.join(ROOT, "include", "conv_ops_sm100.h")]
    if not (force or _stale(target, deps)):
        return target
    os.makedirs(obj_dir, exist_ok=True)
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose_ptxas else []) + (
        ["-DMSDA_DEBUG_BOUNDS"] if debug_bounds else [])
    objs = [os.path.join(obj_dir, os.path.basename(s)[:-3] + ".o") for s in srcs]

    def compile_one(pair):
        src, obj = pair
        return _run([_nvcc()] + flags + ["-c", src, "-o", obj], "nvcc -c " + os.path.basename(src))

    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 1)) as pool:
        logs = list(pool.map(compile_one, zip(srcs, objs)))
    if verbose_ptxas:
        sys.stdout.write("".join(logs))
    _run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared"] + objs + ["-o", target],
         "nvcc link")
    return target


def build_extension(force=False) -> str:
    src = os.path.join(CSRC, "binding.cpp")
    deps = [src, os.path.join(ROOT, "include", "msda_sm100.h"),
            os.path.join(ROOT, "include", "conv_ops_sm100.h"), LIB]
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
    return (build_library(force), build_library(force, debug_bounds=True),
            build_extension(force))


if __name__ == "__main__":
    force = "--force" in sys.argv
    lib = build_library(force, verbose_ptxas="--ptxas" in sys.argv)
    dbg = build_library(force, debug_bounds=True)
    ext = build_extension(force)
    print(lib)
    print(dbg)
    print(ext)
