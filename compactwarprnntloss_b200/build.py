"""In-tree build of the native parts: the C-ABI CUDA library and the torch extension module.

    python -m compactwarprnntloss_b200.build [--force] [--no-ext]

libcwarp_rnnt_b200.so  nvcc, sm_100a only, no torch dependency; exports include/cwarp_rnnt_b200.h
_C.*.so                the thin C++ torch binding (cwarp_rnnt._C replacement), linked against the library above
Both land next to this file so they travel with the source tree; nothing is installed into site-packages.
"""
import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INC = os.path.join(ROOT, "include")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libcwarp_rnnt_b200.so")

CU_SOURCES = ["cwrnnt_prep.cu", "cwrnnt_gather.cu", "cwrnnt_wavefront.cu", "cwrnnt_grad.cu", "cwrnnt_compat.cu",
              "cwrnnt_pack.cu", "cwrnnt_joint.cu", "cwrnnt_align.cu", "cwrnnt_api.cu", "cwrnnt_host.cu", "cwrnnt_static.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", INC, "-I", CSRC]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.isfile(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target, deps):
    if not os.path.isfile(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hs += [os.path.join(INC, f) for f in os.listdir(INC)]
    return hs


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = _headers()
    sources = [s for s in CU_SOURCES if os.path.isfile(os.path.join(CSRC, s))]
    jobs = []
    for s in sources:
        src, obj = os.path.join(CSRC, s), os.path.join(OBJ, s[:-3] + ".o")
        if force or _newer(obj, [src] + headers):
            jobs.append([_nvcc()] + NVCC_FLAGS + ["-c", src, "-o", obj])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for cmd, res in zip(jobs, ex.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs)):
                if verbose or res.returncode:
                    sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
                if res.returncode:
                    raise RuntimeError("nvcc failed: " + cmd[-3])
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in sources]
    if force or jobs or _newer(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-cudart", "shared", "-Xlinker", "--no-undefined"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB


def ext_path() -> str:
    return os.path.join(PKG, "_C" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_extension(force: bool = False, verbose: bool = False) -> str:
    """g++ build of the pybind/torch binding against libtorch and the C-ABI library (rpath $ORIGIN)."""
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths
    src = os.path.join(CSRC, "torch_binding.cpp")
    out = ext_path()
    if not force and not _newer(out, [src, LIB] + _headers()):
        return out
    cxx = os.environ.get("CXX", "g++")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-DTORCH_EXTENSION_NAME=_C",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for p in include_paths("cuda"):
        cmd += ["-isystem", p]
    cmd += ["-isystem", sysconfig.get_paths()["include"], "-I", INC, src, "-o", out]
    for p in library_paths("cuda"):
        cmd += ["-L", p, "-Wl,-rpath," + p]
    cmd += ["-L", PKG, "-l:libcwarp_rnnt_b200.so", "-Wl,-rpath,$ORIGIN",
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("torch binding build failed")
    return out


def build_all(force: bool = False, verbose: bool = False, ext: bool = True):
    lib = build_library(force, verbose)
    mod = build_extension(force, verbose) if ext and os.path.isfile(os.path.join(CSRC, "torch_binding.cpp")) else None
    return lib, mod


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv, ext="--no-ext" not in sys.argv))
