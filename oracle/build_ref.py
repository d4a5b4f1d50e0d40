"""Build recipe for the GPU checker `oracle/_ref/`: the reference's own three source files, unmodified.

TEST INFRASTRUCTURE ONLY. Nothing of the product imports this file or its output.

The reference (maxwellzh/CompactWarpRNNTLoss) is a CUDA-only torch extension: `cwarp_cuda.cpp`,
`cwarp_cuda_gather_kernel.cu`, `cwarp_cuda_rnnt_kernel.cu`. Its own `setup.py` refuses to run without a
visible GPU (setup.py:15-16) and emits sm_60..sm_86 SASS only (setup.py:35-39), which cannot load on a
B200. This recipe therefore compiles the same three files *where they lie* in the mounted reference tree
with `-gencode arch=compute_100a,code=sm_100a` and writes only build products into `oracle/_ref/`
(git-ignored). No reference source is copied into the repository.

The result, `oracle/_ref/cwarp_rnnt_ref_C.so`, exports the reference's three pybind functions
(cwarp_cuda.cpp:138-153): `_cwarp_rnnt_forward`, `_cwarp_rnnt_backward`, `_cwarp_rnnt_loss`.
It is used (a) to generate the golden fixtures under `tests/golden/` on a B200 and (b) as a live GPU
comparator in the `-m gpu` tests and in `bench.py --impl reference_cuda` when the file is present.

Usage:  python oracle/build_ref.py <path-to-reference-tree>      (or CWRNNT_REFERENCE_ROOT=<path> in the environment)
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "cwarp_rnnt_ref_C"


def reference_root(arg=None):
    """Where the reference tree is mounted: the argument, else CWRNNT_REFERENCE_ROOT. There is no built-in default."""
    root = arg or os.environ.get("CWRNNT_REFERENCE_ROOT")
    if not root:
        raise FileNotFoundError("the reference tree's location is not known: pass it as the argument or set "
                                "CWRNNT_REFERENCE_ROOT")
    return root


def build(ref_root=None, verbose: bool = False) -> str:
    ref_root = reference_root(ref_root)
    srcs = [os.path.join(ref_root, f) for f in
            ("cwarp_cuda.cpp", "cwarp_cuda_gather_kernel.cu", "cwarp_cuda_rnnt_kernel.cu")]
    for s in srcs:
        if not os.path.isfile(s):
            raise FileNotFoundError(s)
    so = os.path.join(OUT, NAME + ".so")
    if os.path.isfile(so) and all(os.path.getmtime(so) >= os.path.getmtime(s) for s in srcs):
        return so
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    from torch.utils.cpp_extension import load
    load(name=NAME, sources=srcs, build_directory=OUT, verbose=verbose, is_python_module=False,
         extra_cuda_cflags=["-gencode=arch=compute_100a,code=sm_100a", "-O3"])
    return so


def load_ref():
    """Import the prebuilt checker; returns the module or None when it was never built."""
    so = os.path.join(OUT, NAME + ".so")
    if not os.path.isfile(so):
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), verbose=True))
