"""Compile the reference's own CUDA renderer into oracle/_ref/ (test infrastructure only).

    python oracle/build_ref.py [/path/to/mlp-splatting]

Without an argument the checkout is looked for in $MLPSP_REFERENCE_ROOT, then in a directory named
"reference" beside this repository.

The reference's single translation unit (scannet/cuda/np_tile_kernels.cu, which includes its three
.cuh files) is compiled for sm_100a from where it lies, with the flags the reference's loader uses
by default (-DMLPSP_MAX_TILE_PRIMS=1536, scannet/cumodel.py:96-130), as a torch extension module
named mlpsp_ref_ext.  Nothing is copied into this repository; only the built module lands in
oracle/_ref/ (git-ignored).  The GPU tests load it, when present, to compare this library's output
with the reference kernels' output on the same device.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "mlpsp_ref_ext"


def reference_root():
    """The reference checkout: $MLPSP_REFERENCE_ROOT, else ../reference relative to this repository."""
    return os.environ.get("MLPSP_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root=None, verbose=False):
    src = os.path.join(ref_root or reference_root(), "scannet", "cuda", "np_tile_kernels.cu")
    if not os.path.exists(src):
        return None
    so = os.path.join(OUT, NAME + ".so")
    if os.path.exists(so) and os.path.getmtime(so) >= os.path.getmtime(src):
        return so
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load
    load(name=NAME, sources=[src], build_directory=OUT, verbose=verbose, is_python_module=True,
         extra_cuda_cflags=["-DMLPSP_MAX_TILE_PRIMS=1536", "-lineinfo"], with_cuda=True)
    obj = os.path.join(OUT, "np_tile_kernels.cuda.o")   # only the module travels to the GPU box
    if os.path.exists(so) and os.path.exists(obj):
        os.remove(obj)
    return so if os.path.exists(so) else None


def load_module():
    """Import the built module (None when it has not been built)."""
    so = os.path.join(OUT, NAME + ".so")
    if not os.path.exists(so):
        return None
    import importlib.util
    import torch  # noqa: F401  (the module links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True))
