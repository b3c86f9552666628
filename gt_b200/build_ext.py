"""Build the native extension in-tree (``gt_b200/_ext/gt_b200_native*.so``) for sm_100a.

``python -m gt_b200.build_ext`` compiles every ``csrc/*.cu`` with ``nvcc -gencode arch=compute_100a,code=sm_100a`` (explicit
``-gencode`` flags bypass torch's own architecture list) and links them with the pybind11 binding through
``torch.utils.cpp_extension`` + ninja.  No GPU is needed to build."""
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
BUILD = os.path.join(ROOT, "_ext")
NAME = "gt_b200_native"
CU = ["attn.cu", "attn_tile.cu", "spmm.cu", "rowops.cu", "gemm.cu", "p2p.cu"]


def sources():
    files = [os.path.join(CSRC, "binding.cpp")]
    files += [os.path.join(CSRC, f) for f in CU if os.path.exists(os.path.join(CSRC, f))]
    return files


def build(verbose=False):
    from torch.utils import cpp_extension
    os.makedirs(BUILD, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    return cpp_extension.load(
        name=NAME, sources=sources(), build_directory=BUILD, verbose=verbose, with_cuda=True,
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
                           "--use_fast_math", "-Xptxas", "-v", "--expt-relaxed-constexpr"],
        extra_ldflags=["-lcuda"] if os.path.exists("/usr/local/cuda/lib64/stubs/libcuda.so") and False else [],
    )


def load_prebuilt():
    """Import the already built module from ``_ext`` without invoking a compiler; ``None`` if it is not there."""
    import importlib.util
    import glob
    import torch  # noqa: F401  (the extension links against libtorch)
    cands = sorted(glob.glob(os.path.join(BUILD, NAME + "*.so")))
    if not cands:
        return None
    spec = importlib.util.spec_from_file_location(NAME, cands[-1])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    m = build(verbose="-v" in sys.argv)
    print("built", m.__file__)
