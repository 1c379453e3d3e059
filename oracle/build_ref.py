"""Builds the reference project's own device kernels, compiled for sm_100a straight from the reference
checkout with the reference's own compiler flags (-O3 --use_fast_math ...); nothing is copied into this
tree and the output folder oracle/_ref/ is git-ignored:

    libcpmcu_ref_kernels.so   the stages listed in oracle/ref_kernels.cu (seconds to build)
    libcpmcu_ref_marlin.so    the W4A16 GEMM, oracle/ref_marlin.cu + the reference's gptq_marlin.cu
                              (needs the PyTorch headers; many minutes to build, so only on request)

TEST INFRASTRUCTURE: only tests/ and the fixture generator tests/golden/make_ref_golden.py load the
results.  Where no reference checkout is present (the GPU machine) the prebuilt libraries are used as is.

    python -m oracle.build_ref [--force] [--marlin]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libcpmcu_ref_kernels.so")
REFERENCE = os.environ.get("CPMCU_REFERENCE_DIR", "/root/reference")


MARLIN_LIB = os.path.join(OUT_DIR, "libcpmcu_ref_marlin.so")
# the flags of the reference's release build (its setup.py), with the target changed to sm_100a
REFERENCE_FLAGS = ["-std=c++17", "-O3", "--use_fast_math", "-w", "-lineinfo",
                   "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
                   "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "--expt-relaxed-constexpr", "--expt-extended-lambda",
                   "-DENABLE_DTYPE_BF16", "-gencode", "arch=compute_100a,code=sm_100a"]


def _cut_eagle_kernels(src_dir, dst):
    """eagle.cuh defines the draft-tree kernels (log_softmax, cumsum, update_tree, build_dynamic_tree ...)
    ahead of `struct Skip`, but its #include list pulls in the attention code, which needs the un-vendored
    CUTLASS tree.  The kernel section is cut out verbatim into the build folder and removed after the
    compile."""
    lines = open(os.path.join(src_dir, "model", "eagle.cuh")).read().split("\n")
    first = next(i for i, l in enumerate(lines) if l.startswith("namespace {"))
    last = next(i for i, l in enumerate(lines) if l.startswith("struct Skip"))
    while not lines[last - 1].startswith("template"):
        last -= 1
    with open(dst, "w") as f:
        f.write("\n".join(lines[first:last - 1]) + "\n")


def build_ref(force=False, verbose=False):
    """Returns the library path, or None when neither a reference checkout nor a prebuilt library exists."""
    src_dir = os.path.join(REFERENCE, "src")
    if not os.path.isdir(src_dir):
        return LIB if os.path.exists(LIB) else None
    wrapper = os.path.join(HERE, "ref_kernels.cu")
    deps = [wrapper, os.path.abspath(__file__)]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(d) for d in deps):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    inc = os.path.join(OUT_DIR, "eagle_kernels.inc")
    _cut_eagle_kernels(src_dir, inc)
    cmd = ["nvcc", "-shared", "-Xcompiler", "-fPIC"] + REFERENCE_FLAGS + [
           "-I", src_dir, "-I", OUT_DIR, "-o", LIB,
           wrapper, os.path.join(src_dir, "utils.cu"), os.path.join(src_dir, "signal_handler.cu"),
           "-lcublas", "-ldl"]
    if verbose:
        print(" ".join(cmd))
    try:
        subprocess.run(cmd, check=True)
    finally:
        if os.path.exists(inc):
            os.remove(inc)
    return LIB


def build_ref_marlin(force=False, verbose=False):
    """The reference's Marlin W4A16 GEMM.  Returns the library path or None."""
    src_dir = os.path.join(REFERENCE, "src")
    if not os.path.isdir(src_dir):
        return MARLIN_LIB if os.path.exists(MARLIN_LIB) else None
    wrapper = os.path.join(HERE, "ref_marlin.cu")
    if not force and os.path.exists(MARLIN_LIB) and os.path.getmtime(MARLIN_LIB) >= os.path.getmtime(wrapper):
        return MARLIN_LIB
    import sysconfig
    import torch
    tdir = os.path.dirname(torch.__file__)
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["nvcc", "-shared", "-Xcompiler", "-fPIC"] + REFERENCE_FLAGS + [
           "-I", src_dir, "-I", os.path.join(tdir, "include"),
           "-I", os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
           "-I", sysconfig.get_paths()["include"], "-o", MARLIN_LIB,
           wrapper, os.path.join(src_dir, "qgemm", "gptq_marlin", "gptq_marlin.cu"),
           "-L", os.path.join(tdir, "lib"), "-lc10", "-ltorch_cpu", "-Xlinker", "-rpath=" + os.path.join(tdir, "lib")]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return MARLIN_LIB


if __name__ == "__main__":
    print(build_ref(force="--force" in sys.argv, verbose=True))
    if "--marlin" in sys.argv:
        print(build_ref_marlin(force="--force" in sys.argv, verbose=True))
