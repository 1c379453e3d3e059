"""Builds the reference project's own device code, compiled for sm_100 straight from a reference checkout
with the reference's own compiler flags (-O3 --use_fast_math ...); nothing is copied into this tree and the
output folders (oracle/_ref/, baseline/_ref/) are git-ignored:

    libcpmcu_ref_kernels.so   the stages listed in oracle/ref_kernels.cu (seconds to build)
    libcpmcu_ref_marlin.so    the W4A16 GEMM, oracle/ref_marlin.cu + the reference's gptq_marlin.cu
                              (needs the PyTorch headers; many minutes to build, so only on request)
    libcpmcu_ref_flash.so     the attention code, oracle/ref_flash.cu + the reference's four head_dim-128 bf16
                              flash_attn translation units (about four minutes each, in parallel)
    baseline/_ref/cpmcu/      the reference's whole extension `cpmcu.C` (entry.cu, utils.cu, signal_handler.cu,
                              perf.cu, gptq_marlin.cu and the same four flash_attn units, the source list of
                              its setup.py) next to a copy of its Python package: the reference CUDA build
                              that bench.py times beside this library

The reference's `src/cutlass` submodule is empty in the checkout; the header-only CUTLASS tree that ships
inside this image's Python packages (flashinfer/data/cutlass/include) is put on the include path instead.

TEST / BENCHMARK INFRASTRUCTURE: only tests/, the fixture generators under tests/golden/ and bench.py's
reference arm load the results.  Where no reference checkout is present (the GPU machine) the prebuilt
libraries are used as they are.  The checkout is looked for in $CPMCU_REFERENCE_DIR, else in a folder named
`reference` beside this repository.

    python -m oracle.build_ref [--force] [--marlin] [--flash] [--extension]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libcpmcu_ref_kernels.so")
REFERENCE = os.environ.get("CPMCU_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


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


# ---------------------------------------------------------------------------- attention + whole extension
FLASH_LIB = os.path.join(OUT_DIR, "libcpmcu_ref_flash.so")
EXT_DIR = os.path.join(os.path.dirname(HERE), "baseline", "_ref")
FLASH_UNITS = ["flash_attn/src/flash_fwd_hdim128_bf16_sm80.cu", "flash_attn/src/flash_fwd_hdim128_bf16_causal_sm80.cu",
               "flash_attn/src/flash_fwd_split_hdim128_bf16_sm80.cu",
               "flash_attn/src/flash_fwd_split_hdim128_bf16_causal_sm80.cu"]
# the source list of the reference's setup.py for CPMCU_DTYPE=bf16
EXTENSION_UNITS = ["entry.cu", "utils.cu", "signal_handler.cu", "perf.cu", "qgemm/gptq_marlin/gptq_marlin.cu"] + FLASH_UNITS


def _cutlass_include():
    import importlib.util
    for pkg, sub in (("flashinfer", ("data", "cutlass", "include")), ("tilelang", ("3rdparty", "cutlass", "include"))):
        spec = importlib.util.find_spec(pkg)
        if spec is not None and spec.submodule_search_locations:
            d = os.path.join(list(spec.submodule_search_locations)[0], *sub)
            if os.path.isdir(os.path.join(d, "cute")):
                return d
    raise RuntimeError("no CUTLASS/CuTe header tree found in the installed Python packages")


def _extension_flags(src_dir):
    """The nvcc line of the reference's setup.py (release mode, CPMCU_DTYPE=bf16, CPMCU_CUDA_ARCH=100)."""
    import sysconfig
    import pybind11
    import torch
    tdir = os.path.dirname(torch.__file__)
    return ["-std=c++17", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
            "-U__CUDA_NO_HALF2_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "--expt-relaxed-constexpr",
            "--expt-extended-lambda", "-DENABLE_DTYPE_BF16", "-O3", "--use_fast_math", "-w",
            "-gencode", "arch=compute_100,code=sm_100", "-D_ARCH100", "-Xcompiler", "-fPIC",
            "-I", os.path.join(src_dir, "flash_attn"), "-I", os.path.join(src_dir, "flash_attn", "src"),
            "-I", _cutlass_include(), "-I", src_dir, "-I", os.path.join(tdir, "include"),
            "-I", os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
            "-I", sysconfig.get_paths()["include"], "-I", pybind11.get_include(), "-DTORCH_EXTENSION_NAME=C"]


def _compile_units(units, src_dir, force=False, verbose=False, jobs=None):
    """Compiles reference translation units (paths relative to its src/) and files of this folder into the
    object cache ($CPMCU_REF_OBJ_DIR, default <tmp>/cpmcu_ref_obj); returns the object paths."""
    import concurrent.futures
    import tempfile
    obj_dir = os.environ.get("CPMCU_REF_OBJ_DIR") or os.path.join(tempfile.gettempdir(), "cpmcu_ref_obj")
    os.makedirs(obj_dir, exist_ok=True)
    flags = _extension_flags(src_dir)

    def one(unit):
        src = unit if os.path.isabs(unit) else os.path.join(src_dir, unit)
        obj = os.path.join(obj_dir, os.path.splitext(os.path.basename(unit))[0] + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < os.path.getmtime(src):
            cmd = ["nvcc"] + flags + ["-c", src, "-o", obj]
            if verbose:
                print(" ".join(cmd), flush=True)
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (unit, res.stdout[-4000:], res.stderr[-4000:]))
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs or max(1, (os.cpu_count() or 2) - 2)) as ex:
        return list(ex.map(one, units))


def build_ref_flash(force=False, verbose=False):
    """The reference's attention entry points (mha_fwd_kvcache, mha_fwd_stage1).  Returns the library path or None."""
    src_dir = os.path.join(REFERENCE, "src")
    if not os.path.isdir(src_dir):
        return FLASH_LIB if os.path.exists(FLASH_LIB) else None
    wrapper = os.path.join(HERE, "ref_flash.cu")
    if not force and os.path.exists(FLASH_LIB) and os.path.getmtime(FLASH_LIB) >= os.path.getmtime(wrapper):
        return FLASH_LIB
    objs = _compile_units(FLASH_UNITS + [wrapper], src_dir, force=force, verbose=verbose)
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["nvcc", "-shared", "-o", FLASH_LIB] + objs + ["-gencode", "arch=compute_100,code=sm_100", "-lcudart"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return FLASH_LIB


def extension_path():
    import sysconfig
    return os.path.join(EXT_DIR, "cpmcu", "C" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_ref_extension(force=False, verbose=False):
    """The reference's whole extension, importable as `cpmcu` from baseline/_ref/ (what `pip install --target
    baseline/_ref` of the reference would leave there).  Returns baseline/_ref or None."""
    import shutil
    src_dir = os.path.join(REFERENCE, "src")
    ext = extension_path()
    if not os.path.isdir(src_dir):
        return EXT_DIR if os.path.exists(ext) else None
    if not force and os.path.exists(ext):
        return EXT_DIR
    objs = _compile_units(EXTENSION_UNITS, src_dir, force=force, verbose=verbose)
    import torch
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    pkg = os.path.join(EXT_DIR, "cpmcu")
    if os.path.isdir(pkg):
        shutil.rmtree(pkg)
    shutil.copytree(os.path.join(REFERENCE, "cpmcu"), pkg, ignore=shutil.ignore_patterns("__pycache__", "*.so"))
    for root, dirs, files in os.walk(EXT_DIR):   # the checkout may be read-only; the copy must stay removable
        for name in dirs + files:
            os.chmod(os.path.join(root, name), 0o755 if name in dirs else 0o644)
    cmd = ["nvcc", "-shared", "-o", ext] + objs + ["-gencode", "arch=compute_100,code=sm_100", "-lcudart", "-lcublas",
           "-ldl", "-L", tlib, "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-Xlinker", "-rpath=" + tlib]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return EXT_DIR


if __name__ == "__main__":
    print(build_ref(force="--force" in sys.argv, verbose=True))
    if "--marlin" in sys.argv:
        print(build_ref_marlin(force="--force" in sys.argv, verbose=True))
    if "--flash" in sys.argv:
        print(build_ref_flash(force="--force" in sys.argv, verbose=True))
    if "--extension" in sys.argv:
        print(build_ref_extension(force="--force" in sys.argv, verbose=True))
