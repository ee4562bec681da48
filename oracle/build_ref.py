"""Build the reference's own CUDA extensions for sm_100a into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  The sources are compiled where they lie in the
reference checkout (nothing is copied into this repository); only objects and
the six extension modules (fused_gatconv, fused_gmmconv, fused_edgeconv,
mhsddmm, mhtranspose, format_conversion) are written, all under oracle/_ref/.
The reference's setup.py asks for -arch=sm_70; the only change here is the
target architecture.  The modules need a GPU to run: on a GPU box the tests
compare them with the oracle and with the new kernels, and
tests/golden/make_golden.py records their outputs as fixtures.

    python oracle/build_ref.py /path/to/reference      (or DGNN_REFERENCE_ROOT=/path/to/reference)

Without either, a checkout named `reference` beside this repository is used when it exists.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_REF = os.environ.get("DGNN_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

EXTENSIONS = {
    "fused_gatconv": ["dgNN/src/fused_gatconv/fused_gatconv.cpp", "dgNN/src/fused_gatconv/fused_gatconv_kernel.cu"],
    "fused_edgeconv": ["dgNN/src/fused_edgeconv/fused_edgeconv.cpp", "dgNN/src/fused_edgeconv/fused_edgeconv_kernel.cu"],
    "fused_gmmconv": ["dgNN/src/fused_gmmconv/fused_gmmconv.cpp", "dgNN/src/fused_gmmconv/fused_gmmconv_kernel.cu"],
    "mhsddmm": ["dgNN/src/sddmm/mhsddmm.cc", "dgNN/src/sddmm/mhsddmm_kernel.cu"],
    "mhtranspose": ["dgNN/src/csr2csc/mhtranspose.cc", "dgNN/src/csr2csc/mhtranspose_kernel.cu"],
    "format_conversion": ["dgNN/src/convert/convert.cpp", "dgNN/src/convert/convert_kernel.cu"],
}


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout)
        raise RuntimeError("reference build step failed")


def build(ref_root: str = DEFAULT_REF, force: bool = False) -> list[str]:
    import torch
    from torch.utils import cpp_extension as ce

    if not os.path.isdir(os.path.join(ref_root, "dgNN", "src")):
        raise FileNotFoundError(f"no reference checkout at {ref_root}")
    os.makedirs(os.path.join(OUT, "obj"), exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", f"-I{cuda_home}/include"]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    built = []
    for name, sources in EXTENSIONS.items():
        target = os.path.join(OUT, name + suffix)
        built.append(target)
        if os.path.exists(target) and not force:
            continue
        common = [f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H", abi, "-DNDEBUG", "-O2", *inc]
        objs = []
        for src in sources:
            path = os.path.join(ref_root, src)
            obj = os.path.join(OUT, "obj", name + "_" + os.path.basename(src) + ".o")
            if src.endswith(".cu"):
                _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-Xcompiler", "-fPIC",
                      "--expt-relaxed-constexpr", *common, "-c", path, "-o", obj])
            else:
                _run(["g++", "-std=c++17", "-fPIC", *common, "-c", path, "-o", obj])
            objs.append(obj)
        _run(["g++", "-shared", "-o", target, *objs, f"-L{torch_lib}", f"-L{cuda_home}/lib64",
              f"-Wl,-rpath,{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
              "-lcudart", "-lcurand", "-lcusparse"])
    return built


def load():
    """Import the six reference modules from oracle/_ref (None if they were not built)."""
    import importlib.util

    import torch  # noqa: F401  (the modules link against libtorch)
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    mods = {}
    for name in EXTENSIONS:
        path = os.path.join(OUT, name + suffix)
        if not os.path.exists(path):
            return None
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods


if __name__ == "__main__":
    for p in build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REF, force="--force" in sys.argv):
        print(p)
