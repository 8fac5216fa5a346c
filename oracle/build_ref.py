"""Test infrastructure, not product code: builds the comparator oracle/_ref/_ac4k_ref*.so from the reference's own
sources where they lie in the reference checkout (nothing is copied into this repository).

What is built: the reference's three quantiser kernels and its RoPE kernel (lib/cuda/sm120/quantize_nvfp4.cu,
quantize_fp8.cu, quantize_int8.cu, rope3d.cu) with the flags of its setup.py:164-183 (-O3, --use_fast_math, ...),
except the architecture, which is `-gencode arch=compute_100a,code=sm_100a`, plus the binding in oracle/ref_shim.cc.
The reference's GEMM and attention kernels are left out: their `mma.sync ... kind::mxf4nvf4` / sm_120a MMAs do not
assemble for sm_100a.

The reference checkout is looked for in $AC4K_REFERENCE_DIR, then in ~/reference; without one (the GPU box) an
existing build is used as it is and a missing one stays missing: the tests that need it skip.

    python oracle/build_ref.py [--force]
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
SOURCES = ["quantize_nvfp4.cu", "quantize_fp8.cu", "quantize_int8.cu", "rope3d.cu"]


def reference_dir() -> str | None:
    for cand in (os.environ.get("AC4K_REFERENCE_DIR"), os.path.join(os.path.expanduser("~"), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "lib", "cuda", "sm120")):
            return cand
    return None


def module_path() -> str:
    return os.path.join(OUT_DIR, "_ac4k_ref" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_ref(force: bool = False) -> str | None:
    """Returns the path of the built module, or None when there is neither a reference checkout nor an earlier build."""
    target = module_path()
    ref = reference_dir()
    if ref is None:
        return target if os.path.exists(target) else None
    srcs = [os.path.join(ref, "lib", "cuda", "sm120", s) for s in SOURCES]
    shim = os.path.join(HERE, "ref_shim.cc")
    deps = srcs + [shim, os.path.abspath(__file__)]
    if not force and os.path.exists(target) and all(os.path.getmtime(target) >= os.path.getmtime(d) for d in deps):
        return target
    import torch
    from torch.utils import cpp_extension
    os.makedirs(os.path.join(OUT_DIR, "obj"), exist_ok=True)
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    incs = []
    for inc in cpp_extension.include_paths():
        incs += ["-isystem", inc]
    incs += ["-isystem", sysconfig.get_paths()["include"],
             "-I", os.path.join(ref, "include"), "-I", os.path.join(ref, "lib", "cuda", "common"),
             "-I", os.path.join(ref, "lib", "cuda", "sm120")]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    nvcc_flags = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "--use_fast_math", "-DAC4K_ARCH_SM120=1",
                  "-DAC4K_BACKEND_CUDA=1", "-DNDEBUG", "-w", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", abi]
    jobs, objs = [], []
    for s in srcs:
        obj = os.path.join(OUT_DIR, "obj", os.path.basename(s)[:-3] + ".o")
        objs.append(obj)
        jobs.append([nvcc, *nvcc_flags, *incs, "-c", s, "-o", obj])
    shim_obj = os.path.join(OUT_DIR, "obj", "ref_shim.o")
    objs.append(shim_obj)
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    jobs.append([cxx, "-O2", "-std=c++17", "-fPIC", "-DTORCH_API_INCLUDE_EXTENSION_H", abi, *incs,
                 "-isystem", os.path.join(cuda_home, "include"), "-c", shim, "-o", shim_obj])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("building the reference comparator failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)

    with concurrent.futures.ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(run, jobs))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    run([cxx, "-shared", "-o", target, *objs, "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
         "-ltorch_python", "-L", os.path.join(cuda_home, "lib64"), "-lcudart", f"-Wl,-rpath,{torch_lib}"])
    return target


def load():
    """The built module, or None when it has not been built (it links against torch's libraries, so torch is imported first)."""
    path = module_path()
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401
    spec = importlib.util.spec_from_file_location("_ac4k_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build_ref(force="--force" in sys.argv))
