"""Build the C-ABI shared library `libac4k_b200.so` in-tree with nvcc for sm_100a.

    python ac4k_kernel_b200/build.py [--force] [--verbose] [--pybind]

One nvcc invocation per .cu (in parallel), then a link step.  The library links the CUDA
runtime statically and resolves the driver entry point it needs (tensor-map encoding) at
run time, so it has no link-time dependency on libcuda.

`--pybind` (or build_pybind()) also compiles csrc/bindings_pybind.cc with the host compiler into
`native/_cuda_ops*.so`: the pybind11 module with the reference's names and signatures, linked
against the library above.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libac4k_b200.so")

SOURCES = ["cabi.cu", "quantize_nvfp4.cu", "quantize_rowwise.cu", "linear_nvfp4.cu",
           "linear_nvfp4_2cta.cu", "linear_nvfp4_skinny.cu", "mha_nvfp4.cu", "rope3d.cu", "mha_int8_fp8.cu", "quantize_int8_block.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", 
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build_hooks(force: bool = False) -> str:
    """The same library with -DAC4K_DEBUG_HOOKS (measurement switches exported, wait limit adjustable) as
    `build_hooks/libac4k_b200_hooks.so`: used by the wait-expiry test and by experiments, never shipped."""
    return build(force=force, extra="-DAC4K_DEBUG_HOOKS", obj_dir=os.path.join(PKG_DIR, "build_hooks"),
                 lib_path=os.path.join(PKG_DIR, "build_hooks", "libac4k_b200_hooks.so"))


def build(force: bool = False, verbose: bool = False, extra: str | None = None, obj_dir: str | None = None,
          lib_path: str | None = None) -> str:
    nvcc = _nvcc()
    OBJ_DIR = obj_dir or globals()["OBJ_DIR"]
    LIB_PATH = lib_path or globals()["LIB_PATH"]
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "ac4k_b200.h"))
    headers.append(os.path.abspath(__file__))
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    # objects built with other extra flags (a debug or trace build) are stale
    extra = os.environ.get("AC4K_NVCC_EXTRA", "") if extra is None else extra
    stamp = os.path.join(OBJ_DIR, "flags.txt")
    if not os.path.exists(stamp) or open(stamp).read() != extra:
        force = True
    with open(stamp, "w") as f:
        f.write(extra)
    objs = []
    jobs = []
    for src in srcs:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or not _newer(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, *extra.split(), "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stdout + r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=4) as ex:
        for out in ex.map(run, jobs):
            if verbose and out.strip():
                print(out)
    if jobs or force or not _newer(LIB_PATH, objs):
        run([nvcc, "-shared", "-o", LIB_PATH, *objs, "-cudart", "static", "-Xcompiler", "-fPIC"])
    return LIB_PATH


def build_pybind(force: bool = False) -> str:
    """Compile the pybind11 `_cuda_ops` module (host code only) against torch's headers and link it to
    libac4k_b200.so (found through an $ORIGIN-relative run path).  Returns the path of the module."""
    import sysconfig
    import torch
    from torch.utils import cpp_extension
    src = os.path.join(CSRC, "bindings_pybind.cc")
    out_dir = os.path.join(PKG_DIR, "native")
    os.makedirs(out_dir, exist_ok=True)
    target = os.path.join(out_dir, "_cuda_ops" + sysconfig.get_config_var("EXT_SUFFIX"))
    deps = [src, os.path.join(ROOT, "include", "ac4k_b200.h"), os.path.abspath(__file__)]
    if not os.path.exists(LIB_PATH):
        build()
    if not force and _newer(target, deps):
        return target
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cuda_home = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-DTORCH_EXTENSION_NAME=_cuda_ops", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += ["-isystem", sysconfig.get_paths()["include"], "-isystem", os.path.join(cuda_home, "include"),
            "-I", os.path.join(ROOT, "include"), src, "-o", target,
            "-L", PKG_DIR, "-l:libac4k_b200.so", "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch",
            "-ltorch_python", "-Wl,-rpath,$ORIGIN/..", f"-Wl,-rpath,{torch_lib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the pybind module failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return target


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
    if "--hooks" in sys.argv:
        print(build_hooks(force="--force" in sys.argv))
    if "--pybind" in sys.argv:
        print(build_pybind(force="--force" in sys.argv))
