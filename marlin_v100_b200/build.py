"""In-tree build of the CUDA library: one nvcc object per .cu file, linked into
``marlin_v100_b200/lib/libmarlin_b200.so`` (sm_100a only).  ``python -m marlin_v100_b200.build``."""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libmarlin_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(PKG, "build")
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(PKG), "include", "marlin_b200.h"))
    srcs = sources()
    objs = [os.path.join(obj_dir, os.path.basename(s)[:-3] + ".o") for s in srcs]

    def compile_one(pair):
        src, obj = pair
        if not force and not _stale(obj, [src] + headers):
            return ""
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        logs = list(ex.map(compile_one, zip(srcs, objs)))
    if verbose:
        for log in logs:
            if log:
                sys.stderr.write(log)
    if force or _stale(LIB_PATH, objs):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


TORCH_EXT_DIR = os.path.join(CSRC, "torch")
TORCH_MODULES = {"_C": "ops_dense.cpp", "_moe_C": "ops_moe.cpp"}


def torch_module_path(name: str) -> str:
    return os.path.join(PKG, f"{name}.abi3.so")


def build_torch_ops(force: bool = False) -> list[str]:
    """The two torch extension modules `_C` / `_moe_C` (operator schemas of the reference, bodies forwarding to
    libmarlin_b200.so).  Host C++ only: compiled with g++ against torch's headers, linked to the library by a
    relative rpath, so the three files can be copied together into another package (`vllm/`)."""
    from torch.utils import cpp_extension as ce
    import sysconfig
    build()
    lib_dir = os.path.join(os.path.dirname(ce.__file__), "..", "lib")
    lib_dir = os.path.abspath(lib_dir)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    incs = [*ce.include_paths(), sysconfig.get_paths()["include"], os.path.join(cuda_home, "include"),
            os.path.join(os.path.dirname(PKG), "include"), TORCH_EXT_DIR]
    common = os.path.join(TORCH_EXT_DIR, "binding_common.h")
    header = os.path.join(os.path.dirname(PKG), "include", "marlin_b200.h")
    outs = []

    def one(item):
        name, src = item
        src = os.path.join(TORCH_EXT_DIR, src)
        out = torch_module_path(name)
        if not force and not _stale(out, [src, common, header, LIB_PATH]):
            return out
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DPy_LIMITED_API=0x03090000",
               f"-DTORCH_EXTENSION_NAME={name}", "-D_GLIBCXX_USE_CXX11_ABI=1",
               *[f"-I{i}" for i in incs], src, "-o", out,
               f"-L{LIB_DIR}", "-lmarlin_b200", f"-L{lib_dir}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10",
               "-lc10_cuda", "-Wl,-rpath,$ORIGIN/lib", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{lib_dir}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed for {src}:\n{r.stdout}\n{r.stderr}")
        return out

    with concurrent.futures.ThreadPoolExecutor(max_workers=2) as ex:
        outs = list(ex.map(one, TORCH_MODULES.items()))
    return outs


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
    if "--torch-ops" in sys.argv:
        print(build_torch_ops(force="--force" in sys.argv))
