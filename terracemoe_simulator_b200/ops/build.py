"""Build the native library ``ops/lib/terrace_b200_ops.so`` in-tree.

Device code (``csrc/*.cu``) is compiled with plain ``nvcc -gencode
arch=compute_100a,code=sm_100a -lineinfo`` and includes no torch header, so a file takes
seconds; only the binding translation units (``csrc/*.cpp``) see torch.  Everything is linked
into one shared object that ``torch.ops.load_library`` picks up.

Counterpart of the reference's ``terrace/ops/csrc/build_ext.py`` and ``ascendc/build.sh`` (which
drive the AscendC toolchain).  Usage: ``python -m terracemoe_simulator_b200.ops.build [-v]``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(HERE, "build")
LIB_NAME = "terrace_b200_ops.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# sources whose results are compared with PyTorch oracles bit for bit (router selection, plan,
# normalisation): IEEE division and the accurate expf / rsqrtf, no --use_fast_math
PRECISE_MATH = {"router_sm100.cu", "moe_kernels.cu"}


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    if os.path.isfile(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()[:16]


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"command failed ({proc.returncode}): {' '.join(cmd)}\n"
                           f"{proc.stdout}\n{proc.stderr}")
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout, proc.stderr, flush=True)


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile (if sources changed) and return the path of the shared library."""
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    headers = sorted(f for f in os.listdir(CSRC) if f.endswith((".h", ".cuh")))
    out = os.path.join(LIB_DIR, LIB_NAME)
    stamp = os.path.join(LIB_DIR, LIB_NAME + ".stamp")
    digest = _digest([os.path.join(CSRC, f) for f in cu + cpp + headers] + [__file__],
                     torch.__version__)
    if (not force and os.path.isfile(out) and os.path.isfile(stamp)
            and open(stamp).read().strip() == digest):
        return out

    nvcc = _nvcc()
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "include")
    torch_inc = []
    for p in include_paths("cuda"):
        torch_inc += ["-isystem", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    jobs = []
    objs = []
    for f in cu:
        o = os.path.join(OBJ_DIR, f + ".o")
        objs.append(o)
        fast = [] if f in PRECISE_MATH else ["--use_fast_math"]
        jobs.append([nvcc, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", *fast,
                     "-Xcompiler", "-fPIC", "-I", CSRC, "-c", os.path.join(CSRC, f), "-o", o])
    for f in cpp:
        o = os.path.join(OBJ_DIR, f + ".o")
        objs.append(o)
        jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                     "-DTORCH_API_INCLUDE_EXTENSION_H", "-I", CSRC, "-isystem", cuda_inc,
                     *torch_inc, "-c", os.path.join(CSRC, f), "-o", o])
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        list(pool.map(lambda c: _run(c, verbose), jobs))
    lib_flags = []
    for p in library_paths("cuda"):
        lib_flags += ["-L", p, f"-Wl,-rpath,{p}"]
    _run(["g++", "-shared", "-o", out, *objs, *lib_flags, "-lc10", "-lc10_cuda", "-ltorch_cpu",
          "-ltorch_cuda", "-ltorch", "-lcudart"], verbose)
    with open(stamp, "w") as f:
        f.write(digest)
    return out


def main(argv) -> int:
    path = build(verbose="-v" in argv, force="-f" in argv)
    print(path)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
