"""Build the reference project's own CUDA operators for sm_100a -- test infrastructure, not product.

    python oracle/build_ref.py [/path/to/reference]        # default /root/reference

Compiles the reference's sources where they lie (csrc/*.cu + csrc/pybind.cpp, nothing is copied into
this repository) with the flags of its setup.py (-O3 --use_fast_math --expt-extended-lambda), retargeted
from its sm_120 to `-gencode arch=compute_100a,code=sm_100a`, and links them into

    oracle/_ref/ms_cuda_ref.so

which is git-ignored (it still travels to the GPU box with the working tree).  Loading that library
(`torch.ops.load_library`) registers the reference's `torch.ops.msaq.*` operators -- the same names this
repository's `ms_cuda` registers, so it is only ever loaded in a process of its own (oracle/ref_cuda.py).
It is the reference's "certified CUDA path": a second oracle for the GPU parity tests and the same-box
timing anchor of the benchmark.  Nothing under ms_kernel_b200/ uses it.
"""

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "ms_cuda_ref.so")
SOURCES = ["pybind.cpp", "w_gemv.cu", "wa_gemm.cu", "kv_attention.cu", "rotate.cu", "mxint8.cu"]   # setup.py:45-52
NVCC_FLAGS = ["-O3", "-gencode", "arch=compute_100a,code=sm_100a", "--use_fast_math", "--expt-extended-lambda",
              "-std=c++17", "-Xcompiler", "-fPIC", "-w"]


def _digest(paths, extra):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()


def build(ref_root="/root/reference", force=False):
    """Returns the library path, or None when the reference checkout is not there."""
    csrc = os.path.join(ref_root, "csrc")
    if not os.path.isdir(csrc):
        return LIB if os.path.exists(LIB) else None
    import torch
    from torch.utils import cpp_extension as ce

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUT_DIR, exist_ok=True)
    srcs = [os.path.join(csrc, s) for s in SOURCES]
    deps = srcs + [os.path.join(csrc, "core", "ms_utils.cuh")]
    digest = _digest(deps, " ".join(NVCC_FLAGS) + torch.__version__)
    stamp = os.path.join(OUT_DIR, "ref.stamp")
    if not force and os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read().strip() == digest:
        return LIB
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = [csrc, os.path.join(csrc, "core")] + ce.include_paths() + [sysconfig.get_paths()["include"],
                                                                     os.path.join(cuda_home, "include")]
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    defs = ["-D_GLIBCXX_USE_CXX11_ABI=%d" % abi, "-DTORCH_EXTENSION_NAME=ms_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H"]

    def compile_one(src):
        obj = os.path.join(OUT_DIR, os.path.basename(src) + ".o")
        cmd = [nvcc] + NVCC_FLAGS + defs + sum((["-isystem", i] for i in inc), []) + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("reference build failed: %s\n%s" % (" ".join(cmd), (r.stdout + r.stderr)[-4000:]))
        return obj

    with cf.ThreadPoolExecutor(max_workers=len(srcs)) as ex:
        objs = list(ex.map(compile_one, srcs))
    torch_lib = ce.library_paths()[0]
    cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-L" + torch_lib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda",
                                                  "-lc10_cuda", "-ltorch_python", "-Xlinker", "-rpath," + torch_lib]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference link failed:\n" + (r.stdout + r.stderr)[-4000:])
    for o in objs:
        os.remove(o)
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else "/root/reference"
    print(build(root, force="--force" in sys.argv))
