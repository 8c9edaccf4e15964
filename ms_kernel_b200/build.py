"""In-tree build of the native code.

    python -m ms_kernel_b200.build            # build what is out of date
    python -m ms_kernel_b200.build --force

Produces, next to this file:
  libmsaq_b200.so            the C-ABI library (nvcc, sm_100a only, no torch)
  ms_cuda.<abi>.so           the torch operator module that forwards to it

nvcc cross-compiles without a GPU, so the build runs on a CPU-only machine.
"""

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
ROOT = os.path.dirname(HERE)

CU_SOURCES = ["capi.cu", "kv_pack.cu", "gemv.cu", "gemv_generic.cu", "kv_decode.cu", "layer_glue.cu", "wa_gemv.cu", "peer_exchange.cu"]
LIB_NAME = "libmsaq_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
] + os.environ.get("MSAQ_NVCC_EXTRA", "").split()      # e.g. -DMSAQ_TRACE for the time-stamp diagnostic build


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the native code cannot be built")
    return exe


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(ROOT, "include", "msaq_b200.h"))
    return hs


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    return r.stdout + r.stderr


def _stamp_ok(stamp, digest, outputs):
    if not all(os.path.exists(o) for o in outputs):
        return False
    try:
        with open(stamp) as f:
            return f.read().strip() == digest
    except OSError:
        return False


def build_library(force=False, verbose=False):
    """Compile the CUDA sources and link libmsaq_b200.so.  Returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    out = os.path.join(HERE, LIB_NAME)
    srcs = [os.path.join(CSRC, s) for s in CU_SOURCES]
    digest = _digest(srcs + _headers(), " ".join(NVCC_FLAGS))
    stamp = os.path.join(OBJ, "lib.stamp")
    if not force and _stamp_ok(stamp, digest, [out]):
        return out
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src):
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        log = _run([nvcc] + NVCC_FLAGS + extra + ["-c", src, "-o", obj])
        return obj, log

    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(compile_one, srcs))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    _run([nvcc, "-shared", "-o", out] + [o for o, _ in results])
    with open(stamp, "w") as f:
        f.write(digest)
    return out


def torch_module_path():
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(HERE, "ms_cuda" + suffix)


def build_torch_module(force=False):
    """Compile csrc/torch_ops.cpp into the importable `ms_cuda` module."""
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OBJ, exist_ok=True)
    lib = build_library(force=force)
    out = torch_module_path()
    src = os.path.join(CSRC, "torch_ops.cpp")
    digest = _digest([src, os.path.join(ROOT, "include", "msaq_b200.h")], torch.__version__)
    stamp = os.path.join(OBJ, "torch.stamp")
    if not force and _stamp_ok(stamp, digest, [out]):
        return out
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]
    torch_lib = ce.library_paths()[0]
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi, "-DTORCH_EXTENSION_NAME=ms_cuda", "-w"]
    for i in inc:
        cmd += ["-isystem", i]
    cmd += [src, "-o", out, "-L" + HERE, "-l:" + LIB_NAME, "-L" + torch_lib,
            "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
            "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    _run(cmd)
    with open(stamp, "w") as f:
        f.write(digest)
    assert os.path.exists(lib)
    return out


def build_all(force=False, verbose=False):
    lib = build_library(force=force, verbose=verbose)
    mod = build_torch_module(force=force)
    return lib, mod


if __name__ == "__main__":
    paths = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("\n".join(paths))
