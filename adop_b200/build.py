"""In-tree build of the CUDA library (sm_100a only) and, for tests, of the CPU checker.

    python -m adop_b200.build            # libadop_raster.so (+ oracle/libadop_oracle.so)
"""
import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
SOURCES = ["capi_common.cu", "raster_forward.cu", "raster_forward_static.cu", "raster_backward.cu", "pose_tonemap.cu",
           "peer_reduce.cu", "peer_update.cu", "points_preprocess.cu"]
CONTRACTION_ALLOWED = {"pose_tonemap.cu"}
LIB = os.path.join(PKG_DIR, "libadop_raster.so")

# -fmad=false: the arithmetic header promises the same bits on host and device
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--use_fast_math=false"]


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _deps():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    inc = os.path.join(ROOT, "include", "adop")
    deps += [os.path.join(inc, f) for f in os.listdir(inc) if f.endswith(".h")]
    return deps


def build_library(force=False, verbose=False):
    if not force and _newer(LIB, _deps()):
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    objdir = os.path.join(PKG_DIR, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    objs = []
    inc = os.path.join(ROOT, "include", "adop")
    shared = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    shared += [os.path.join(inc, f) for f in os.listdir(inc) if f.endswith(".h")]
    for src in SOURCES:  # one nvcc per translation unit, side by side; objects newer than their sources are kept
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        if not force and _newer(obj, [os.path.join(CSRC, src)] + shared):
            objs.append(obj)
            continue
        # the rasterizer's arithmetic promises host/device bit equality (no contraction); the photometric kernels and the
        # pose update are checked within a tolerance and may fuse multiply-adds
        use = [f for f in flags if f != "-fmad=false"] if src in CONTRACTION_ALLOWED else flags
        cmd = [nvcc] + use + ["-I", os.path.join(ROOT, "include"), "-c", "-o", obj, os.path.join(CSRC, src)]
        procs.append((cmd, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, obj, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
        objs.append(obj)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed: " + " ".join(cmd))
    return LIB


TORCH_OP_SRC = os.path.join(CSRC, "torch_op.cpp")
TORCH_OP_LIB = os.path.join(PKG_DIR, "libadop_torch.so")


def build_torch_op(force=False, verbose=False):
    """The libTorch autograd operator over the C ABI (adop_b200/libadop_torch.so); links against libadop_raster.so."""
    build_library()
    deps = [TORCH_OP_SRC, os.path.join(ROOT, "include", "adop", "adop_raster.h"), LIB]
    if not force and _newer(TORCH_OP_LIB, deps):
        return TORCH_OP_LIB
    import torch
    from torch.utils import cpp_extension
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [os.environ.get("CXX_HOST", "/usr/bin/g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-Wno-deprecated-declarations",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in cpp_extension.include_paths() + ["/usr/local/cuda/include", os.path.join(ROOT, "include")]:
        cmd += ["-I", inc]
    cmd += [TORCH_OP_SRC, "-o", TORCH_OP_LIB, "-L", tlib, "-L", PKG_DIR, "-ladop_raster", "-ltorch", "-ltorch_cpu", "-lc10",
            "-ltorch_cuda", "-lc10_cuda", "-L", "/usr/local/cuda/lib64", "-lcudart",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("building the libTorch operator failed")
    return TORCH_OP_LIB


def build_oracle(force=False):
    """The CPU checker (test infrastructure; never loaded by the library)."""
    odir = os.path.join(ROOT, "oracle")
    if force:
        subprocess.run(["make", "-C", odir, "clean"], check=True, capture_output=True)
    r = subprocess.run(["make", "-C", odir], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("oracle build failed")
    return os.path.join(odir, "libadop_oracle.so")


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
    print(build_torch_op(force="--force" in sys.argv, verbose=True))
    print(build_oracle(force="--force" in sys.argv))
