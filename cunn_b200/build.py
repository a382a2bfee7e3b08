"""Builds libTHCUNN.so (the sm_100a kernels + C ABI) in-tree with nvcc.

    python -m cunn_b200.build [--force] [--verbose]

Objects are compiled in parallel into cunn_b200/lib/obj and linked into
cunn_b200/lib/libTHCUNN.so.  nvcc cross-compiles, so no GPU is needed.
"""
import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
SO = os.path.join(LIBDIR, "libTHCUNN.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-ccbin", "/usr/bin/g++",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
    "-DCUNN_BUILDING=1",
]


if os.environ.get("CUNN_B200_DEV_HOOKS"):      # sweep builds only: tuning switches that are not part of the library
    FLAGS.append("-DCUNN_B200_DEV_HOOKS=1")


# Build inside a cutorch tree: CUNN_B200_USE_REAL_THC=<directory holding THC/THC.h>[:<directory holding libTHC.so>]
# makes the THNN layer use cutorch's own THCState / THCudaTensor and resolve its tensor calls in libTHC.
LINK_EXTRA = []
_thc = os.environ.get("CUNN_B200_USE_REAL_THC")
if _thc:
    inc, _, libdir = _thc.partition(":")
    FLAGS += ["-DCUNN_B200_USE_REAL_THC=1", "-I", inc]
    LINK_EXTRA = (["-L", libdir] if libdir else []) + ["-lTHC"]


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _deps_mtime():
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(CSRC, "*.inc")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return max([os.path.getmtime(h) for h in hdrs] + [os.path.getmtime(__file__)])


def _compile(src, obj, verbose):
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def build(force=False, verbose=False):
    os.makedirs(OBJDIR, exist_ok=True)
    stamp = os.path.join(OBJDIR, "flags.txt")
    flags = " ".join(FLAGS)
    if not os.path.exists(stamp) or open(stamp).read() != flags:
        force = True                                # objects built with other flags do not mix
    dep_t = _deps_mtime()
    jobs, objs = [], []
    for src in _sources():
        obj = os.path.join(OBJDIR, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), dep_t):
            jobs.append((src, obj))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for src, rc, out in ex.map(lambda j: _compile(j[0], j[1], verbose), jobs):
            if verbose or rc:
                sys.stderr.write(out)
            if rc:
                raise RuntimeError("nvcc failed on " + src)
    with open(stamp, "w") as f:
        f.write(flags)
    if jobs or not os.path.exists(SO):
        cmd = [NVCC, "-shared", "-ccbin", "/usr/bin/g++", "-o", SO] + objs + ["--cudart", "static", "-Xlinker", "--no-undefined"] + LINK_EXTRA
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of libTHCUNN.so failed")
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
