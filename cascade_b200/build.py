"""Builds the device library (libcascade_b200.so) in-tree with nvcc for sm_100a.

Run as ``python -m cascade_b200.build``. Nothing is compiled at import time: the loader fails loudly when the
library is missing.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcascade_b200.so")
SOURCES = ["ctx.cu", "radix_sort.cu", "partition.cu", "doubling.cu", "build_sa.cu", "build_multi.cu", "exchange.cu", "comm_shm.cu", "query.cu", "corpus.cu", "host_tools.cu", "validate.cu", "stream_build.cu", "symbols.cu", "rank_shards.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-O3,-fopenmp", "--expt-relaxed-constexpr",
]


def _nvcc():
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    return "nvcc"


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if os.path.isfile(os.path.join(CSRC, f))]
    deps += [os.path.join(CSRC, "host", f) for f in os.listdir(os.path.join(CSRC, "host"))] + [os.path.join(HERE, "..", "include", "cascade_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compiles every .cu source to an object in parallel and links the shared library."""
    if not force and not needs_build():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    procs = []
    for s in srcs:
        obj = os.path.join(objdir, s.replace(".cu", ".o"))
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, s), "-o", obj]
        procs.append((s, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for s, obj, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}")
        objs.append(obj)
    cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-lcudart", "-Xcompiler", "-fopenmp", "-lgomp", "-lrt"]
    subprocess.check_call(cmd)
    build_tools()
    return LIB


def build_tools():
    """The command lines of the drop-in surface: bin/cascade and bin/query, linked against the library, and bin/sa_convert
    (host code only)."""
    bindir = os.path.join(HERE, "bin")
    os.makedirs(bindir, exist_ok=True)
    for name, src in (("cascade", "cascade_main.cpp"), ("query", "query_main.cpp")):
        cmd = [_nvcc(), "-O2", "-std=c++17", os.path.join(CSRC, "host", src), "-o", os.path.join(bindir, name), "-L" + HERE, "-lcascade_b200",
               "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/..", "-lcudart"]
        subprocess.check_call(cmd)
    subprocess.check_call(["g++", "-O2", "-std=c++17", os.path.join(CSRC, "host", "sa_convert_main.cpp"), "-o", os.path.join(bindir, "sa_convert")])


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
