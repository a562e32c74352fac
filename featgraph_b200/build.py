"""Compiles the CUDA sources under csrc/ into csrc/libfeatgraph_b200.so (sm_100a only).

Run as ``python -m featgraph_b200.build``.  The shared library is built in-tree and is
loaded with ctypes through the C ABI declared in include/featgraph_b200.h.
"""
import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(CSRC, "libfeatgraph_b200.so")
SOURCES = ["api.cu", "spmm.cu", "spmm_noalloc.cu", "sddmm.cu", "peer.cu"]
HEADERS = ["common.cuh", os.path.join("..", "..", "include", "featgraph_b200.h")]

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps)


def build_library(force=False, verbose=False, defines=(), output=None):
    """Build the library if it is missing or older than a source; returns its path.

    Every source is compiled to an object file in its own nvcc process (the operator-pair
    instantiations make spmm.cu and sddmm.cu the long poles), then the objects are linked."""
    output = output or LIB_PATH
    if not force and output == LIB_PATH and not is_stale():
        return LIB_PATH
    import tempfile
    common = [_nvcc()] + [f for f in NVCC_FLAGS if f != "-shared"] + ["-D" + d for d in defines]
    common += ["-Xptxas", "-v"] if verbose else []
    with tempfile.TemporaryDirectory(prefix="fg_build_") as tmp:
        jobs = []
        for src in SOURCES:
            obj = os.path.join(tmp, src.replace(".cu", ".o"))
            cmd = common + ["-c", os.path.join(CSRC, src), "-o", obj]
            jobs.append((cmd, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                                    stderr=subprocess.STDOUT, text=True)))
        objs = []
        for cmd, obj, proc in jobs:
            out, _ = proc.communicate()
            if verbose:
                sys.stderr.write(out)
            if proc.returncode != 0:
                raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + out)
            objs.append(obj)
        link = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", output]
        res = subprocess.run(link + objs, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + " ".join(link) + "\n" + res.stdout + res.stderr)
    return output


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
