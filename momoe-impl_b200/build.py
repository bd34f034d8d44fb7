"""Builds libmomoe_b200.so (sm_100a only) in-tree with nvcc.

    python momoe-impl_b200/build.py            # product library -> momoe-impl_b200/momoe/libmomoe_b200.so

nvcc cross-compiles, so this runs on machines without a GPU.  The library links cudart statically and
resolves the one driver entry point it needs at run time, so it also loads without a driver.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SOURCES = ["common.cu", "routing.cu", "grouped_gemm.cu", "decode_gemm.cu", "ep.cu"]
LIB_PATH = os.path.join(HERE, "momoe", "libmomoe_b200.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--threads", "4",
]


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def build(out=LIB_PATH, extra_flags=(), force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    deps.append(os.path.join(HERE, "..", "include", "momoe_b200.h"))
    if not force and not _stale(out, deps):
        return out
    tmp = out + ".tmp%d" % os.getpid()     # written beside the target, then renamed: readers never see a partial file
    cmd = [nvcc, "-shared", "-o", tmp] + NVCC_FLAGS + list(extra_flags) + srcs
    if verbose:
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError("nvcc failed building " + out)
    os.replace(tmp, out)
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True,
                extra_flags=["-Xptxas", "-v"] if "--ptxas" in sys.argv else []))
