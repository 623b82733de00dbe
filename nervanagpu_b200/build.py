"""Builds libnervana_b200.so (sm_100a only) in-tree with nvcc.

Usage: python -m nervanagpu_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libnervana_b200.so")

SOURCES = ["runtime.cu", "tc_host.cu", "gemm.cu", "conv.cu", "pool.cu", "ew_rt.cu", "legacy_api.cu", "comm.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=default",
    "--expt-relaxed-constexpr",
    "-cudart", "static",
]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "nervana_b200.h"))
    objs = []
    procs = []
    for s in srcs:
        o = s[:-3] + ".o"
        objs.append(o)
        if force or _newer(o, [s] + headers):
            # NVCC_EXTRA: extra compiler flags for development builds (e.g. -DNG_TC_TIMELINE)
            extra = os.environ.get("NVCC_EXTRA", "").split()
            cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write("nvcc failed on %s:\n%s\n" % (s, out))
        elif verbose and out:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("build of libnervana_b200.so failed")
    if force or procs or _newer(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + [
            "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
            "-L/usr/local/cuda/lib64", "-lnvrtc", "-ldl", "-lpthread",
            "-Xlinker", "-rpath,/usr/local/cuda/lib64",
        ]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
