"""Builds ``libjitnn_b200.so`` in-tree with nvcc for sm_100a.

    python -m jitnn_b200.build [--force] [--verbose]

Each ``csrc/*.cu`` is compiled to an object under ``csrc/build/`` (only when it or a header is
newer than its object) and the objects are linked into ``jitnn_b200/libjitnn_b200.so``.
"""
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libjitnn_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found: the CUDA toolkit is needed to build libjitnn_b200.so")
    return path


def _newest_header():
    heads = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return max(os.path.getmtime(h) for h in heads)


def _compile(src, obj, verbose, extra):
    cmd = [nvcc()] + NVCC_FLAGS + extra + ["-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, res.stdout, res.stderr))
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)


def build(force=False, verbose=False, ptxas_info=False):
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    header_time = _newest_header()
    jobs = []
    objects = []
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), header_time)
        if stale:
            jobs.append((src, obj))
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, os.cpu_count() or 1)) as pool:
        for f in [pool.submit(_compile, s, o, verbose or ptxas_info, extra) for s, o in jobs]:
            f.result()
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc(), "-shared", "-o", LIB] + objects + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_info="--ptxas" in sys.argv))
