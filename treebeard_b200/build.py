"""Builds the native library in-tree (nvcc, sm_100a)."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libtreebeard-runtime.so")


def build(jobs: int = 0, verbose: bool = False) -> str:
    """Compiles every CUDA/C++ source under csrc/ into lib/libtreebeard-runtime.so, the two
    module-side libraries and the walk micro-benchmark
    (``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo``).  Needs no GPU."""
    jobs = jobs or os.cpu_count() or 4
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), f"-j{jobs}", "all", "probes"]
    res = subprocess.run(cmd, capture_output=not verbose, text=True)
    if res.returncode != 0:
        raise RuntimeError("native build failed:\n" + (res.stdout or "") + (res.stderr or ""))
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose=True))
