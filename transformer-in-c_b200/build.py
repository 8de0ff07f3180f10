"""Compiles the CUDA sources of this package into libvitb200.so (sm_100a only).

nvcc cross-compiles without a GPU.  The library is kept in-tree, next to this
file, so a checkout that is copied to a GPU machine carries it along.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY = os.path.join(HERE, "libvitb200.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
    "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
]


def sources():
    return sorted(glob.glob(os.path.join(HERE, "csrc", "*.cu")))


def stale():
    if not os.path.exists(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    inputs = sources() + glob.glob(os.path.join(HERE, "csrc", "*.h")) + \
        glob.glob(os.path.join(HERE, "csrc", "*.cuh")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return any(os.path.getmtime(path) > built for path in inputs)


def build(force=False, verbose=False):
    if not force and not stale():
        return LIBRARY
    flags = list(NVCC_FLAGS)
    if verbose:
        flags += ["-Xptxas", "-v"]
    objects = []
    jobs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for source in sources():
        obj = os.path.join(HERE, "build",
                           os.path.basename(source)[:-3] + ".o")
        objects.append(obj)
        command = ["nvcc", *[f for f in flags if f != "-shared"], "-c",
                   source, "-o", obj]
        jobs.append(subprocess.Popen(command))
    failed = [job for job in jobs if job.wait() != 0]
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIBRARY, *objects, "-lcudart",
                    "-ldl"], check=True)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
