"""Builds the reference's own CPU implementation into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  Nothing here is part of the shipped library; the
outputs are used as the checker in tests/, __graft_entry__.smoke() and the
cpu_baseline / --impl reference legs of bench.py.

The reference sources are compiled where they lie (they are never copied into
this repository) with the flags of the reference Makefile:2
(-std=c99 -O2).  Outputs, all under oracle/_ref/ (git-ignored):

  libvithost.so   ops.c vit.c autodiff.c arena.c augmentation.c  +  our flat
                  ctypes-friendly entry points
                  (transformer-in-c_b200/host/vit_host.c): the CHECKER.  No
                  backend is ever installed into this copy; it is loaded
                  with local symbol scope and only runs the CPU loops.

The same sources are compiled a second time into
transformer-in-c_b200/host/libvithost.so: the CALLER, the unmodified host
program that drives the backend through the op table (what the reference's
own binaries are once they link the backend).  Both copies are linked with
-Bsymbolic, so each keeps its own op table and allocator hook when both are
loaded into one process and results of one can be checked against the other.

  test_device     the reference's CPU-vs-device acceptance test
                  (tests/test_device.c, -DENABLE_CUDA) linked against
                  libvitb200.so instead of the reference's cuda_backend.o
  test_vision     the reference's CPU unit tests (oracle sanity)
  checkpoint_roundtrip
                  tests/checkpoint_roundtrip.c (ours) on the reference's
                  vit_model_save / vit_model_load, linked like test_device

  libtrainer_pieces.so
                  tests/trainer_pieces.c (ours) around the reference's trainer
                  source and loader: shuffle, pixel statistics, normalisation
                  and vision_dataset_load_pgm_csv, the checker of the
                  device-resident dataset

  reference_cuda_step
                  oracle/reference_cuda_step.c (ours, a timing driver) with the
                  reference's own src/cuda_backend.cu compiled for sm_100a and
                  cuBLAS: the secondary GPU baseline of bench.py

The reference tree is looked for at the path given as argument, else in
$VITB200_REFERENCE_ROOT, else in a directory named `reference` next to this
repository.

Usage: python oracle/build_ref.py [reference_root]
"""
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OUT = os.path.join(REPO, "oracle", "_ref")
PACKAGE = os.path.join(REPO, "transformer-in-c_b200")
CORE = ["ops.c", "vit.c", "autodiff.c", "arena.c"]
EXTRA = ["dataset.c", "augmentation.c", "transformer.c"]  # test_vision needs them


def run(command):
    subprocess.run(command, check=True)


def default_reference_root():
    return os.environ.get("VITB200_REFERENCE_ROOT") or \
        os.path.join(os.path.dirname(REPO), "reference")


def build(reference_root=None):
    """Returns True when the outputs were (re)built, False when the reference
    tree is not present (the GPU box: prebuilt files are used as they are)."""
    reference_root = reference_root or default_reference_root()
    source = os.path.join(reference_root, "src")
    include = os.path.join(reference_root, "include")
    if not os.path.isdir(source):
        return False
    os.makedirs(OUT, exist_ok=True)
    flags = ["-std=c99", "-O2", "-fPIC", "-I" + include]
    core = [os.path.join(source, name) for name in CORE]
    for library in (os.path.join(OUT, "libvithost.so"),
                    os.path.join(PACKAGE, "host", "libvithost.so")):
        run(["gcc", *flags, "-shared", "-Wl,-Bsymbolic", "-o", library, *core,
             os.path.join(source, "augmentation.c"),
             os.path.join(PACKAGE, "host", "vit_host.c"), "-lm"])
    run(["gcc", *flags, "-o", os.path.join(OUT, "test_vision"),
         os.path.join(reference_root, "tests", "test_vision.c"), *core,
         *[os.path.join(source, name) for name in EXTRA], "-lm"])
    run(["gcc", *flags, "-w", "-shared", "-I" + os.path.join(reference_root, "examples"),
         "-o", os.path.join(OUT, "libtrainer_pieces.so"),
         os.path.join(REPO, "tests", "trainer_pieces.c"), *core,
         os.path.join(source, "dataset.c"),
         os.path.join(source, "augmentation.c"), "-lm"])
    library = os.path.join(PACKAGE, "libvitb200.so")
    if os.path.exists(library):
        run(["gcc", *flags, "-DENABLE_CUDA", "-o",
             os.path.join(OUT, "test_device"),
             os.path.join(reference_root, "tests", "test_device.c"), *core,
             "-L" + PACKAGE, "-lvitb200",
             "-Wl,-rpath,$ORIGIN/../../transformer-in-c_b200", "-lm"])
        run(["gcc", *flags, "-I" + os.path.join(REPO, "include"), "-o",
             os.path.join(OUT, "checkpoint_roundtrip"),
             os.path.join(REPO, "tests", "checkpoint_roundtrip.c"), *core,
             "-L" + PACKAGE, "-lvitb200",
             "-Wl,-rpath,$ORIGIN/../../transformer-in-c_b200", "-lm"])
    # The reference's CUDA backend, unmodified, for the same GPU.
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    if os.path.exists(nvcc):
        backend_object = os.path.join(OUT, "reference_cuda_backend.o")
        run([nvcc, "-O2", "-std=c++17", "-gencode",
             "arch=compute_100a,code=sm_100a", "-I" + include, "-c",
             os.path.join(source, "cuda_backend.cu"), "-o", backend_object])
        run(["gcc", *flags, "-DENABLE_CUDA", "-o",
             os.path.join(OUT, "reference_cuda_step"),
             os.path.join(REPO, "oracle", "reference_cuda_step.c"), *core,
             backend_object, "-L" + os.path.join(cuda_home, "lib64"),
             "-Wl,-rpath," + os.path.join(cuda_home, "lib64"),
             "-lcublas", "-lcudart", "-lstdc++", "-lm"])
    return True


if __name__ == "__main__":
    built = build(*sys.argv[1:2])
    print("built" if built else "reference tree not found; nothing built")
