"""A few training steps on one GPU, with whatever VITB200_* switches the
environment of this process carries (started by tests/test_switches_gpu.py).

argv: output.npz steps.  Tensor-core products are forced on so that the
tcgen05 product kernel is among the kernels the switches act on.  Writes the
per-step losses and the final weights.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from conftest import HOST_LIBRARY, PACKAGE, load_module  # noqa: E402

CONFIG = (1, 28, 28, 4, 64, 4, 2, 11)
BATCH = 64


def main():
    output, steps = sys.argv[1], int(sys.argv[2])
    vh = load_module("vitb200_vit_host", os.path.join(PACKAGE, "vit_host.py"))
    host_lib = vh.load_host_library(HOST_LIBRARY)
    backend = vh.Backend()
    backend.set_gemm_precision(2)
    backend.enable()
    host = vh.VitHost(host_lib, CONFIG, BATCH)
    losses = []
    for step in range(steps):
        images, labels = vh.synthetic_batch(BATCH, 28, 28, 11, 900 + step)
        losses.append(host.train_step(images, labels, 1e-3, 0.05, None, 0.1))
    arrays = {"w/" + name: value for name, value in host.parameters(0).items()}
    arrays["losses"] = np.asarray(losses, dtype=np.float64)
    arrays["launches"] = np.asarray([backend.kernel_launches()], dtype=np.int64)
    arrays["status"] = np.asarray([backend.tensor_core_status()], dtype=np.int64)
    assert backend.declined_ops() == 0
    np.savez(output, **arrays)
    host.close()
    backend.disable()
    backend.close()


if __name__ == "__main__":
    main()
