"""One rank of a data-parallel run (started by tests/test_dp_gpu.py).

argv: rank world directory steps [micro_batches].  Rank r trains on its
contiguous shard of a fixed global batch with the backend on GPU r, in
`micro_batches` passes per optimiser step when given (gradient accumulation);
the NCCL id travels through a file in `directory`.  Writes the final parameters and per-step losses to
directory/rank<r>.npz.  world = 1 is the single-GPU yardstick on the whole batch.
"""
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from conftest import HOST_LIBRARY, PACKAGE, load_module  # noqa: E402

CONFIG = (1, 28, 28, 4, 32, 4, 2, 11)
GLOBAL_BATCH = 8


def main():
    rank, world, directory, steps = (int(sys.argv[1]), int(sys.argv[2]),
                                     sys.argv[3], int(sys.argv[4]))
    micro_batches = int(sys.argv[5]) if len(sys.argv) > 5 else 1
    os.environ["VITB200_DEVICE"] = str(rank)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    vh = load_module("vitb200_vit_host", os.path.join(PACKAGE, "vit_host.py"))
    host_lib = vh.load_host_library(HOST_LIBRARY)
    backend = vh.Backend()
    backend.set_gemm_precision(1)  # FP32: the comparison is about the exchange
    if world > 1:
        id_path = os.path.join(directory, "nccl_id")
        if rank == 0:
            with open(id_path + ".tmp", "wb") as handle:
                handle.write(backend.dp_unique_id())
            os.rename(id_path + ".tmp", id_path)
        deadline = time.time() + 60
        while not os.path.exists(id_path):
            if time.time() > deadline:
                raise RuntimeError("rank 0 never published the NCCL id")
            time.sleep(0.05)
        backend.dp_init(rank, world, open(id_path, "rb").read())
    backend.enable()
    images, labels = vh.synthetic_batch(GLOBAL_BATCH, 28, 28, 11, 21)
    shard = GLOBAL_BATCH // world
    images = images[rank * shard:(rank + 1) * shard]
    labels = labels[rank * shard:(rank + 1) * shard]
    if micro_batches > 1:
        backend.set_gradient_accumulation(micro_batches)
        model = vh.VitHost(host_lib, CONFIG, shard // micro_batches)
        images = np.ascontiguousarray(images)
        labels = np.ascontiguousarray(labels)
        losses = [model.train_step_accumulated(images, labels, micro_batches,
                                               1e-3, 0.05, None, 0.1)
                  for _ in range(steps)]
    else:
        model = vh.VitHost(host_lib, CONFIG, shard)
        losses = [model.train_step(images, labels, 1e-3, 0.05, None, 0.1)
                  for _ in range(steps)]
    out = {"losses": np.array(losses)}
    for name, value in model.parameters(0).items():
        out["w/" + name] = value
    counters = backend.dp_counters()
    out["overlapped"] = counters["overlapped_tensors"]
    out["late"] = counters["late_tensors"]
    out["flat_ranges"] = counters["flat_ranges"]
    np.savez(os.path.join(directory, f"rank{rank}.npz"), **out)
    model.close()
    backend.disable()
    backend.dp_shutdown()
    backend.close()


if __name__ == "__main__":
    main()
