"""Writes the golden fixtures in this directory by running the REFERENCE's own
compiled CPU code (oracle/_ref/libvithost.so: the reference's ops.c / vit.c /
autodiff.c, no device backend installed) on seeded synthetic inputs.

Run here, where the reference tree is mounted:

    python oracle/build_ref.py && python tests/golden/make_golden.py

Each fixture stores the case description (enough to regenerate the inputs),
the initial parameters produced by vit_model_init_seeded, and the reference's
outputs: loss, every parameter gradient (before the optimiser step), and the
parameters and Adam moments after N calls to vit_model_train_batch_smoothed
with the per-step losses.  Cases are small so the files stay a few hundred KB.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
sys.path.insert(0, os.path.join(REPO, "tests"))
from conftest import HOST_LIBRARY, PACKAGE, load_module  # noqa: E402

# name: (config (c,h,w,patch,d,heads,layers,classes), batch, seed, steps,
#        label smoothing, class weights?)
CASES = {
    "tiny_p7_d16": ((1, 28, 28, 7, 16, 2, 2, 11), 3, 7, 3, 0.1, False),
    "p4_d32_h4_l2": ((1, 28, 28, 4, 32, 4, 2, 11), 4, 11, 2, 0.1, True),
    "p14_d8_h1_c5": ((1, 28, 28, 14, 8, 1, 1, 5), 2, 3, 2, 0.0, False),
}
LEARNING_RATE, WEIGHT_DECAY = 1e-3, 0.05


def class_weights(classes):
    return (0.5 + 0.1 * np.arange(classes)).astype(np.float32)


def main():
    vh = load_module("vitb200_vit_host", os.path.join(PACKAGE, "vit_host.py"))
    lib = vh.load_host_library(HOST_LIBRARY)
    for name, (config, batch, seed, steps, smoothing, weighted) in CASES.items():
        images, labels = vh.synthetic_batch(batch, config[1], config[2],
                                            config[7], seed)
        weights = class_weights(config[7]) if weighted else None
        host = vh.VitHost(lib, config, batch, seed=42)
        out = {"config": np.array(config), "batch": batch, "seed": seed,
               "steps": steps, "label_smoothing": smoothing,
               "weighted": int(weighted), "images": images,
               "labels": labels.astype(np.int64)}
        for k, v in host.parameters(0).items():
            out["init/" + k] = v
        out["loss"] = host.gradients(images, labels, weights, smoothing)
        out["logits"] = host.forward(images)
        for k, v in host.parameters(1).items():
            out["grad/" + k] = v
        losses = [host.train_step(images, labels, LEARNING_RATE, WEIGHT_DECAY,
                                  weights, smoothing) for _ in range(steps)]
        out["step_losses"] = np.array(losses, np.float32)
        for what, tag in ((0, "after/"), (2, "m/"), (3, "v/")):
            for k, v in host.parameters(what).items():
                out[tag + k] = v
        host.close()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(name, "loss", out["loss"], "losses", losses,
              os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
