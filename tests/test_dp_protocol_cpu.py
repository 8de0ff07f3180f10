"""World-size-2 check of the data-parallel protocol on CPU (gloo).

What the GPU backend does between ranks is: sum the shard gradients, fold
1/world into the clip scale, apply the same AdamW on every rank.  Here two
gloo processes run the reference's own CPU code (oracle/_ref/libvithost.so) on
their shards, exchange gradients with torch.distributed, apply the oracle's
clip + AdamW with that scaling, and must reproduce what the reference's
vit_model_train_batch_smoothed does on the whole batch in one process.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from conftest import HOST_LIBRARY, PACKAGE, REPO, load_module  # noqa: E402

CONFIG = (1, 28, 28, 7, 16, 2, 2, 11)
GLOBAL_BATCH, LR, WD, SMOOTHING = 6, 1e-3, 0.05, 0.1


def _free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _rank(rank, world, port, directory):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, REPO)
    from oracle import vit_oracle as vo
    vh = load_module("vitb200_vit_host", os.path.join(PACKAGE, "vit_host.py"))
    lib = vh.load_host_library(HOST_LIBRARY)
    images, labels = vh.synthetic_batch(GLOBAL_BATCH, 28, 28, 11, 33)
    shard = GLOBAL_BATCH // world
    rows = slice(rank * shard, (rank + 1) * shard)
    host = vh.VitHost(lib, CONFIG, shard)
    loss = host.gradients(images[rows], labels[rows], None, SMOOTHING)
    grads = host.parameters(1)
    names = vo.parameter_names(CONFIG[6])
    for name in names:                      # the one exchange step
        tensor = torch.from_numpy(grads[name])
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
    inverse_world = np.float32(1.0 / world)
    clip, _ = vo.clip_scale([grads[n] * inverse_world for n in names], vo.CLIP_NORM)
    scale = np.float32(clip) * inverse_world   # what the optimiser kernel multiplies by
    params = host.parameters(0)
    updated = {}
    for name in names:
        updated[name], _, _ = vo.adamw_update(
            params[name], grads[name] * scale, np.zeros_like(params[name]),
            np.zeros_like(params[name]), 1, LR, WD if vo.decays(name) else 0.0)
    total = torch.tensor([loss], dtype=torch.float64)
    dist.all_reduce(total)
    np.savez(os.path.join(directory, f"rank{rank}.npz"),
             loss=total.item() / world, **updated)
    host.close()
    dist.destroy_process_group()


@pytest.mark.skipif(not os.path.exists(HOST_LIBRARY),
                    reason="oracle/_ref/libvithost.so not built")
def test_sharded_gradients_reproduce_the_full_batch_step(tmp_path):
    world = 2
    mp.spawn(_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world,
             join=True)
    vh = load_module("vitb200_vit_host", os.path.join(PACKAGE, "vit_host.py"))
    lib = vh.load_host_library(HOST_LIBRARY)
    images, labels = vh.synthetic_batch(GLOBAL_BATCH, 28, 28, 11, 33)
    whole = vh.VitHost(lib, CONFIG, GLOBAL_BATCH)
    loss = whole.train_step(images, labels, LR, WD, None, SMOOTHING)
    expected = whole.parameters(0)
    whole.close()
    ranks = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    assert abs(float(ranks[0]["loss"]) - loss) <= 1e-5
    for name, value in expected.items():
        np.testing.assert_array_equal(ranks[0][name], ranks[1][name])
        keep = np.ones(value.shape[1], bool)
        if name.endswith("query_key_value_bias"):
            keep[16:32] = False  # key bias: zero gradient, rounding noise only
        np.testing.assert_allclose(ranks[0][name][:, keep], value[:, keep],
                                   rtol=0, atol=2e-5, err_msg=name)
