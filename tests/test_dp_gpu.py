"""Data-parallel training on 2 GPUs against single-GPU training on the same
global batch: with gradients summed over ranks and the 1/world factor folded
into the clip scale, every rank must end with the weights a single GPU gets
(up to FP32 summation order), and all ranks must agree bit for bit."""
import os
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

from conftest import REPO

pytestmark = pytest.mark.gpu
WORKER = os.path.join(REPO, "tests", "dp_worker.py")
STEPS = 5


def run_world(world, directory, micro_batches=1):
    os.makedirs(directory, exist_ok=True)
    children = [subprocess.Popen([sys.executable, WORKER, str(rank), str(world),
                                  directory, str(STEPS), str(micro_batches)])
                for rank in range(world)]
    # All ranks are watched together: the first one that fails (or the
    # deadline) ends the others at once, so that no rank is left behind
    # blocked in a collective on a shared GPU after the test has gone.
    deadline = time.monotonic() + 300
    try:
        running = list(children)
        while running:
            for child in list(running):
                status = child.poll()
                if status is None:
                    continue
                assert status == 0, f"a rank exited with status {status}"
                running.remove(child)
            assert time.monotonic() < deadline, "ranks did not finish in 300 s"
            time.sleep(0.05)
    finally:
        for child in children:
            if child.poll() is None:
                child.kill()
        for child in children:
            child.wait()
    return [np.load(os.path.join(directory, f"rank{rank}.npz"))
            for rank in range(world)]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_match_one_gpu_on_the_same_global_batch(tmp_path):
    single = run_world(1, str(tmp_path / "single"))[0]
    ranks = run_world(2, str(tmp_path / "pair"))
    names = [k for k in single.files if k.startswith("w/")]
    for name in names:
        # identical reduced gradients and identical update rule on every rank
        np.testing.assert_array_equal(ranks[0][name], ranks[1][name])
        keep = np.ones(single[name].shape[-1], bool)
        if name.endswith("query_key_value_bias"):
            keep[32:64] = False  # key bias: zero gradient, rounding noise only
        np.testing.assert_allclose(ranks[0][name][..., keep],
                                   single[name][..., keep], rtol=0, atol=2e-4,
                                   err_msg=name)
    # the global loss is the mean of the shard losses
    np.testing.assert_allclose(
        (ranks[0]["losses"] + ranks[1]["losses"]) / 2, single["losses"],
        rtol=0, atol=1e-4)
    # from the third step on gradients are exchanged while backward still runs
    assert int(ranks[0]["overlapped"]) > 0
    assert int(ranks[0]["late"]) >= 2 * len(names)
    # and leave as a few contiguous ranges of one arena, not tensor by tensor
    assert 0 < int(ranks[0]["flat_ranges"]) <= 3 * (STEPS - 2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_accumulating_two_micro_batches_match_one_gpu(tmp_path):
    """Global batch 8 = 2 ranks x 2 micro-batches x 2 images: each gradient is
    exchanged once per optimiser step, after the second micro-batch has added
    to it, and 1 / (world x micro-batches) turns the sum into the mean."""
    single = run_world(1, str(tmp_path / "single"))[0]
    ranks = run_world(2, str(tmp_path / "pair"), micro_batches=2)
    names = [k for k in single.files if k.startswith("w/")]
    for name in names:
        np.testing.assert_array_equal(ranks[0][name], ranks[1][name])
        keep = np.ones(single[name].shape[-1], bool)
        if name.endswith("query_key_value_bias"):
            keep[32:64] = False
        np.testing.assert_allclose(ranks[0][name][..., keep],
                                   single[name][..., keep], rtol=0, atol=2e-4,
                                   err_msg=name)
    np.testing.assert_allclose(
        (ranks[0]["losses"] + ranks[1]["losses"]) / 2, single["losses"],
        rtol=0, atol=1e-4)
    # exactly one exchange per parameter and optimiser step (not one per
    # micro-batch), overlapped with backward once the schedule is known
    assert int(ranks[0]["overlapped"]) > 0
    assert int(ranks[0]["overlapped"]) + int(ranks[0]["late"]) == STEPS * len(names)
