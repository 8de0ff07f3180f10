"""The launch-level mechanisms of the backend can each be turned off through
the environment (read once per process, hence child processes): chained
launches (programmatic dependent launch) and the batched zero fill of the small
gradients.  Neither may change what is computed: the same training run with either switched
off gives the same losses (to the order of the float atomics, 2e-5 relative)
and the same weights (5e-3 of the largest entry after Adam's amplification of
rounding noise; the key bias, whose exact gradient is zero, left out)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import REPO

pytestmark = pytest.mark.gpu
WORKER = os.path.join(REPO, "tests", "switch_worker.py")
STEPS = 4
D_MODEL = 64


def run(path, **switches):
    environment = dict(os.environ)
    environment.update(switches)
    subprocess.run([sys.executable, WORKER, path, str(STEPS)], check=True,
                   env=environment, timeout=300)
    return np.load(path)


@pytest.fixture(scope="module")
def reference_run(tmp_path_factory):
    return run(str(tmp_path_factory.mktemp("switches") / "default.npz"))


@pytest.mark.parametrize("switches", [
    {"VITB200_CHAINED_LAUNCHES": "0"},
    {"VITB200_NO_BATCHED_ZERO_FILL": "1"},
    {"VITB200_CHAINED_LAUNCHES": "0", "VITB200_NO_BATCHED_ZERO_FILL": "1"},
], ids=["plain-launches", "memset-nodes", "both"])
def test_switching_a_mechanism_off_changes_no_result(reference_run, switches,
                                                     tmp_path):
    other = run(str(tmp_path / "other.npz"), **switches)
    assert int(other["status"][0]) == 0 and int(reference_run["status"][0]) == 0
    np.testing.assert_allclose(other["losses"], reference_run["losses"],
                               rtol=2e-5, atol=0)
    assert len(set(reference_run["losses"].tolist())) == STEPS
    for name in reference_run.files:
        if not name.startswith("w/"):
            continue
        ours, theirs = other[name], reference_run[name]
        if name.endswith("query_key_value_bias"):
            keep = np.ones(ours.shape[1], bool)
            keep[D_MODEL:2 * D_MODEL] = False
            ours, theirs = ours[:, keep], theirs[:, keep]
        scale = max(float(np.abs(theirs).max()), 1e-6)
        assert float(np.abs(ours - theirs).max()) / scale <= 5e-3, name
    if "VITB200_NO_BATCHED_ZERO_FILL" in switches:
        # Two launches per step fewer: the fills of the parameter list and of
        # the activation-gradient list.
        assert int(other["launches"][0]) < int(reference_run["launches"][0])
