"""Checkpoints of device-resident models: the reference's own writer and reader
(vit_model_save / vit_model_load, src/vit.c:1203-1259) working on tensor memory
whose contents live on the device, and the direct device <-> file path
(vitb200_checkpoint_save / _load), whose files must be byte-identical to the
reference's.  The program is tests/checkpoint_roundtrip.c, built by
oracle/build_ref.py against the reference's sources and libvitb200.so."""
import os
import subprocess

import pytest

from conftest import REPO

pytestmark = pytest.mark.gpu

BINARY = os.path.join(REPO, "oracle", "_ref", "checkpoint_roundtrip")


@pytest.mark.skipif(not os.path.exists(BINARY), reason="run oracle/build_ref.py first")
def test_checkpoint_round_trip_through_the_reference_writer(tmp_path):
    done = subprocess.run([BINARY, str(tmp_path / "model.ckpt")],
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr + done.stdout
    assert "checkpoint_roundtrip: ok" in done.stdout
