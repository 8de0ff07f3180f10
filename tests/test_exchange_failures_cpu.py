"""Failure detection for the gradient exchange, among CPU processes only.

A collective blocks until every rank takes part, so the cases a job can meet
(a rank that never starts, a rank that leaves between two steps, a rank that
stalls) are detected on the host, through a key/value store, before anything
is launched: ExchangeGroup in transformer-in-c_b200/vit_host.py.  These tests
run its ranks as separate processes over a torch.distributed TCPStore and
make the failures on the host: a process that never publishes, exits, or
sleeps.  No GPU, no NCCL, nothing that can hang a device."""
import datetime
import os
import socket
import subprocess
import sys
import time

import pytest

from conftest import PACKAGE

RANK = r"""
import datetime, os, sys, time
import importlib.util
from torch.distributed import TCPStore
spec = importlib.util.spec_from_file_location("vit_host", os.path.join(sys.argv[1], "vit_host.py"))
vh = importlib.util.module_from_spec(spec); spec.loader.exec_module(vh)
rank, world, port, scenario = int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
store = TCPStore("127.0.0.1", port, world_size=None, is_master=(rank == 0),
                 timeout=datetime.timedelta(seconds=20), wait_for_workers=False)
group = vh.ExchangeGroup(store, rank, world, timeout=2.0)
try:
    if scenario == "silent_root" and rank == 0:
        time.sleep(4.0)                      # never publishes the id
        print("RESULT idle"); sys.exit(0)
    if scenario == "missing_rank" and rank == world - 1:
        print("RESULT absent"); sys.exit(0)  # never joins
    unique_id = group.rendezvous(lambda: bytes(range(128)))
    assert unique_id == bytes(range(128))
    for step in range(1, 6):
        group.before_step(step)
        time.sleep(0.02)                     # the step itself
        if scenario == "leaves" and rank == 1 and step == 2:
            group.leave()                    # between steps, nothing in flight
            print("RESULT left"); sys.exit(0)
        if scenario == "stalls" and rank == 1 and step == 2:
            time.sleep(5.0)                  # stops making progress
            print("RESULT stalled"); sys.exit(0)
    print("RESULT finished")
except vh.ExchangeError as error:
    print("RESULT error:", error)
if rank == 0:
    time.sleep(1.0)                          # keep the store up for the others
"""


def free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def run_ranks(world, scenario):
    port = free_port()
    children = []
    for rank in range(world):
        children.append(subprocess.Popen(
            [sys.executable, "-c", RANK, PACKAGE, str(rank), str(world), str(port),
             scenario], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
        if rank == 0:
            time.sleep(0.5)   # the store's server side first
    results = []
    try:
        for child in children:
            out, err = child.communicate(timeout=60)
            lines = [l for l in out.splitlines() if l.startswith("RESULT")]
            results.append(lines[-1] if lines else "RESULT crashed: " + err[-300:])
    finally:
        for child in children:
            if child.poll() is None:
                child.kill()
                child.wait()
    return results


def test_all_ranks_present_run_to_the_end():
    assert run_ranks(3, "healthy") == ["RESULT finished"] * 3


def test_a_root_that_never_publishes_the_id_times_the_others_out():
    results = run_ranks(2, "silent_root")
    assert results[0] == "RESULT idle"
    assert "never published the exchange id" in results[1]


def test_a_rank_that_never_joins_is_named_before_any_collective():
    results = run_ranks(3, "missing_rank")
    assert results[2] == "RESULT absent"
    for line in results[:2]:
        assert "not every rank joined" in line and "joined/2" in line


def test_a_rank_that_leaves_between_steps_stops_the_others_before_their_next_launch():
    results = run_ranks(3, "leaves")
    assert results[1] == "RESULT left"
    for line in (results[0], results[2]):
        assert "rank 1 has left the exchange" in line


def test_a_rank_that_stalls_is_reported_with_the_step_it_was_last_seen_at():
    results = run_ranks(2, "stalls")
    assert "rank 1 has not reached step" in results[0]
    assert "last seen at step 2" in results[0] or "last seen at step 3" in results[0]
