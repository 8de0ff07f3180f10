"""The backend is built without the host's headers; this test compiles
translation units that include both and lets the compiler compare the
structures' layouts and every op slot's signature.

The host's headers are looked for in $VITB200_REFERENCE_ROOT/include, else in
a directory named `reference` next to this repository."""
import os
import subprocess

import pytest

from conftest import REPO

REFERENCE_INCLUDE = os.path.join(
    os.environ.get("VITB200_REFERENCE_ROOT") or
    os.path.join(os.path.dirname(REPO), "reference"), "include")

pytestmark = pytest.mark.skipif(
    not os.path.isdir(REFERENCE_INCLUDE),
    reason="reference headers not present on this machine")


def compile_and_run(tmp_path, source):
    binary = tmp_path / source[:-2]
    subprocess.run(
        ["gcc", "-std=gnu11", "-Wall", "-Werror", "-I" + REFERENCE_INCLUDE,
         "-I" + os.path.join(REPO, "include"),
         os.path.join(REPO, "tests", source), "-o", str(binary)],
        check=True)
    assert subprocess.run([str(binary)]).returncode == 0


def test_mirrored_structs_match_host_headers(tmp_path):
    compile_and_run(tmp_path, "abi_layout_check.c")


def test_op_slot_signatures_match_host_headers(tmp_path):
    compile_and_run(tmp_path, "abi_signature_check.c")
