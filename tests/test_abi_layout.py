"""The backend is built without the host's headers; this test compiles one
translation unit that includes both and lets the compiler compare layouts."""
import os
import subprocess

import pytest

from conftest import REPO

REFERENCE_INCLUDE = "/root/reference/include"


@pytest.mark.skipif(not os.path.isdir(REFERENCE_INCLUDE),
                    reason="reference headers not present on this machine")
def test_mirrored_structs_match_host_headers(tmp_path):
    binary = tmp_path / "abi_layout_check"
    subprocess.run(
        ["gcc", "-std=c11", "-Wall", "-Werror", "-I" + REFERENCE_INCLUDE,
         "-I" + os.path.join(REPO, "include"),
         os.path.join(REPO, "tests", "abi_layout_check.c"), "-o", str(binary)],
        check=True)
    assert subprocess.run([str(binary)]).returncode == 0
