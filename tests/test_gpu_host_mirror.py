"""Runs the reference's hgemm tests restated in C++ against the host mirror
(moondream-zig_b200/host/moondream.hpp), i.e. through hgemm::matmul / hgemm_trans::matmul /
attention::* / rope::* with the reference's names and error behaviour."""
import os
import subprocess

import pytest

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu


def test_cpp_mirror_runs_reference_matmul_tests():
    exe = entry.build_cpp_tests()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all ok" in r.stdout
    assert r.stdout.count("ok ") >= 20
