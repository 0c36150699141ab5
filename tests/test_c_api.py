"""The C interface of the host core from a C program (no Python in that process)."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs a C compiler")
def test_c_program_drives_engine_and_scheduler(tmp_path):
    from ccinfer_b200.csrc import build
    lib = build.library_path("host")
    exe = str(tmp_path / "check")
    inc = os.path.join(os.path.dirname(os.path.abspath(build.__file__)), "host")
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-I", inc, os.path.join(HERE, "c_api", "check.c"),
                    lib, "-Wl,-rpath," + os.path.dirname(lib), "-o", exe], check=True)
    out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    assert out.startswith("ok steps ")
    figures = dict(zip(out.split()[1::2], out.split()[2::2]))
    assert int(figures["preemptions"]) > 0        # 14 pages of 4 tokens do not hold five requests at once
    assert int(figures["steps"]) > 20
