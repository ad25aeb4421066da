"""A plain-C program links liboptengine.so and drives the path with no Python in between."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_c_client_runs(tmp_path):
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    lib_dir = os.path.join(ROOT, "gograd_b200")
    exe = tmp_path / "c_client"
    subprocess.run([cc, "-std=c11", "-Wall", "-Wextra", os.path.join(lib_dir, "csrc", "examples", "c_client.c"),
                    "-I", os.path.join(ROOT, "include"), "-L", lib_dir, "-loptengine", f"-Wl,-rpath,{lib_dir}", "-lm",
                    "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert "c_client ok" in out.stdout


def test_c_step_rate_runs(tmp_path):
    """Eager steps issued from C: one launch per step, and the program reports what a step costs
    without an interpreter in between (a few microseconds; the bound asserted here is loose)."""
    import re
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    lib_dir = os.path.join(ROOT, "gograd_b200")
    exe = tmp_path / "c_step_rate"
    subprocess.run([cc, "-std=gnu11", "-Wall", "-Wextra", os.path.join(lib_dir, "csrc", "examples", "c_step_rate.c"),
                    "-I", os.path.join(ROOT, "include"), "-L", lib_dir, "-loptengine", f"-Wl,-rpath,{lib_dir}", "-lm",
                    "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    print(out.stdout)
    found = re.search(r"host issue ([0-9.]+) us/step, with the device drained ([0-9.]+) us/step", out.stdout)
    assert found, out.stdout
    assert float(found.group(2)) < 100.0


def test_c_zero1_runs(tmp_path):
    """The sharded step driven from one plain-C process over every GPU of the box (one rank with a single
    GPU): one oe_zero1_adamw_step call per rank and step, no collective library, results equal to the
    host loop written out in the same file, bit for bit."""
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    lib_dir = os.path.join(ROOT, "gograd_b200")
    exe = tmp_path / "c_zero1"
    subprocess.run([cc, "-std=c11", "-O1", "-ffp-contract=off", "-Wall", "-Wextra",
                    os.path.join(lib_dir, "csrc", "examples", "c_zero1.c"), "-I", os.path.join(ROOT, "include"), "-L", lib_dir,
                    "-loptengine", f"-Wl,-rpath,{lib_dir}", "-lm", "-lpthread", "-o", str(exe)], check=True)
    for mode in ([], ["copies"]):   # "copies": staged gradient copies and a shadow copy, asked for explicitly
        out = subprocess.run([str(exe)] + mode, capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, f"mode {mode}: {out.stderr}"
        assert "c_zero1 ok" in out.stdout
