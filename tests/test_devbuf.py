"""The library's device-buffer handle keeps `p == nullptr <=> bytes == 0`, also after a failed allocation, so that no
growth guard can skip a needed allocation and pass a null pointer to a kernel.  Checked on the host with an allocator
that fails on demand (tests/devbuf_check.cpp); nothing here touches a GPU."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_devbuf_invariant_after_failed_allocation(tmp_path):
    exe = tmp_path / "devbuf_check"
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "thrml-rs_b200", "csrc"),
                    os.path.join(ROOT, "tests", "devbuf_check.cpp"), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stdout + out.stderr


def test_no_growth_guard_tests_bytes_alone():
    """Guards must go through DevBuf::holds / reserve (which test the pointer too)."""
    csrc = os.path.join(ROOT, "thrml-rs_b200", "csrc")
    for name in os.listdir(csrc):
        text = open(os.path.join(csrc, name)).read()
        assert ".bytes <" not in text and ".bytes >=" not in text, name
