"""The hand-out of device work counters to staged launches (tt-buda_b200/csrc/work_slots.hpp) is plain C++:
compiled here with a fake completion backend and run on the CPU."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_work_slot_ring_never_shares_a_busy_slot(tmp_path):
    exe = str(tmp_path / "work_slots_test")
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX", "CFLAGS", "CXXFLAGS")}
    subprocess.run(["g++", "-std=c++17", "-O1", "-pthread", "-I", os.path.join(ROOT, "tt-buda_b200", "csrc"),
                    os.path.join(ROOT, "tests", "cpp", "work_slots_test.cpp"), "-o", exe], check=True, env=env)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().endswith("ok")


def test_multiply_and_shift_division_matches_plain_division(tmp_path):
    """fast_div (work-item arithmetic of the general kernel flavour) for dividends below 2^31, compiled for the host."""
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    exe = str(tmp_path / "fast_div_test")
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX", "CFLAGS", "CXXFLAGS")}
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "tt-buda_b200", "csrc"), "-I", cuda_inc,
                    os.path.join(ROOT, "tests", "cpp", "fast_div_test.cpp"), "-o", exe], check=True, env=env)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.startswith("ok"), r.stdout + r.stderr
