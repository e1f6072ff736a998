"""ThreadSanitizer over the host builds of the cross-rank protocols.

compute-sanitizer's racecheck cannot follow accesses that cross GPUs, and the
upstream recipes rest on hand-chosen PTX qualifiers
(symm_mem_recipes/triton_barrier.py:112-139).  Here the same protocols, built
for the host with the same release / acquire placement, run with threads as
ranks under TSAN: a missing ordering is a reported race.
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "symm_mem_recipes_b200", "csrc")


def _build(tmp_path_factory, sanitizers: str) -> str:
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    out = str(tmp_path_factory.mktemp("san") / "protocol_stress")
    cmd = ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizers}", "-fno-sanitize-recover=all", "-I", CSRC,
           "-I", cuda_inc,
           os.path.join(ROOT, "tests", "native", "protocol_stress.cpp"),
           os.path.join(CSRC, "symm", "host_backend.cpp"), os.path.join(CSRC, "oracle", "cpu_reference.cpp"),
           "-o", out, "-lpthread", "-lrt"]
    built = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    if built.returncode != 0:
        pytest.skip(f"-fsanitize={sanitizers} build not available here: " + built.stderr[-300:])
    return out


@pytest.fixture(scope="module")
def stress_binary(tmp_path_factory):
    return _build(tmp_path_factory, "thread")


@pytest.fixture(scope="module")
def stress_binary_asan(tmp_path_factory):
    return _build(tmp_path_factory, "address,undefined")


@pytest.mark.parametrize("world_size,iters", [(2, 400), (4, 200), (8, 60)])
def test_protocols_are_race_free_under_tsan(stress_binary, world_size, iters):
    run = subprocess.run([stress_binary, str(world_size), str(iters)], capture_output=True, text=True, timeout=600,
                         env={**os.environ, "TSAN_OPTIONS": "halt_on_error=0 exitcode=66"})
    assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[-2000:]
    assert run.returncode == 0, (run.returncode, run.stdout[-500:], run.stderr[-500:])
    assert "failures=0" in run.stdout


def test_protocols_are_clean_under_asan_and_ubsan(stress_binary_asan):
    """Out-of-bounds slots or misaligned / overflowing arithmetic in the host builds would stop the run."""
    run = subprocess.run([stress_binary_asan, "4", "100"], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, (run.returncode, run.stdout[-500:], run.stderr[-2000:])
    assert "failures=0" in run.stdout and "ERROR: AddressSanitizer" not in run.stderr
    assert "runtime error" not in run.stderr
