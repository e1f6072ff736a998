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


@pytest.fixture(scope="module")
def stress_binary(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    out = str(tmp_path_factory.mktemp("tsan") / "protocol_stress")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-I", CSRC, "-I", cuda_inc,
           os.path.join(ROOT, "tests", "native", "protocol_stress.cpp"),
           os.path.join(CSRC, "symm", "host_backend.cpp"), os.path.join(CSRC, "oracle", "cpu_reference.cpp"),
           "-o", out, "-lpthread", "-lrt"]
    built = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    if built.returncode != 0:
        pytest.skip("ThreadSanitizer build not available here: " + built.stderr[-300:])
    return out


@pytest.mark.parametrize("world_size,iters", [(2, 400), (4, 200), (8, 60)])
def test_protocols_are_race_free_under_tsan(stress_binary, world_size, iters):
    run = subprocess.run([stress_binary, str(world_size), str(iters)], capture_output=True, text=True, timeout=600,
                         env={**os.environ, "TSAN_OPTIONS": "halt_on_error=0 exitcode=66"})
    assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[-2000:]
    assert run.returncode == 0, (run.returncode, run.stdout[-500:], run.stderr[-500:])
    assert "failures=0" in run.stdout
