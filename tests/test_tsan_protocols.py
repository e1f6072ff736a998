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


def _build(tmp_path_factory, sanitizers: str, program: str = "protocol_stress") -> str:
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    out = str(tmp_path_factory.mktemp("san") / program)
    cmd = ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizers}", "-fno-sanitize-recover=all", "-I", CSRC,
           "-I", cuda_inc,
           os.path.join(ROOT, "tests", "native", program + ".cpp"),
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


@pytest.fixture(scope="module")
def fused_stress_binary(tmp_path_factory):
    return _build(tmp_path_factory, "thread", "fused_protocol_stress")


@pytest.mark.parametrize("world_size,ctas,calls", [(2, 3, 200), (4, 3, 100), (8, 2, 40)])
def test_fused_kernel_protocol_is_race_free_under_tsan(fused_stress_binary, world_size, ctas, calls):
    """Arrival counters that count calls, the call number published by the last CTA, the entry
    barrier per CTA index: the protocol of matmul_reduce_scatter and of the push gather, one
    thread per CTA."""
    run = subprocess.run([fused_stress_binary, str(world_size), str(ctas), str(calls)], capture_output=True,
                         text=True, timeout=600, env={**os.environ, "TSAN_OPTIONS": "halt_on_error=0 exitcode=66"})
    assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[-2000:]
    assert run.returncode == 0 and "failures=0" in run.stdout, (run.returncode, run.stdout[-500:])


def test_fused_kernel_protocol_needs_its_entry_barrier(fused_stress_binary):
    """Without the entry barrier a rank's stores of call n + 1 race with a slower rank's reads of
    call n: the model must show it (so a clean run above means something)."""
    run = subprocess.run([fused_stress_binary, "4", "3", "150", "no-entry-barrier"], capture_output=True, text=True,
                         timeout=600, env={**os.environ, "TSAN_OPTIONS": "halt_on_error=0 exitcode=66"})
    assert "WARNING: ThreadSanitizer: data race" in run.stderr or "failures=0" not in run.stdout


@pytest.mark.parametrize("world_size,tiles,calls", [(2, 3, 300), (4, 2, 150), (8, 2, 40)])
def test_gemv_exchange_is_race_free_under_tsan(fused_stress_binary, world_size, tiles, calls):
    """The barrier-free exchange of the fused GEMV + all-reduce: partials into the half of the inbox
    chosen by the parity of the call number, the call number as the flag."""
    run = subprocess.run([fused_stress_binary, str(world_size), str(tiles), str(calls), "gemv"], capture_output=True,
                         text=True, timeout=600, env={**os.environ, "TSAN_OPTIONS": "halt_on_error=0 exitcode=66"})
    assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[-2000:]
    assert run.returncode == 0 and "failures=0" in run.stdout, (run.returncode, run.stdout[-500:])


def test_gemv_exchange_needs_both_halves(fused_stress_binary):
    """With one half a rank that is a call ahead overwrites partials a slower rank still reads."""
    run = subprocess.run([fused_stress_binary, "4", "2", "100", "gemv-one-parity"], capture_output=True, text=True,
                         timeout=600, env={**os.environ, "TSAN_OPTIONS": "halt_on_error=0 exitcode=66"})
    assert "WARNING: ThreadSanitizer: data race" in run.stderr or "failures=0" not in run.stdout
