"""Helpers for multi-rank tests: run a function as N ranks of one host.

CPU tests use backend "gloo"; GPU tests use "nccl" with one GPU per rank.  The
rendezvous address is always 127.0.0.1.
"""
from __future__ import annotations

import os
import signal
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    """A port that is free now, drawn at random from a range the kernel does
    not hand out as ephemeral ports (so nothing grabs it before rank 0 binds)."""
    import random

    for _ in range(64):
        port = random.randint(20000, 29999)
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            try:
                s.bind(("127.0.0.1", port))
                return port
            except OSError:
                continue
    raise RuntimeError("no free port found")


def _entry(rank: int, world_size: int, backend: str, port: int, fn, args, errq):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["LOCAL_RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world_size)

    # A rank that the parent gives up on is asked to stop with SIGTERM: leave through the `finally`
    # below (orderly unbinding of multicast memory) instead of dying with its mappings in place.
    # The teardown itself may wait for peers that are gone (a process-group shutdown can retry for
    # minutes), so an alarm ends the process if it has not left within 20 s.
    def _on_sigterm(signum, frame):
        signal.alarm(20)
        raise SystemExit(143)

    signal.signal(signal.SIGTERM, _on_sigterm)
    ok = False
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world_size,
                                    device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group(backend, rank=rank, world_size=world_size)
        fn(rank, world_size, *args)
        ok = True
    except BaseException:  # noqa: BLE001 - reported to the parent
        errq.put((rank, traceback.format_exc()))
    finally:
        # Orderly teardown even after a failure: every rank unbinds its
        # multicast memory only after meeting the others (or a short timeout).
        try:
            from symm_mem_recipes_b200.parallel import symm_mem
            symm_mem.shutdown()
        except BaseException:  # noqa: BLE001
            if ok:
                errq.put((rank, traceback.format_exc()))
        try:
            dist.destroy_process_group()
        except BaseException:  # noqa: BLE001
            pass


def spawn_ranks(fn, world_size: int, backend: str = "gloo", args=(), timeout_s: float = 300.0) -> None:
    """Run `fn(rank, world_size, *args)` in `world_size` fresh processes and
    raise in the parent if any rank failed or the deadline passed."""
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world_size, backend, port, fn, args, errq))
             for r in range(world_size)]
    import time

    for p in procs:
        p.start()
    deadline = time.monotonic() + timeout_s
    while time.monotonic() < deadline and any(p.is_alive() for p in procs):
        if any(p.exitcode not in (0, None) for p in procs):
            # a rank died: give the others a moment to notice, then stop waiting
            deadline = min(deadline, time.monotonic() + 30.0)
        time.sleep(0.05)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
    for p in hung:
        p.join(30)        # bounded device waits end within their timeout, then the rank tears down in order
        if p.is_alive():
            p.kill()
            p.join(10)
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    if hung:
        errors.append((-1, f"{len(hung)} rank(s) did not finish within {timeout_s} s"))
    bad_exit = [(i, p.exitcode) for i, p in enumerate(procs) if p.exitcode not in (0, None)]
    if errors or bad_exit:
        msg = "\n".join(f"--- rank {r} ---\n{tb}" for r, tb in errors)
        raise RuntimeError(f"rank failure(s); exit codes {bad_exit}\n{msg}")


def seeded_normal_bf16(numel: int, rank: int, device="cpu", std: float = 1.0, seed: int = 42) -> torch.Tensor:
    """bf16 N(0, std) values that depend only on (seed, rank): every process
    can regenerate any rank's input (upstream seeds with 42 + rank,
    symm_mem_recipes/triton_all_gather_matmul.py:364)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed + rank)
    t = (torch.randn(numel, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)
    return t.to(device)


def guarded_empty(shape, dtype: torch.dtype, device, guard_bytes: int = 4096, fill: int = 0xA5):
    """An output buffer between two canary regions.  Returns `(tensor, intact)`:
    `tensor` is contiguous, 256-byte aligned and filled with the canary pattern
    too (every element must be overwritten by the op under test); `intact()`
    is true while no byte of the guard regions before and after it has changed.
    Stands in for a memory checker in the kernel tests: a store past either end
    of the output shows up on the host."""
    numel = 1
    for s in shape:
        numel *= int(s)
    nbytes = numel * dtype.itemsize
    assert guard_bytes % 256 == 0
    raw = torch.full((guard_bytes + (nbytes + 255) // 256 * 256 + guard_bytes,), fill, dtype=torch.uint8,
                     device=device)
    tensor = raw[guard_bytes:guard_bytes + nbytes].view(dtype).view(*shape)

    def intact() -> bool:
        front = bool((raw[:guard_bytes] == fill).all())
        back = bool((raw[guard_bytes + nbytes:] == fill).all())
        return front and back

    return tensor, intact
