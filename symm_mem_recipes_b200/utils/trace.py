"""NVTX ranges around the public ops, for timelines taken with an external
profiler (upstream's only instrumentation is `torch.profiler` inside its
benchmark helpers, symm_mem_recipes/utils.py:46-52, and a Triton launch-metadata
hook, triton_all_gather_matmul.py:59-69).

Off by default and then free of cost: `traced(name)` returns the function it is
given.  `SMR_NVTX=1` in the environment at import time turns every decorated op
into `range_push(name + shape summary) ... range_pop()`.
"""
from __future__ import annotations

import functools
import os
from contextlib import contextmanager
from typing import Callable

import torch

ENABLED = os.environ.get("SMR_NVTX", "") == "1"


def _push(msg: str) -> None:
    torch.cuda.nvtx.range_push(msg)


def _pop() -> None:
    torch.cuda.nvtx.range_pop()


@contextmanager
def nvtx_range(name: str, enabled: bool | None = None):
    """`with nvtx_range("phase"):`; a no-op unless enabled (argument, else SMR_NVTX=1)."""
    on = ENABLED if enabled is None else enabled
    if on:
        _push(name)
    try:
        yield
    finally:
        if on:
            _pop()


def _describe(args) -> str:
    shapes = [f"{tuple(a.shape)}" for a in args if isinstance(a, torch.Tensor)]
    return " ".join(shapes[:3])


def traced(name: str, enabled: bool | None = None) -> Callable:
    """Decorator: an NVTX range named `name` plus the shapes of the first tensor arguments."""
    on = ENABLED if enabled is None else enabled

    def wrap(fn):
        if not on:
            return fn

        @functools.wraps(fn)
        def inner(*args, **kwargs):
            _push(f"{name} {_describe(args)}")
            try:
                return fn(*args, **kwargs)
            finally:
                _pop()
        return inner
    return wrap
