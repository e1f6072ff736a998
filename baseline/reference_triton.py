"""Runs the upstream Triton one-shot all-reduce as a same-box baseline.

Baseline harness only: nothing in the product imports this file.  The upstream
sources are used unmodified from `baseline/_ref` (the offline pip install of
the reference); the only accommodation is a stub for the `expecttest` module
that `symm_mem_recipes/utils.py:7` pulls in through torch's test utilities and
that is not installed here.  The upstream all-gather matmul cannot be run this
way: it imports a Triton API that no longer exists.
"""
from __future__ import annotations

import os
import sys
import types
import unittest


def load_reference_one_shot():
    """Returns (one_shot_all_reduce, alloc) where `alloc(numel, device)` gives a
    bf16 tensor in torch's own symmetric memory, as the upstream driver does
    (symm_mem_recipes/triton_one_shot_all_reduce.py:141-151)."""
    here = os.path.dirname(os.path.abspath(__file__))
    ref = os.path.join(here, "_ref")
    if not os.path.isdir(os.path.join(ref, "symm_mem_recipes")):
        raise ImportError("baseline/_ref is not installed")
    if "expecttest" not in sys.modules:
        stub = types.ModuleType("expecttest")
        stub.TestCase = unittest.TestCase
        sys.modules["expecttest"] = stub
    if ref not in sys.path:
        sys.path.insert(0, ref)
    import torch
    import torch.distributed as dist
    from symm_mem_recipes.triton_one_shot_all_reduce import one_shot_all_reduce
    from torch._C._distributed_c10d import _SymmetricMemory
    from torch.distributed._symmetric_memory import enable_symm_mem_for_group

    group_name = dist.group.WORLD.group_name
    enable_symm_mem_for_group(group_name)

    def alloc(numel: int, device):
        return _SymmetricMemory.empty_strided_p2p(
            size=(numel,), stride=(1,), dtype=torch.bfloat16, device=device, group_name=group_name)

    return one_shot_all_reduce, alloc
