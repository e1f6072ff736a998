"""symm_mem_recipes_b200: symmetric-memory collectives and fused
compute+collective kernels for NVIDIA B200 (sm_100a).

One process per GPU (`torch.distributed`, backend "nccl") for the plumbing;
all cross-GPU bytes of the ops move by loads, stores and `multimem`
instructions issued from this package's own kernels on peer-mapped memory.
"""
from . import errors  # noqa: F401
from .parallel import symm_mem  # noqa: F401
from . import ops  # noqa: F401
from .ops import (all_reduce, barrier_test, low_latency_all_reduce, multimem_all_reduce_,  # noqa: F401
                  one_shot_all_reduce, two_shot_all_reduce_)

from .ops import all_gather_matmul, matmul, reference_all_gather_matmul  # noqa: F401,E402
from .ops import gemv, gemv_all_reduce, reference_gemv_all_reduce  # noqa: F401,E402
from .ops import matmul_reduce_scatter, reference_matmul_reduce_scatter  # noqa: F401,E402
from .ops import matmul_all_reduce, reference_matmul_all_reduce  # noqa: F401,E402

__version__ = "0.1.0"
