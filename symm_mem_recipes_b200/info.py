"""What this machine offers to the library, as one JSON object.

    python -m symm_mem_recipes_b200.info

Lists the GPUs with their compute capability and SM count, whether each
supports NVLink multicast (NVLS, needed by `multimem_all_reduce_` and the push
gather's broadcast), the peer-access matrix (needed by everything else), the
library's own limits, and whether the native module is built.  Runs without a
GPU (and says so).  No upstream counterpart.
"""
from __future__ import annotations

import json
import sys

import torch


def collect() -> dict:
    info: dict = {"torch": torch.__version__, "cuda_runtime": torch.version.cuda}
    try:
        from ._ext import C
        info["native_module"] = C.__file__
        info["limits"] = {"max_world_size": C.MAX_WORLD_SIZE, "signal_pad_bytes": C.SIGNAL_PAD_BYTES,
                          "barrier_block_slots": C.BLOCK_SLOTS, "barrier_channel_slots": C.CHANNEL_SLOTS}
    except Exception as e:  # noqa: BLE001
        C = None
        info["native_module"] = f"unavailable: {type(e).__name__}: {e}"
    if not torch.cuda.is_available():
        info["gpus"] = []
        info["note"] = "no CUDA device visible: only the CPU backend (gloo tests, oracles) can run here"
        return info
    n = torch.cuda.device_count()
    gpus = []
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        g = {"index": i, "name": p.name, "compute_capability": f"{p.major}.{p.minor}",
             "sms": p.multi_processor_count, "memory_gib": round(p.total_memory / 2**30, 1),
             "kernels_of_this_package_run": (p.major, p.minor) == (10, 0)}
        if C is not None:
            try:
                g["nvlink_multicast"] = bool(C.CudaSymmAllocation.multicast_supported(i))
            except Exception as e:  # noqa: BLE001
                g["nvlink_multicast"] = f"unknown: {e}"
        gpus.append(g)
    info["gpus"] = gpus
    info["peer_access"] = [[i == j or bool(torch.cuda.can_device_access_peer(i, j)) for j in range(n)]
                           for i in range(n)]
    info["all_peers_reachable"] = all(all(row) for row in info["peer_access"])
    return info


def main() -> int:
    print(json.dumps(collect(), indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
