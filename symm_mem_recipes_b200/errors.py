"""Exceptions raised from device-side status records."""
from __future__ import annotations

_CODES = {
    0: "ok",
    1: "barrier send timed out (peer never consumed the previous signal)",
    2: "barrier wait timed out (peer never arrived)",
    3: "flag wait timed out",
    4: "mbarrier wait timed out (pipeline stalled)",
    5: "bad argument",
}


# where in which kernel the wait ran out (csrc/device/status.h, enum Where)
_WHERE = {
    1: "barrier kernel / signal", 10: "one-shot all-reduce, entry barrier", 11: "one-shot all-reduce, exit barrier",
    12: "two-shot all-reduce, entry barrier", 13: "two-shot all-reduce, exit barrier",
    14: "multimem all-reduce, entry barrier", 15: "multimem all-reduce, exit barrier",
    20: "GEMM: operands never arrived in shared memory (full barrier)",
    21: "GEMM: shared-memory stage never freed (empty barrier)",
    22: "GEMM: accumulator never completed (TMEM full)", 23: "GEMM: accumulator never drained (TMEM empty)",
    24: "all_gather_matmul: a gathered block never arrived", 25: "all_gather_matmul: entry barrier",
    26: "all_gather_matmul: exit barrier", 30: "gemv_all_reduce: a partial never arrived",
    31: "gemv_all_reduce: call number", 40: "matmul_reduce_scatter: a tile's partials never arrived / exit barrier",
    41: "matmul_reduce_scatter: entry barrier", 42: "matmul_reduce_scatter: exit barrier", 99: "test kernel",
}


class SymmMemError(RuntimeError):
    """A kernel or host protocol of this library reported a failure."""


class SymmMemTimeout(SymmMemError):
    """A bounded wait ran out; carries the decoded status record."""

    def __init__(self, code: int, rank: int, block: int, peer: int, where: int, aux: int = 0):
        self.code, self.rank, self.block, self.peer, self.where, self.aux = (
            int(code), int(rank), int(block), int(peer), int(where), int(aux))
        super().__init__(
            f"{_CODES.get(self.code, 'status %d' % self.code)}: rank={self.rank} "
            f"block={self.block} peer={self.peer} where={self.where} ({_WHERE.get(self.where, 'unknown')}) "
            f"aux={self.aux}")


def raise_for_status(record) -> None:
    """`record` is the (code, rank, block, peer, where, aux) tuple of the native layer."""
    if int(record[0]) != 0:
        raise SymmMemTimeout(*record)
