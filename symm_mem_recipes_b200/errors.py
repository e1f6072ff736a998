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


class SymmMemError(RuntimeError):
    """A kernel or host protocol of this library reported a failure."""


class SymmMemTimeout(SymmMemError):
    """A bounded wait ran out; carries the decoded status record."""

    def __init__(self, code: int, rank: int, block: int, peer: int, where: int, aux: int = 0):
        self.code, self.rank, self.block, self.peer, self.where, self.aux = (
            int(code), int(rank), int(block), int(peer), int(where), int(aux))
        super().__init__(
            f"{_CODES.get(self.code, 'status %d' % self.code)}: rank={self.rank} "
            f"block={self.block} peer={self.peer} where={self.where} aux={self.aux}")


def raise_for_status(record) -> None:
    """`record` is the (code, rank, block, peer, where, aux) tuple of the native layer."""
    if int(record[0]) != 0:
        raise SymmMemTimeout(*record)
