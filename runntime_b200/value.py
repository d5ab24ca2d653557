"""The lazy array type of the operator API: a materialized device buffer or a
pending op (packages/runntime/src/core/graph/value.ts:123-200).  Calling ops
only links nodes; reading a result evaluates what it depends on."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple


def elemBytes(dtype: str) -> int:
    return 2 if dtype == "f16" else 4


@dataclass(frozen=True)
class ValueMeta:
    elems: int
    dtype: str = "f32"
    dims: Optional[Tuple[int, ...]] = None


def matrix(rows: int, cols: int, dtype: str = "f32") -> ValueMeta:
    return ValueMeta(rows * cols, dtype, (rows, cols))


@dataclass(frozen=True)
class PendingOp:
    op: str
    inputs: Tuple["Value", ...]
    scalar: Optional[float] = None
    attrs: Optional[Tuple[float, ...]] = None


class DeviceBuffer:
    """A CUDA device allocation (or a borrowed one: ``keepalive`` holds its owner)."""

    __slots__ = ("ptr", "nbytes", "owned", "keepalive")

    def __init__(self, ptr: int, nbytes: int, owned: bool = True, keepalive=None):
        self.ptr, self.nbytes, self.owned, self.keepalive = ptr, nbytes, owned, keepalive


class Value:
    def __init__(self, shape: ValueMeta, buffer: Optional[DeviceBuffer],
                 pending: Optional[PendingOp]):
        self.shape = shape
        self._buffer = buffer
        self.pending = pending
        self._released: Optional[str] = None

    @property
    def state(self) -> str:
        if self._released is not None:
            return "released"
        return "materialized" if self._buffer is not None else "pending"

    @property
    def releasedReason(self) -> Optional[str]:
        return self._released

    @property
    def buffer(self) -> DeviceBuffer:
        if self._released is not None:
            raise RuntimeError(f"Value.buffer: {self._released}")
        if self._buffer is None:
            raise RuntimeError("Value.buffer: not materialized yet — call eval() first")
        return self._buffer

    def setMaterialized(self, buffer: DeviceBuffer) -> None:
        self._buffer = buffer

    def markReleased(self, reason: str = (
            "buffer was recycled by eval — it must have been a TARGET of the eval that "
            "materialized it (evalValues([primary, v])) to stay alive across evals")) -> None:
        self._released = reason

    @staticmethod
    def materialized(shape: ValueMeta, buffer: DeviceBuffer) -> "Value":
        return Value(shape, buffer, None)

    @staticmethod
    def pending_(shape: ValueMeta, op: str, inputs: Sequence["Value"], scalar=None,
                 attrs=None) -> "Value":
        return Value(shape, None, PendingOp(op, tuple(inputs), scalar,
                                            None if attrs is None else tuple(attrs)))


materialized = Value.materialized
pending = Value.pending_
