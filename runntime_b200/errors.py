"""Typed errors, mirroring packages/runntime/src/core/error.ts:4-36: callers
check ``code``; the message is for people."""
from __future__ import annotations

RUNNTIME_ERROR_CODES = (
    "LOAD_FAILED",
    "LOAD_ABORTED",
    "CHECKPOINT_MISMATCH",
    "UNSUPPORTED_DEVICE",
    "EXECUTION_FAILED",
    "INVALID_ARGUMENT",
    "RESOURCE_DISPOSED",
    "NOT_INITIALIZED",
)


class RunntimeError(Exception):
    def __init__(self, code: str, message: str):
        assert code in RUNNTIME_ERROR_CODES, code
        super().__init__(message)
        self.code = code
        self.message = message


def code_of_status(status: int) -> str:
    """rt_status (include/rt_attn.h) -> error code name; status 0 is success."""
    return RUNNTIME_ERROR_CODES[status - 1]
