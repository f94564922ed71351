"""Error type of the framework.

The reference returns ``Result<T, Error>`` whose ``Error`` carries an ``ErrorCode``
in numbered ranges (include/photon/core/error.hpp:40-87: memory 1-99, IO 100-199,
tensor 200-299, model 300-399, operator 400-499, CUDA 500-599).  In Python the same
information travels as one exception class with a ``code``; callers that want to
branch test ``err.code``, everything else reads the message.
"""
from __future__ import annotations

import enum


class ErrorCode(enum.IntEnum):
    OUT_OF_MEMORY = 1            # page pool or slot pool exhausted
    DOUBLE_FREE = 2
    FILE_NOT_FOUND = 100
    INVALID_FILE = 101
    SHAPE_MISMATCH = 200
    INVALID_INDEX = 201
    INVALID_ARGUMENT = 202
    UNSUPPORTED_MODEL = 300
    INVALID_CONFIG = 301
    WEIGHTS_MISMATCH = 302
    UNSUPPORTED_SIZE = 400       # a kernel refuses a size it cannot run correctly
    NOT_BUILT = 401              # the CUDA extension is missing or failed to compile
    CUDA_ERROR = 500
    INVALID_STATE = 900


class PhotonError(RuntimeError):
    def __init__(self, code: ErrorCode, message: str):
        super().__init__(f"[{code.name}] {message}")
        self.code = code
        self.message = message


def fail(code: ErrorCode, message: str) -> "PhotonError":
    return PhotonError(code, message)
