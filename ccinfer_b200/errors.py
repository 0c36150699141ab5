"""Error types of the engine.

The names follow the error codes of 7QiC/ccInfer (src/base/error_code.h:8-45)
where it has one for the situation.
"""
from __future__ import annotations


class CcinferError(Exception):
    """Base of every error the engine raises on purpose."""

    code = "Unknown"


class ModelUnsupportedArch(CcinferError):
    code = "ModelUnsupportedArch"


class ModelConfigInvalid(CcinferError):
    code = "ModelConfigInvalid"


class ModelUnsupportedDType(CcinferError):
    code = "ModelUnsupportedDType"


class ModelLoadFailed(CcinferError):
    code = "ModelLoadFailed"


class InvalidArgument(CcinferError):
    code = "InvalidArgument"


class Unsupported(CcinferError):
    code = "Unsupported"


class RequestTooLong(CcinferError):
    code = "RequestTooLong"


class KVBlockExhausted(CcinferError):
    code = "KVBlockExhausted"


class KVBlockDoubleFree(CcinferError):
    code = "KVBlockDoubleFree"


class KVInvalidBlockTable(CcinferError):
    code = "KVInvalidBlockTable"


class SlotExhausted(CcinferError):
    code = "SequenceLimitReached"


class ExtensionMissing(CcinferError):
    """The CUDA extension could not be built or loaded; there is no fallback."""

    code = "ExtensionMissing"


class DeviceFault(CcinferError):
    """A kernel reported a bad index through the device status word."""

    code = "CudaLaunchFailed"


class ScratchMoved(CcinferError):
    """A part asked for a larger scratch buffer after CUDA graphs had recorded the pool's addresses."""

    code = "InvalidState"
