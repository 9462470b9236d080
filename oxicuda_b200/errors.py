"""Error types mirroring QuantError (crates/oxicuda-quant/src/error.rs:10-58) and BlasError
(crates/oxicuda-blas/src/error.rs:16-59), raised from the C ABI's status codes."""
from __future__ import annotations


class OxqError(Exception):
    """Base class; `.variant` carries the reference enum variant name, `.status` the C status code."""

    def __init__(self, variant: str, message: str = "", status: int = 0):
        super().__init__(f"{variant}: {message}" if message else variant)
        self.variant = variant
        self.status = status


class QuantError(OxqError):
    pass


class BlasError(OxqError):
    pass


class DnnError(OxqError):
    """DnnError of the reference (crates/oxicuda-dnn/src/error.rs:13-60).  BufferTooSmall counts BYTES here
    (`expected` / `actual` attributes), unlike BlasError::BufferTooSmall, which counts elements."""

    def __init__(self, variant: str, message: str = "", status: int = 0, expected: int | None = None, actual: int | None = None):
        if variant == "BufferTooSmall" and expected is not None:
            message = f"expected {expected} bytes, got {actual} bytes"
        super().__init__(variant, message, status)
        self.expected, self.actual = expected, actual


class DistInferError(OxqError):
    """DistInferError of the reference (crates/oxicuda-dist-infer/src/error.rs): TpFeaturesMisaligned,
    TpInputMisaligned, DimensionMismatch, TooFewRanks, ShardShapeMismatch."""


_QUANT = {1: "EmptyInput", 2: "GroupSizeMismatch", 3: "InvalidScale", 4: "DimensionMismatch", 5: "NonFiniteFp8",
          6: "InvalidBitWidth", 7: "SingularHessian"}
_BLAS = {10: "InvalidDimension", 11: "BufferTooSmall", 12: "DimensionMismatch", 13: "UnsupportedOperation",
         14: "LaunchFailed", 15: "InvalidArgument", 100: "LaunchFailed"}


def raise_for_status(status: int, message: str = ""):
    if status == 0:
        return
    if status in _QUANT:
        raise QuantError(_QUANT[status], message, status)
    if status in _BLAS:
        raise BlasError(_BLAS[status], message, status)
    if status >= 1000:
        raise BlasError("Cuda", f"cudaError {status - 1000}: {message}", status)
    raise OxqError("Unknown", message, status)
