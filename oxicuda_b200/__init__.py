"""oxicuda_b200: hand-written sm_100a kernels behind the OxiCUDA quantizer types and low-precision
GEMM entry points.  `ops` is the device-tensor layer over the C ABI (include/oxq.h); `quant`, `blas`
and `dist_infer` keep the reference's names on top of it."""
from . import errors  # noqa: F401

__all__ = ["errors", "ops", "quant", "blas", "dist_infer"]
