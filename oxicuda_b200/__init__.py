"""oxicuda_b200: hand-written sm_100a kernels behind the OxiCUDA quantizer types and low-precision
GEMM entry points.  `ops` is the device-tensor layer over the C ABI (include/oxq.h) and keeps the reference's
type names where it has them (TensorDesc, Int4QuantConfig, SmoothQuantMigrator, GptqQuantizer ...);
`dist_infer` holds the tensor-parallel layers (ColumnLinear, RowLinear, TpSwiGluMlp); `dnn_weight_quant` the DNN
layer's weight-only plan (WeightQuantPlan with its fused dequantise + GEMV); `errors` the reference's error variants.  `ops` and `dist_infer` import torch, so they are loaded on first use, not with the package."""
from . import errors  # noqa: F401

__all__ = ["errors", "ops", "dist_infer", "dnn_weight_quant"]


def __getattr__(name):
    if name in ("ops", "dist_infer", "dnn_weight_quant"):
        import importlib
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
