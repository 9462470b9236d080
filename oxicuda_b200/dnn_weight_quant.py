"""The weight-only quantization plan of the reference's DNN layer (crates/oxicuda-dnn/src/quantize/gptq_awq.rs) as far as
the inference path needs it: the configuration types with their validate() rules (:65-200), the tensor-size metadata
(QuantizedWeight, :210-232; WeightQuantPlan::quantized_weight_info, :996-1024), the scratch and launch figures the plan
reports (:1029-1085), and the fused dequantise + GEMV (generate_fused_dequant_gemv_ptx, :867-994), which here is a call
of the library's kernel instead of a PTX string.  The plan's quantize / scale-search generators (GPTQ with a Hessian
diagonal, AWQ) are not part of this path and are not mirrored.  Nothing in this module needs a device except
WeightQuantPlan.fused_dequant_gemv."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from .errors import DnnError

QUANT_BLOCK_SIZE = 256                                                    # threads per CTA the reference's launch_params assume


def _invalid(msg: str) -> DnnError:
    return DnnError("InvalidArgument", msg, 15)


class QuantMethodTag(Enum):
    Gptq = "Gptq"
    Awq = "Awq"


@dataclass
class GptqConfig:
    """GptqConfig (gptq_awq.rs:65-135)."""
    bits: int = 4
    group_size: int = 128
    block_size: int = 128
    damp_percent: float = 0.01
    symmetric: bool = True
    act_order: bool = False
    true_sequential: bool = True

    def validate(self) -> None:
        if self.bits not in (2, 3, 4, 8):
            raise _invalid(f"GPTQ bits must be 2, 3, 4, or 8; got {self.bits}")
        if self.group_size == 0:
            raise _invalid("GPTQ group_size must be non-zero")
        if self.block_size == 0:
            raise _invalid("GPTQ block_size must be non-zero")
        if self.damp_percent < 0.0:
            raise _invalid(f"GPTQ damp_percent must be non-negative; got {self.damp_percent}")


@dataclass
class AwqConfig:
    """AwqConfig (gptq_awq.rs:140-200)."""
    bits: int = 4
    group_size: int = 128
    zero_point: bool = True
    search_alpha_min: float = 0.0
    search_alpha_max: float = 1.0
    search_steps: int = 20

    def validate(self) -> None:
        if self.bits not in (4, 8):
            raise _invalid(f"AWQ bits must be 4 or 8; got {self.bits}")
        if self.group_size == 0:
            raise _invalid("AWQ group_size must be non-zero")
        if self.search_alpha_min > self.search_alpha_max:
            raise _invalid(f"AWQ search_alpha_min ({self.search_alpha_min}) must be <= search_alpha_max ({self.search_alpha_max})")
        if self.search_steps == 0:
            raise _invalid("AWQ search_steps must be non-zero")


@dataclass
class WeightQuantMethod:
    """WeightQuantMethod::{Gptq(cfg), Awq(cfg)} (gptq_awq.rs:38-45)."""
    tag: QuantMethodTag
    config: GptqConfig | AwqConfig = field(default_factory=GptqConfig)

    @staticmethod
    def Gptq(config: GptqConfig | None = None) -> "WeightQuantMethod":
        return WeightQuantMethod(QuantMethodTag.Gptq, config if config is not None else GptqConfig())

    @staticmethod
    def Awq(config: AwqConfig | None = None) -> "WeightQuantMethod":
        return WeightQuantMethod(QuantMethodTag.Awq, config if config is not None else AwqConfig())


@dataclass
class QuantizedWeight:
    """QuantizedWeight (gptq_awq.rs:210-232): element counts of the tensors a quantized weight consists of."""
    method: QuantMethodTag
    bits: int
    group_size: int
    rows: int
    cols: int
    packed_weight_elements: int
    scale_elements: int
    zero_point_elements: int
    has_zero_point: bool


class WeightQuantPlan:
    """WeightQuantPlan (gptq_awq.rs:241-1085) for a [rows x cols] weight."""

    def __init__(self, method: WeightQuantMethod, rows: int, cols: int):
        if rows == 0 or cols == 0:
            raise DnnError("InvalidDimension", "weight dimensions must be non-zero", 10)
        method.config.validate()
        group_size = method.config.group_size
        if cols % group_size != 0:
            raise _invalid(f"cols ({cols}) must be divisible by group_size ({group_size})")
        self._method, self._rows, self._cols = method, int(rows), int(cols)

    def _bits(self) -> int:
        return self._method.config.bits

    def _group_size(self) -> int:
        return self._method.config.group_size

    def elements_per_u32(self) -> int:
        return 32 // self._bits()

    def quantized_weight_info(self) -> QuantizedWeight:
        total = self._rows * self._cols
        epu32 = self.elements_per_u32()
        scale_elements = self._rows * (self._cols // self._group_size())
        cfg = self._method.config
        has_zp = (not cfg.symmetric) if self._method.tag is QuantMethodTag.Gptq else cfg.zero_point
        return QuantizedWeight(self._method.tag, self._bits(), self._group_size(), self._rows, self._cols, -(-total // epu32), scale_elements,
                               scale_elements if has_zp else 0, has_zp)

    def workspace_bytes(self) -> int:
        cfg = self._method.config
        if self._method.tag is QuantMethodTag.Gptq:
            return self._cols * 4 + (self._cols * 4 if cfg.act_order else 0) + self._rows * cfg.block_size * 4
        return self._cols * 4 + self._cols * 4 + cfg.search_steps * 4

    def shared_memory_bytes(self) -> int:
        cfg = self._method.config
        return (cfg.block_size if self._method.tag is QuantMethodTag.Gptq else cfg.group_size) * 4

    def launch_params(self) -> tuple[int, int]:
        threads = self._rows if self._method.tag is QuantMethodTag.Gptq else self._rows * self._cols
        return -(-threads // QUANT_BLOCK_SIZE), QUANT_BLOCK_SIZE

    def fused_dequant_gemv(self, packed_w, scales, x):
        """y[row] = sum_col (code[row, col] * scale[row, col / group_size]) * x[col]: the kernel generate_fused_dequant_gemv_ptx
        describes (:867-994), on device tensors: packed_w u32 (or i32) [rows x cols / elements_per_u32], scales f32
        [rows x cols / group_size], x f32 [cols]; returns y f32 [rows].  The device kernel covers 2, 4 and 8 bits."""
        from . import ops
        info = self.quantized_weight_info()
        if packed_w.numel() != info.packed_weight_elements:
            raise DnnError("BufferTooSmall", "packed weight", 11, expected=info.packed_weight_elements * 4, actual=packed_w.numel() * 4)
        if scales.numel() != info.scale_elements:
            raise DnnError("BufferTooSmall", "scales", 11, expected=info.scale_elements * 4, actual=scales.numel() * 4)
        if x.numel() != self._cols:
            raise DnnError("BufferTooSmall", "x", 11, expected=self._cols * 4, actual=x.numel() * 4)
        return ops.fused_dequant_gemv(packed_w.reshape(self._rows, -1), scales, x, self._cols, self._group_size(), self._bits())
