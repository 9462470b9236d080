"""Device-tensor front end of the C ABI: torch tensors supply device memory and the current stream,
every computation happens inside liboxq_b200.so.  Function names follow the C entry points."""
from __future__ import annotations

import ctypes as C

import torch

from . import _ffi
from .errors import raise_for_status

F32, BF16, F16 = 0, 1, 2
ROUND_HALF_EVEN, ROUND_HALF_AWAY = 0, 1
FP8_SPEC_RNE, FP8_REFCOMPAT = 0, 1

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
_TORCH_DT = {F32: torch.float32, BF16: torch.bfloat16, F16: torch.float16}


class Handle:
    """One per host thread and device, like BlasHandle (crates/oxicuda-blas/src/handle.rs:41-52)."""

    def __init__(self, device: int | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("oxicuda_b200 needs a CUDA device (sm_100); there is no CPU fallback")
        self.lib = _ffi.load()
        self.device = torch.cuda.current_device() if device is None else int(device)
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream().cuda_stream
            raise_for_status(self.lib.oxq_handle_create(self.device, C.c_void_p(stream), C.byref(self._h)))
        self._stream = stream

    def close(self):
        if self._h:
            self.lib.oxq_handle_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync_stream(self):
        """Follow torch's current stream (BlasHandle::set_stream)."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        if s != self._stream:
            raise_for_status(self.lib.oxq_set_stream(self._h, C.c_void_p(s)))
            self._stream = s

    def call(self, name: str, *args):
        self.sync_stream()
        rc = getattr(self.lib, name)(self._h, *args)
        if rc:
            raise_for_status(rc, self.lib.oxq_last_error_string(self._h).decode())

    def device_status(self) -> int:
        v = C.c_int32(0)
        raise_for_status(self.lib.oxq_device_status(self._h, C.byref(v)))
        return v.value


_handles: dict[int, Handle] = {}


def handle(device: int | None = None) -> Handle:
    d = torch.cuda.current_device() if device is None else int(device)
    if d not in _handles:
        _handles[d] = Handle(d)
    return _handles[d]


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _chk(t: torch.Tensor, *dtypes):
    if not t.is_cuda:
        raise TypeError("expected a CUDA tensor")
    if not t.is_contiguous():
        raise TypeError("expected a contiguous tensor")
    if dtypes and t.dtype not in dtypes:
        raise TypeError(f"expected dtype in {dtypes}, got {t.dtype}")


# ------------------------------------------------------------------------------------------- INT8

def int8_quant_rows(x: torch.Tensor, rounding: int = ROUND_HALF_EVEN):
    _chk(x, torch.float32)
    rows, cols = (x.shape[0], x.shape[1]) if x.dim() == 2 else (0, 0)
    q = torch.empty((rows, cols), dtype=torch.int8, device=x.device)
    s = torch.empty((rows,), dtype=torch.float32, device=x.device)
    handle(x.device.index).call("oxq_int8_quant_rows", _p(x), rows, cols, _p(q), _p(s), rounding)
    return q, s


def int8_dequant_rows(q: torch.Tensor, scales: torch.Tensor):
    _chk(q, torch.int8)
    _chk(scales, torch.float32)
    rows, cols = q.shape
    y = torch.empty((rows, cols), dtype=torch.float32, device=q.device)
    handle(q.device.index).call("oxq_int8_dequant_rows", _p(q), _p(scales), rows, cols, _p(y))
    return y


# ------------------------------------------------------------------------------------------- FP8

def absmax(x: torch.Tensor, out: torch.Tensor | None = None):
    _chk(x, *_DT)
    out = torch.empty(1, dtype=torch.float32, device=x.device) if out is None else out
    handle(x.device.index).call("oxq_absmax", _p(x), _DT[x.dtype], x.numel(), _p(out))
    return out


def fp8_quant(x: torch.Tensor, scale: torch.Tensor, mode: int = FP8_SPEC_RNE, out: torch.Tensor | None = None):
    _chk(x, *_DT)
    _chk(scale, torch.float32)
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device) if out is None else out
    handle(x.device.index).call("oxq_fp8_quant", _p(x), _DT[x.dtype], x.numel(), _p(scale), _p(q), mode)
    return q


def fp8_quant_dynamic(x: torch.Tensor, out: torch.Tensor | None = None, stats: torch.Tensor | None = None):
    """Returns (codes, stats) with stats[0] = absmax and stats[1] = scale = absmax / 448."""
    _chk(x, *_DT)
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device) if out is None else out
    stats = torch.empty(2, dtype=torch.float32, device=x.device) if stats is None else stats
    handle(x.device.index).call("oxq_fp8_quant_dynamic", _p(x), _DT[x.dtype], x.numel(), _p(q), _p(stats))
    return q, stats


def fp8_dequant(q: torch.Tensor, scale: torch.Tensor, dtype=torch.float32, mode: int = FP8_SPEC_RNE):
    _chk(q, torch.uint8)
    y = torch.empty(q.shape, dtype=dtype, device=q.device)
    handle(q.device.index).call("oxq_fp8_dequant", _p(q), q.numel(), _p(scale), _p(y), _DT[dtype], mode)
    return y


# ------------------------------------------------------------------------------------------- INT4

def int4g_quant_pack(x: torch.Tensor, group: int = 128, rounding: int = ROUND_HALF_AWAY):
    _chk(x, *_DT)
    rows, k = (x.shape[0], x.shape[1]) if x.dim() == 2 else (0, 0)
    ng = rows * (k // group) if group > 0 else 0
    # int32 tensors hold the u32 words and uint16 bit patterns are kept in int16 tensors
    codes = torch.empty((rows, max(k // 8, 0)), dtype=torch.int32, device=x.device)
    scales = torch.empty((rows, k // group if group > 0 else 0), dtype=torch.float16, device=x.device)
    zeros = torch.empty(((ng + 7) // 8,), dtype=torch.int32, device=x.device)
    handle(x.device.index).call("oxq_int4g_quant_pack", _p(x), _DT[x.dtype], rows, k, group, _p(codes), _p(scales),
                                _p(zeros), rounding)
    return codes, scales, zeros


def int4g_dequant(codes, scales, zeros, rows: int, k: int, group: int = 128, dtype=torch.float32):
    y = torch.empty((rows, k), dtype=dtype, device=codes.device)
    handle(codes.device.index).call("oxq_int4g_dequant", _p(codes), _p(scales), _p(zeros), rows, k, group, _p(y),
                                    _DT[dtype])
    return y


def int4g_quant_pack_f32(x: torch.Tensor, group: int = 128, rounding: int = ROUND_HALF_AWAY, check_scales: bool = True):
    """MinMaxQuantizer per group, asymmetric, in the reference's own parameter types: (codes u32 words [rows x k/8],
    scales f32 [rows x k/group], zero_points i32 [rows x k/group]).  With check_scales the scales are read back and a
    non-finite or non-positive one raises QuantError InvalidScale, as calibrate does (minmax.rs:234-236)."""
    _chk(x, torch.float32)
    rows, k = (x.shape[0], x.shape[1]) if x.dim() == 2 else (0, 0)
    gpr = k // group if group > 0 else 0
    codes = torch.empty((rows, max(k // 8, 0)), dtype=torch.int32, device=x.device)
    scales = torch.empty((rows, gpr), dtype=torch.float32, device=x.device)
    zps = torch.empty((rows, gpr), dtype=torch.int32, device=x.device)
    handle(x.device.index).call("oxq_int4g_quant_pack_f32", _p(x), rows, k, group, _p(codes), _p(scales), _p(zps), rounding)
    if check_scales and not bool((torch.isfinite(scales) & (scales > 0)).all()):
        from .errors import QuantError
        raise QuantError("InvalidScale", "a group's scale is not finite and positive", 3)
    return codes, scales, zps


def int4g_dequant_f32(codes, scales, zps, rows: int, k: int, group: int = 128):
    y = torch.empty((rows, k), dtype=torch.float32, device=codes.device)
    handle(codes.device.index).call("oxq_int4g_dequant_f32", _p(codes), _p(scales), _p(zps), rows, k, group, _p(y))
    return y


def fp4_microscale_quant(x: torch.Tensor, block: int = 32):
    """MicroScalingQuantizer::quantize_fp4 (crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:849-876):
    (packed bytes [ceil(n / 2)], f32 scales [ceil(n / block)])."""
    _chk(x, torch.float32)
    n = x.numel()
    packed = torch.empty(max((n + 1) // 2, 1), dtype=torch.uint8, device=x.device)
    scales = torch.empty(max((n + max(block, 1) - 1) // max(block, 1), 1), dtype=torch.float32, device=x.device)
    handle(x.device.index).call("oxq_fp4_microscale_quant", _p(x), n, block, _p(packed), _p(scales))
    return packed[: (n + 1) // 2], scales[: (n + block - 1) // block]


def fp4_microscale_dequant(packed: torch.Tensor, scales: torch.Tensor, n: int, block: int = 32):
    y = torch.empty(max(n, 1), dtype=torch.float32, device=packed.device)
    handle(packed.device.index).call("oxq_fp4_microscale_dequant", _p(packed), _p(scales), n, block, _p(y))
    return y[:n]


class TensorDesc:
    """TensorDesc<T> of the reference's DNN layer (crates/oxicuda-dnn/src/types.rs:108-118) over a torch tensor:
    a borrowed device pointer with dims and strides; numel() and the byte size follow the dims."""

    def __init__(self, tensor: torch.Tensor):
        _chk(tensor, torch.float32, torch.bfloat16, torch.float16)
        self.tensor = tensor
        self.ptr = tensor.data_ptr()
        self.dims = tuple(tensor.shape)
        self.strides = tuple(tensor.stride())

    def numel(self) -> int:
        return self.tensor.numel()

    def nbytes(self) -> int:
        return self.tensor.numel() * self.tensor.element_size()


def _dnn_need(buf: torch.Tensor, elems: int, what: str):
    """DnnError::BufferTooSmall counts bytes (crates/oxicuda-dnn/src/error.rs:33-40)."""
    if buf.numel() < elems:
        from .errors import DnnError
        raise DnnError("BufferTooSmall", what, 11, expected=elems * buf.element_size(), actual=buf.numel() * buf.element_size())


class Int4QuantConfig:
    """Int4QuantConfig of the DNN layer (crates/oxicuda-dnn/src/quantize/int4_quantize.rs:66-104)."""

    def __init__(self, group_size: int, symmetric: bool):
        if group_size == 0:
            from .errors import DnnError
            raise DnnError("InvalidArgument", "INT4 group_size must be non-zero", 15)
        self.group_size, self.symmetric = int(group_size), bool(symmetric)

    def num_groups(self, n: int) -> int:
        return -(-n // self.group_size)

    def packed_bytes(self, n: int) -> int:
        return -(-n // 2)


def quantize_to_int4(x: torch.Tensor, output: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor | None, n: int, config: Int4QuantConfig):
    """quantize_to_int4 (int4_quantize.rs:132-218): fills `output` (ceil(n / 2) bytes), `scales` and, when asymmetric,
    `zeros` (one float per group).  n == 0 does nothing; undersized buffers raise DnnError BufferTooSmall in bytes."""
    if n == 0:
        return
    _chk(x, torch.float32)
    _dnn_need(x, n, "input")
    _dnn_need(output, config.packed_bytes(n), "output")
    _dnn_need(scales, config.num_groups(n), "scales")
    if not config.symmetric:
        if zeros is None:
            from .errors import DnnError
            raise DnnError("BufferTooSmall", "zeros", 11, expected=config.num_groups(n) * 4, actual=0)
        _dnn_need(zeros, config.num_groups(n), "zeros")
    handle(x.device.index).call("oxq_dnn_int4_quant", _p(x), n, config.group_size, 1 if config.symmetric else 0, _p(output), _p(scales),
                                _p(zeros if not config.symmetric else None))


def dequantize_int4(packed: torch.Tensor, scales: torch.Tensor, output: torch.Tensor, n: int, config: Int4QuantConfig):
    """dequantize_int4 (int4_quantize.rs:229-300)."""
    if n == 0:
        return
    _dnn_need(packed, config.packed_bytes(n), "input")
    _dnn_need(scales, config.num_groups(n), "scales")
    _dnn_need(output, n, "output")
    handle(packed.device.index).call("oxq_dnn_int4_dequant", _p(packed), _p(scales), n, config.group_size, 1 if config.symmetric else 0, _p(output))


class Fp4BlockQuantizer:
    """Fp4BlockQuantizer of the DNN layer (crates/oxicuda-dnn/src/quantize/block_scale.rs:346-395): the host-side helper for blocks of
    32 E2M1 codes; compute_scale is max |x| / 6 in f32, or 1 for an all-zero block."""

    MAX_VALUE = 6.0
    REQUIRED_BLOCK_SIZE = 32

    def __init__(self, block_size: int):
        if block_size != self.REQUIRED_BLOCK_SIZE:
            from .errors import DnnError
            raise DnnError("InvalidArgument", f"NVFP4/OCP MXFP4 block size must be {self.REQUIRED_BLOCK_SIZE}, got {block_size}", 15)
        self.block_size = int(block_size)

    def compute_scale(self, block) -> float:
        import numpy as np
        b = np.asarray(block, dtype=np.float32)
        max_abs = np.float32(np.nanmax(np.abs(b))) if b.size and not np.isnan(b).all() else np.float32(0.0)   # f32::max skips NaN
        return 1.0 if max_abs == 0.0 else float(max_abs / np.float32(self.MAX_VALUE))

    def num_scales(self, n: int) -> int:
        return -(-n // self.block_size)


def quantize_block_scaled(desc: TensorDesc, output: torch.Tensor, scales: torch.Tensor, block_size: int):
    """quantize_block_scaled (crates/oxicuda-dnn/src/quantize/block_scale.rs:53-140): one biased byte per element into
    `output`, one f32 scale per block into `scales`."""
    from .errors import DnnError
    n = desc.numel()
    if n == 0:
        return
    if block_size == 0 or (block_size & (block_size - 1)) != 0:
        raise DnnError("InvalidArgument", f"block_size must be a non-zero power of 2, got {block_size}", 15)
    if block_size < 16:
        raise DnnError("InvalidArgument", f"block_size must be >= 16, got {block_size}", 15)
    _dnn_need(output, n, "output")
    _dnn_need(scales, -(-n // block_size), "scales")
    x = desc.tensor
    handle(x.device.index).call("oxq_dnn_block_scaled_quant", _p(x), _DT[x.dtype], n, block_size, _p(output), _p(scales))


def fused_dequant_gemv(packed_w: torch.Tensor, scales: torch.Tensor, x: torch.Tensor, cols: int, group_size: int, bits: int = 4):
    """dnn_fused_dequant_gemv_f32 (crates/oxicuda-dnn/src/quantize/gptq_awq.rs:867-994): y[row] = sum_col (code * scale) * x[col] with
    unsigned codes packed LSB-first in u32 words [rows x cols * bits / 32], f32 scales [rows x cols / group_size], f32 x and y."""
    _chk(x, torch.float32)
    _chk(scales, torch.float32)
    rows = packed_w.shape[0]
    y = torch.empty(rows, dtype=torch.float32, device=x.device)
    handle(x.device.index).call("oxq_dnn_fused_dequant_gemv", _p(packed_w), _p(scales), _p(x), _p(y), rows, cols, group_size, bits)
    return y


# ------------------------------------------------------------------------------------------- block scaled

def sf_mma_bytes(rows: int, sf_cols: int) -> int:
    return int(_ffi.load().oxq_sf_mma_bytes(rows, sf_cols))


def mxfp8_quant(x: torch.Tensor, want_mma_layout: bool = True):
    """Returns (codes [rows x k] u8, sf_rowmajor [rows x k/32] u8, sf_mma bytes or None)."""
    _chk(x, *_DT)
    rows, k = (x.shape[0], x.shape[1]) if x.dim() == 2 else (0, 0)
    codes = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    sf = torch.empty((rows, k // 32), dtype=torch.uint8, device=x.device)
    sf_mma = torch.empty(sf_mma_bytes(rows, k // 32), dtype=torch.uint8, device=x.device) if want_mma_layout else None
    handle(x.device.index).call("oxq_mxfp8_quant", _p(x), _DT[x.dtype], rows, k, _p(codes), _p(sf), _p(sf_mma))
    return codes, sf, sf_mma


def mxfp8_dequant(codes, sf, dtype=torch.float32):
    rows, k = codes.shape
    y = torch.empty((rows, k), dtype=dtype, device=codes.device)
    handle(codes.device.index).call("oxq_mxfp8_dequant", _p(codes), _p(sf), rows, k, _p(y), _DT[dtype])
    return y


def nvfp4_quant(x: torch.Tensor, want_mma_layout: bool = True, stats: torch.Tensor | None = None):
    """absmax pass + encode pass.  Returns (packed [rows x k/2] u8, sf_rowmajor [rows x k/16] u8, sf_mma, stats)
    with stats[0] = absmax and stats[1] = the f32 tensor scale."""
    _chk(x, *_DT)
    rows, k = (x.shape[0], x.shape[1]) if x.dim() == 2 else (0, 0)
    stats = torch.empty(2, dtype=torch.float32, device=x.device) if stats is None else stats
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty((rows, k // 16), dtype=torch.uint8, device=x.device)
    sf_mma = torch.empty(sf_mma_bytes(rows, k // 16), dtype=torch.uint8, device=x.device) if want_mma_layout else None
    h = handle(x.device.index)
    if rows > 0 and k > 0:
        h.call("oxq_absmax", _p(x), _DT[x.dtype], x.numel(), _p(stats))
    h.call("oxq_nvfp4_quant", _p(x), _DT[x.dtype], rows, k, _p(stats), _p(packed), _p(sf), _p(sf_mma))
    return packed, sf, sf_mma, stats


def nvfp4_dequant(packed, sf, stats, dtype=torch.float32):
    rows, k = packed.shape[0], packed.shape[1] * 2
    y = torch.empty((rows, k), dtype=dtype, device=packed.device)
    handle(packed.device.index).call("oxq_nvfp4_dequant", _p(packed), _p(sf), _p(stats), rows, k, _p(y), _DT[dtype])
    return y


# ------------------------------------------------------------------------------------------- next to the hot path

def quantize_to_int8(x: torch.Tensor, out: torch.Tensor | None = None, scale: torch.Tensor | None = None):
    """Per-tensor INT8 of oxicuda-dnn (crates/oxicuda-dnn/src/quantize/int8_quantize.rs:33-38): returns (codes, scale[1])."""
    _chk(x, torch.float32, torch.bfloat16, torch.float16)
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device) if out is None else out
    sc = torch.empty(1, dtype=torch.float32, device=x.device) if scale is None else scale
    handle(x.device.index).call("oxq_int8_quant_tensor", _p(x), _DT[x.dtype], x.numel(), _p(q), _p(sc))
    return q, sc


def dequantize_from_int8(q: torch.Tensor, scale: torch.Tensor, dtype=torch.float32):
    """out[i] = (float)q[i] * scale[0] (int8_quantize.rs:101-107)."""
    y = torch.empty(q.shape, dtype=dtype, device=q.device)
    handle(q.device.index).call("oxq_int8_dequant_tensor", _p(q), _p(scale), q.numel(), _p(y), _DT[dtype])
    return y


def block_int8_quant(x: torch.Tensor, block: int):
    """BlockQuantizedInt8::quantize on a device tensor (int8_quantize.rs:404-432): (codes, scales[ceil(n / block)])."""
    _chk(x, torch.float32)
    if block <= 0:
        raise ValueError("block_size must be > 0")
    n = x.numel()
    q = torch.empty(n, dtype=torch.int8, device=x.device)
    sc = torch.empty(max((n + block - 1) // block, 1), dtype=torch.float32, device=x.device)
    handle(x.device.index).call("oxq_int8_block_quant", _p(x), n, block, _p(q), _p(sc))
    return q, sc[: (n + block - 1) // block]


def block_int8_dequant(q: torch.Tensor, scales: torch.Tensor, block: int):
    y = torch.empty(q.numel(), dtype=torch.float32, device=q.device)
    handle(q.device.index).call("oxq_int8_block_dequant", _p(q), _p(scales), q.numel(), block, _p(y))
    return y


def nf4_quant(x: torch.Tensor, block: int = 64):
    """Nf4Quantizer::encode (crates/oxicuda-quant/src/scheme/nf4.rs:93-130): (packed bytes [n / 2], absmax [n / block])."""
    _chk(x, torch.float32)
    n = x.numel()
    packed = torch.empty(max(n // 2, 1), dtype=torch.uint8, device=x.device)
    am = torch.empty(max(n // max(block, 1), 1), dtype=torch.float32, device=x.device)
    handle(x.device.index).call("oxq_nf4_quant", _p(x), n, block, _p(packed), _p(am))
    return packed[: n // 2], am[: n // block]


def nf4_dequant(packed: torch.Tensor, absmaxs: torch.Tensor, block: int = 64, dtype=torch.float32):
    """Nf4Quantizer::decode (nf4.rs:137-155)."""
    n = packed.numel() * 2
    if block <= 0 or absmaxs.numel() != n // block:
        from .errors import QuantError
        raise QuantError("DimensionMismatch", f"expected {n // max(block, 1)} absmax values, got {absmaxs.numel()}", 4)
    y = torch.empty(n, dtype=dtype, device=packed.device)
    handle(packed.device.index).call("oxq_nf4_dequant", _p(packed), _p(absmaxs), n, block, _p(y), _DT[dtype])
    return y


def gemm_nf4(x: torch.Tensor, packed: torch.Tensor, absmaxs: torch.Tensor, n: int, block: int = 64, out: torch.Tensor | None = None):
    """Y = X . dequant(W)^T for up to 8 batch rows; `packed` / `absmaxs` are nf4_quant's tensors of a row-major [n x k] weight."""
    _chk(x, torch.bfloat16)
    _chk(packed, torch.uint8)
    _chk(absmaxs, torch.float32)
    m, k = x.shape
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device) if out is None else out
    handle(x.device.index).call("oxq_gemm_nf4", m, n, k, _p(x), _p(packed), _p(absmaxs), block, _p(y))
    return y


def rmsnorm_int8_quant_rows(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, want_normed: bool = False):
    """RmsNorm::forward (crates/oxicuda-lm/src/layer/norm.rs:73-95) fused with the per-row INT8 quantizer: returns
    (codes int8 [rows x cols], scales f32 [rows]) and, if asked, the normalised activations in x's dtype."""
    _chk(x, torch.float32, torch.bfloat16, torch.float16)
    _chk(weight, torch.float32)
    rows, cols = x.shape
    if weight.numel() != cols:
        from .errors import QuantError
        raise QuantError("DimensionMismatch", f"expected {cols} weights, got {weight.numel()}", 4)
    q = torch.empty((rows, cols), dtype=torch.int8, device=x.device)
    sc = torch.empty(rows, dtype=torch.float32, device=x.device)
    y = torch.empty_like(x) if want_normed else None
    handle(x.device.index).call("oxq_rmsnorm_int8_quant_rows", _p(x), _DT[x.dtype], _p(weight), rows, cols, C.c_float(eps), _p(q), _p(sc), _p(y))
    return (q, sc, y) if want_normed else (q, sc)


def rmsnorm_fp8_quant_rows(x: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, eps: float = 1e-5):
    """RmsNorm::forward fused with the E4M3 quantizer at a calibrated per-tensor scale: codes uint8 [rows x cols]."""
    _chk(x, torch.float32, torch.bfloat16, torch.float16)
    _chk(weight, torch.float32)
    rows, cols = x.shape
    if weight.numel() != cols:
        from .errors import QuantError
        raise QuantError("DimensionMismatch", f"expected {cols} weights, got {weight.numel()}", 4)
    q = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
    handle(x.device.index).call("oxq_rmsnorm_fp8_quant_rows", _p(x), _DT[x.dtype], _p(weight), rows, cols, C.c_float(eps), _p(scale), _p(q))
    return q


def silu_gate_fp8_quant(gate: torch.Tensor, up: torch.Tensor, scale: torch.Tensor):
    """silu(gate) * up (the reference's silu_gate kernel) fused with the E4M3 quantizer at a calibrated per-tensor scale."""
    _chk(gate, torch.float32, torch.bfloat16, torch.float16)
    _chk(up, gate.dtype)
    if gate.shape != up.shape:
        from .errors import QuantError
        raise QuantError("DimensionMismatch", f"gate {tuple(gate.shape)} vs up {tuple(up.shape)}", 4)
    q = torch.empty(gate.shape, dtype=torch.uint8, device=gate.device)
    handle(gate.device.index).call("oxq_silu_gate_fp8_quant", _p(gate), _p(up), _DT[gate.dtype], gate.numel(), _p(scale), _p(q))
    return q


def quantize_to_fp8(x: torch.Tensor, out: torch.Tensor | None = None, scale: torch.Tensor | None = None):
    """quantize_to_fp8 of the reference's DNN layer (crates/oxicuda-dnn/src/quantize/fp8_quantize.rs:47-118): per-tensor
    scale = absmax / 448 into a one-element buffer, E4M3 codes.  Returns (codes, scale)."""
    stats = torch.empty(2, dtype=torch.float32, device=x.device)
    q, _ = fp8_quant_dynamic(x, out=out, stats=stats)
    if scale is None:
        scale = stats[1:2]
    else:
        scale[:1].copy_(stats[1:2])
    return q, scale


def dequantize_from_fp8(q: torch.Tensor, scale: torch.Tensor, dtype=torch.float32):
    """dequantize_from_fp8 (fp8_quantize.rs:121-170): out[i] = e4m3(q[i]) * scale[0]."""
    return fp8_dequant(q, scale, dtype=dtype)


class SmoothQuantMigrator:
    """SmoothQuantMigrator of the reference (crates/oxicuda-quant/src/scheme/smooth_quant.rs:54-293) on device tensors."""

    def __init__(self, alpha: float = 0.5):
        self.alpha = float(alpha)

    @staticmethod
    def _col_absmax(x: torch.Tensor) -> torch.Tensor:
        _chk(x, torch.float32)
        if x.dim() != 2:
            from .errors import QuantError
            raise QuantError("DimensionMismatch", f"expected a matrix, got {tuple(x.shape)}", 4)
        st = torch.empty(max(x.shape[1], 1), dtype=torch.float32, device=x.device)
        handle(x.device.index).call("oxq_smooth_col_absmax", _p(x), x.shape[0], x.shape[1], _p(st))
        return st[: x.shape[1]]

    compute_act_stats = _col_absmax
    compute_weight_stats = _col_absmax

    def compute_migration_scales(self, act_max: torch.Tensor, weight_max: torch.Tensor) -> torch.Tensor:
        from .errors import QuantError
        if act_max.numel() == 0:
            raise QuantError("EmptyInput", "SmoothQuantMigrator::compute_migration_scales", 1)
        if act_max.numel() != weight_max.numel():
            raise QuantError("DimensionMismatch", f"expected {act_max.numel()}, got {weight_max.numel()}", 4)
        sc = torch.empty_like(act_max)
        handle(act_max.device.index).call("oxq_smooth_scales", _p(act_max), _p(weight_max), act_max.numel(), C.c_float(self.alpha), _p(sc))
        return sc

    @staticmethod
    def _apply(x: torch.Tensor, scales: torch.Tensor, divide: bool):
        from .errors import QuantError
        _chk(x, torch.float32)
        if x.dim() != 2 or scales.numel() != x.shape[1]:
            raise QuantError("DimensionMismatch", f"expected {x.shape[-1]} scales, got {scales.numel()}", 4)
        handle(x.device.index).call("oxq_smooth_apply", _p(x), x.shape[0], x.shape[1], _p(scales), 1 if divide else 0)
        return x

    @staticmethod
    def smooth_activations(acts: torch.Tensor, scales: torch.Tensor):
        """In place acts[t, j] /= max(scales[j], 1e-12)."""
        return SmoothQuantMigrator._apply(acts, scales, True)

    @staticmethod
    def smooth_weights(weights: torch.Tensor, scales: torch.Tensor):
        """In place weights[r, j] *= scales[j]."""
        return SmoothQuantMigrator._apply(weights, scales, False)

    def smooth_layer(self, acts: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """Smooths both matrices in place and returns the per-channel scales (smooth_quant.rs:274-293)."""
        sc = self.compute_migration_scales(self.compute_act_stats(acts), self.compute_weight_stats(weights))
        self.smooth_activations(acts, sc)
        self.smooth_weights(weights, sc)
        return sc


class GptqConfig:
    """GptqConfig of the reference (crates/oxicuda-quant/src/scheme/gptq.rs:30-54); block_size has no effect there or here."""

    def __init__(self, bits: int = 4, block_size: int = 128, percdamp: float = 0.01, symmetric: bool = True):
        self.bits, self.block_size, self.percdamp, self.symmetric = int(bits), int(block_size), float(percdamp), bool(symmetric)


class GptqOutput:
    """GptqOutput of the reference (gptq.rs:58-96) on device tensors: codes [n_rows, n_cols] i32, per-column scales and zero points."""

    def __init__(self, quantized, scales, zero_points, n_rows, n_cols):
        self.quantized, self.scales, self.zero_points, self.n_rows, self.n_cols = quantized, scales, zero_points, n_rows, n_cols

    def dequantize(self) -> torch.Tensor:
        return (self.quantized.to(torch.float32) - self.zero_points.to(torch.float32)[None, :]) * self.scales[None, :]

    def reconstruction_mse(self, original: torch.Tensor) -> float:
        return float(((self.dequantize() - original.reshape(self.n_rows, self.n_cols)) ** 2).mean())


class GptqQuantizer:
    """GptqQuantizer of the reference (gptq.rs:104-257) on device tensors; the whole layer is quantized on the GPU."""

    def __init__(self, config: GptqConfig | None = None):
        self.config = config or GptqConfig()
        self.workspace: torch.Tensor | None = None      # kept after a call: H^-1 and the factor's inverse, for inspection

    def quantize_layer(self, weights: torch.Tensor, n_rows: int, n_cols: int, hessian: torch.Tensor) -> GptqOutput:
        from .errors import QuantError
        if weights.numel() == 0:
            raise QuantError("EmptyInput", "GptqQuantizer::quantize_layer", 1)
        if weights.numel() != n_rows * n_cols:
            raise QuantError("DimensionMismatch", f"expected {n_rows * n_cols}, got {weights.numel()}", 4)
        if hessian.numel() != n_cols * n_cols:
            raise QuantError("DimensionMismatch", f"expected {n_cols * n_cols}, got {hessian.numel()}", 4)
        _chk(weights, torch.float32)
        _chk(hessian, torch.float32)
        dev = weights.device
        nbytes = C.c_size_t(0)
        raise_for_status(_ffi.load().oxq_gptq_workspace_bytes(n_rows, n_cols, C.byref(nbytes)))
        ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
        q = torch.empty((n_rows, n_cols), dtype=torch.int32, device=dev)
        sc = torch.empty(n_cols, dtype=torch.float32, device=dev)
        zp = torch.empty(n_cols, dtype=torch.int32, device=dev)
        info = torch.zeros(2, dtype=torch.int32, device=dev)
        handle(dev.index).call("oxq_gptq_quantize_layer", _p(weights), n_rows, n_cols, _p(hessian), self.config.bits,
                               1 if self.config.symmetric else 0, C.c_double(self.config.percdamp), _p(q), _p(sc), _p(zp), _p(info),
                               _p(ws), nbytes.value)
        host = info.cpu()                                 # the reference returns the error synchronously: wait for the stream
        if int(host[0]) != 0:
            raise QuantError("SingularHessian", f"min_diag = {float(host[1:2].view(torch.float32)[0]):.3e}", 7)
        self.workspace = ws
        return GptqOutput(q, sc, zp, n_rows, n_cols)


def bias_add_(y: torch.Tensor, bias: torch.Tensor):
    """In place y[m, n] += bias[n] (bf16 matrix, f32 bias)."""
    _chk(bias, torch.float32)
    handle(y.device.index).call("oxq_bias_add_bf16", _p(y), y.stride(0), _p(bias), y.shape[0], y.shape[1])
    return y


# ------------------------------------------------------------------------------------------- GEMMs

def gemm_fp8(x_q, w_q, sx, sw, out: torch.Tensor | None = None):
    """Y = bf16((X . W^T) * sx * sw); x_q [M x K] u8, w_q [N x K] u8 (E4M3 bytes)."""
    m, k = x_q.shape
    n = w_q.shape[0]
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x_q.device) if out is None else out
    handle(x_q.device.index).call("oxq_gemm_fp8", m, n, k, _p(x_q), x_q.stride(0), _p(w_q), w_q.stride(0), _p(sx), _p(sw),
                                  _p(y), y.stride(0))
    return y


def gemm_fp8_ex(alpha: float, x_q, w_q, sx, sw, beta: float, y: torch.Tensor):
    """In place Y = alpha * (X . W^T) * sx * sw + beta * Y (gemm's general form, crates/oxicuda-blas/src/level3/gemm_api.rs:73-82)."""
    m, k = x_q.shape
    n = w_q.shape[0]
    handle(x_q.device.index).call("oxq_gemm_fp8_ex", m, n, k, C.c_float(alpha), _p(x_q), x_q.stride(0), _p(w_q), w_q.stride(0), _p(sx), _p(sw),
                                  C.c_float(beta), _p(y), y.stride(0))
    return y


def gemm_bf16_ex(alpha: float, x, w, beta: float, y: torch.Tensor):
    """In place Y = alpha * (X . W^T) + beta * Y on bf16 matrices."""
    m, k = x.shape
    n = w.shape[0]
    handle(x.device.index).call("oxq_gemm_bf16_ex", m, n, k, C.c_float(alpha), _p(x), x.stride(0), _p(w), w.stride(0), C.c_float(beta), _p(y), y.stride(0))
    return y


OP_K_MAJOR, OP_MN_MAJOR = 0, 1


def gemm_fp8_op(m: int, n: int, k: int, alpha: float, a, a_major: int, b, b_major: int, sa, sb, beta: float, y: torch.Tensor):
    """gemm's operand forms (crates/oxicuda-blas/src/level3/gemm_api.rs:73-82) for E4M3 operands: a is [m x k] (K-major) or
    [k x m] (MN-major) in memory, b is [n x k] (K-major) or [k x n] (MN-major); y [m x n] bf16 is updated in place."""
    handle(a.device.index).call("oxq_gemm_fp8_op", m, n, k, C.c_float(alpha), _p(a), a.stride(0), a_major, _p(b), b.stride(0), b_major,
                                _p(sa), _p(sb), C.c_float(beta), _p(y), y.stride(0))
    return y


def gemm_bf16_op(m: int, n: int, k: int, alpha: float, a, a_major: int, b, b_major: int, beta: float, y: torch.Tensor):
    handle(a.device.index).call("oxq_gemm_bf16_op", m, n, k, C.c_float(alpha), _p(a), a.stride(0), a_major, _p(b), b.stride(0), b_major,
                                C.c_float(beta), _p(y), y.stride(0))
    return y


def gemm_fp8_swiglu(x_q, w_gu_q, sx, sw, out: torch.Tensor | None = None):
    """H = bf16(silu(g) * u); w_gu_q holds gate/up rows interleaved in blocks of 128 (see interleave_gate_up)."""
    m, k = x_q.shape
    n2 = w_gu_q.shape[0]
    y = torch.empty((m, n2 // 2), dtype=torch.bfloat16, device=x_q.device) if out is None else out
    handle(x_q.device.index).call("oxq_gemm_fp8_swiglu", m, n2, k, _p(x_q), x_q.stride(0), _p(w_gu_q), w_gu_q.stride(0),
                                  _p(sx), _p(sw), _p(y), y.stride(0))
    return y


def gemm_bf16(x, w, out: torch.Tensor | None = None):
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device) if out is None else out
    handle(x.device.index).call("oxq_gemm_bf16", m, n, k, _p(x), x.stride(0), _p(w), w.stride(0), _p(y), y.stride(0))
    return y


def gemm_bf16_swiglu(x, w_gu, out: torch.Tensor | None = None):
    m, k = x.shape
    n2 = w_gu.shape[0]
    y = torch.empty((m, n2 // 2), dtype=torch.bfloat16, device=x.device) if out is None else out
    handle(x.device.index).call("oxq_gemm_bf16_swiglu", m, n2, k, _p(x), x.stride(0), _p(w_gu), w_gu.stride(0), _p(y),
                                y.stride(0))
    return y


def swiglu_interleaved(gu: torch.Tensor, out: torch.Tensor | None = None):
    """gu [m x 2n] bf16 in interleaved 128-column blocks -> silu(gate) * up [m x n]."""
    m, n2 = gu.shape
    y = torch.empty((m, n2 // 2), dtype=torch.bfloat16, device=gu.device) if out is None else out
    handle(gu.device.index).call("oxq_swiglu_interleaved", _p(gu), m, n2 // 2, _p(y))
    return y


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[inter x k] gate and up weights -> [2*inter x k] with blocks of 128 gate rows followed by the 128 matching
    up rows (a one-off, load-time layout change; inter must be a multiple of 128)."""
    inter, k = w_gate.shape
    assert inter % 128 == 0 and w_up.shape == w_gate.shape
    g = w_gate.reshape(inter // 128, 128, k)
    u = w_up.reshape(inter // 128, 128, k)
    return torch.stack([g, u], dim=1).reshape(2 * inter, k).contiguous()


def gemm_w8a8(x_q, w_q, sx_rows, sw_rows, out: torch.Tensor | None = None):
    m, k = x_q.shape
    n = w_q.shape[0]
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x_q.device) if out is None else out
    handle(x_q.device.index).call("oxq_gemm_w8a8", m, n, k, _p(x_q), x_q.stride(0), _p(w_q), w_q.stride(0), _p(sx_rows),
                                  _p(sw_rows), _p(y), y.stride(0))
    return y


def gemm_w8a32(x, w_q, sw_rows):
    m, k = x.shape
    n = w_q.shape[0]
    y = torch.empty((m, n), dtype=torch.float32, device=x.device)
    handle(x.device.index).call("oxq_gemm_w8a32", m, n, k, _p(x), _p(w_q), _p(sw_rows), _p(y))
    return y


def gemm_w4a16_workspace(m: int, n: int, k: int, device) -> torch.Tensor:
    """Zero-filled workspace; every call leaves it zero-filled again, so it can be reused."""
    nbytes = int(_ffi.load().oxq_gemm_w4a16_workspace_bytes(m, n, k))
    return torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=device)


def gemm_w4a16(x, codes, scales, zeros, group: int = 128, workspace: torch.Tensor | None = None,
               out: torch.Tensor | None = None):
    m, k = x.shape
    n = codes.shape[0]
    ws = gemm_w4a16_workspace(m, n, k, x.device) if workspace is None else workspace
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device) if out is None else out
    handle(x.device.index).call("oxq_gemm_w4a16", m, n, k, _p(x), _p(codes), _p(scales), _p(zeros), group, _p(y), _p(ws),
                                ws.numel())
    return y


def gemm_mxfp8(x_codes, x_sf_mma, w_codes, w_sf_mma, out: torch.Tensor | None = None):
    m, k = x_codes.shape
    n = w_codes.shape[0]
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x_codes.device) if out is None else out
    handle(x_codes.device.index).call("oxq_gemm_mxfp8", m, n, k, _p(x_codes), _p(x_sf_mma), _p(w_codes), _p(w_sf_mma),
                                      _p(y), y.stride(0))
    return y


def gemm_nvfp4(x_packed, x_sf_mma, x_stats, w_packed, w_sf_mma, w_stats, out: torch.Tensor | None = None):
    """x_stats / w_stats are the 2-float tensors of nvfp4_quant; element 1 is the tensor scale."""
    m, k = x_packed.shape[0], x_packed.shape[1] * 2
    n = w_packed.shape[0]
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x_packed.device) if out is None else out
    handle(x_packed.device.index).call("oxq_gemm_nvfp4", m, n, k, _p(x_packed), _p(x_sf_mma), _p(x_stats[1:]),
                                       _p(w_packed), _p(w_sf_mma), _p(w_stats[1:]), _p(y), y.stride(0))
    return y


# ------------------------------------------------------------------------------------------- collective

def multimem_all_reduce_bf16(multicast_ptr: int, numel: int, rank: int, world: int, device_index: int | None = None):
    """In-place all-reduce over the multicast mapping of a symmetric bf16 buffer; the caller provides the barriers."""
    handle(device_index).call("oxq_multimem_all_reduce_bf16", C.c_void_p(multicast_ptr), numel, rank, world)


def multimem_all_reduce_bf16_2d_sync(multicast_ptr: int, rows: int, cols: int, ld: int, rank: int, world: int, flags_local: torch.Tensor,
                                     flags_multicast_ptr: int, device_index: int | None = None):
    """In-place all-reduce of a column block of a symmetric bf16 matrix with the cross-rank synchronisation inside the kernel."""
    handle(device_index).call("oxq_multimem_all_reduce_bf16_2d_sync", C.c_void_p(multicast_ptr), rows, cols, ld, rank, world, _p(flags_local),
                              C.c_void_p(flags_multicast_ptr))


def gemm_fp8_all_reduce(x_q, w_q, sx, sw, y_local: torch.Tensor, y_multicast_ptr: int, flags_local: torch.Tensor, flags_multicast_ptr: int,
                        rank: int, world: int):
    """FP8 GEMM of this rank's K-shard with the all-reduce over the ranks fused in (RowLinear::forward_partial + all_reduce):
    y_local is this rank's [m x n] view of a symmetric bf16 buffer, flags_local its int32 flag words (zero before the first
    call); the *_multicast_ptr arguments are the multicast addresses of the same two buffers."""
    m, k = x_q.shape
    n = w_q.shape[0]
    handle(x_q.device.index).call("oxq_gemm_fp8_all_reduce", m, n, k, _p(x_q), x_q.stride(0), _p(w_q), w_q.stride(0), _p(sx), _p(sw), _p(y_local),
                                  C.c_void_p(y_multicast_ptr), y_local.stride(0), _p(flags_local), C.c_void_p(flags_multicast_ptr),
                                  flags_local.numel(), rank, world)
    return y_local


def multimem_all_reduce_bf16_2d(multicast_ptr: int, rows: int, cols: int, ld: int, rank: int, world: int, device_index: int | None = None):
    """In-place all-reduce of a [rows x cols] column block (leading dimension ld) of a symmetric bf16 matrix."""
    handle(device_index).call("oxq_multimem_all_reduce_bf16_2d", C.c_void_p(multicast_ptr), rows, cols, ld, rank, world)
