"""Helpers shared by the GPU parity tests (numpy <-> torch conversions without value changes)."""
import numpy as np
import torch


def dev():
    return torch.device("cuda:0")


def to_dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev())


def bf16_dev(bits_u16: np.ndarray) -> torch.Tensor:
    """uint16 bf16 bit patterns -> bfloat16 device tensor."""
    return torch.from_numpy(np.ascontiguousarray(bits_u16).view(np.int16)).to(dev()).view(torch.bfloat16)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def u32(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy().view(np.uint32)


def u16(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def ulp_diff_f32(a: np.ndarray, b: np.ndarray) -> int:
    ai = np.ascontiguousarray(a, np.float32).view(np.int32).astype(np.int64)
    bi = np.ascontiguousarray(b, np.float32).view(np.int32).astype(np.int64)
    return int(np.abs(ai - bi).max()) if ai.size else 0


def sf_to_mma_layout(sf: np.ndarray) -> np.ndarray:
    """Row-major scale factors [rows x cols] -> 128x4 tiled byte order (numpy restatement of the layout)."""
    rows, cols = sf.shape
    rt, ct = (rows + 127) // 128, (cols + 3) // 4
    out = np.zeros(rt * ct * 512, np.uint8)
    r, c = np.meshgrid(np.arange(rows), np.arange(cols), indexing="ij")
    off = ((r // 128) * ct + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
    out[off.ravel()] = sf.ravel()
    return out
