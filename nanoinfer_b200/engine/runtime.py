"""Runtime: device, compute dtype and the matrix products of the forward pass.

float32 is a true 32-bit path: every product runs through the package's own FFMA kernel
and no reduced-precision tensor-core mode is ever switched on.  bfloat16 keeps weights,
activations and cache in bfloat16 with FP32 accumulation; the residual stream, norm
statistics, softmax and rotation angles stay FP32 in both.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..kernels import ops

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16,
           "bf16": torch.bfloat16}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype {name} is not supported (float32 or bfloat16)")
        return name
    if name not in _DTYPES:
        raise ValueError(f"dtype '{name}' is not supported (float32 or bfloat16)")
    return _DTYPES[name]


@dataclass
class Runtime:
    device: torch.device
    dtype: torch.dtype
    page_size: int

    def __post_init__(self) -> None:
        ops.require_cuda()
        if self.device.type != "cuda":
            raise ops.KernelError(f"device {self.device} is not a CUDA device; there is no CPU path")

    def weight(self, t: torch.Tensor) -> torch.Tensor:
        """A matrix weight on the device in the compute dtype."""
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def gain(self, t: torch.Tensor) -> torch.Tensor:
        """A norm gain on the device; gains are applied in FP32."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    def empty(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, device=self.device, dtype=dtype or self.dtype)

    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None
               ) -> torch.Tensor:
        """y[M, N] = x[M, K] . w[N, K]^T.  ``out_dtype`` float32 asks for FP32 results
        (logits); the default is the compute dtype."""
        m, n = x.shape[0], w.shape[0]
        out_dtype = out_dtype or self.dtype
        if self.dtype == torch.float32:
            out = self.empty(m, n, dtype=torch.float32)
            ops.gemm_f32(x, w, out)
            return out
        return ops.linear_bf16(x, w, out_dtype)
