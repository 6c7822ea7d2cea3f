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
    fused_decode: bool = False    # steps of up to 8 single tokens as ONE persistent kernel (slower than the chain of kernels so far)

    def __post_init__(self) -> None:
        import os
        if os.environ.get("NANOINFER_B200_MID_BATCH"):          # for measurements: which projections take the swapped kernel
            self.mid_batch_mask = int(os.environ["NANOINFER_B200_MID_BATCH"])
        self._workspaces = {}
        self._retired = []
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

    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
               residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """y[M, N] = x[M, K] . w[N, K]^T.  ``out_dtype`` float32 asks for FP32 results
        (logits); the default is the compute dtype.  With ``residual`` (the FP32 residual
        stream) the kernel MAY add the product into it and return None; otherwise the product
        is returned and the caller adds it."""
        m, n = x.shape[0], w.shape[0]
        out_dtype = out_dtype or self.dtype
        if self.dtype == torch.float32:
            out = self.empty(m, n, dtype=torch.float32)
            ops.gemm_f32(x, w, out)
            return out
        if residual is None and self.swapped_gemm(m, n, x.shape[1]):
            out = self.empty(m, n, dtype=out_dtype)
            ops.gemm_swap_tc(x, w, out, ops.STORE_BF16 if out_dtype == torch.bfloat16 else ops.STORE_F32)
            return out
        return ops.linear_bf16(x, w, out_dtype, residual)

    def skinny(self, n_rows: int, k: int) -> bool:
        """True if a product of n_rows activations with inner size k goes to the package's own
        bandwidth kernel (and so may carry fused prologues and epilogues)."""
        return self.dtype == torch.bfloat16 and 0 < n_rows <= ops.SKINNY_ROWS and k % 8 == 0

    # Which projections of a step of 9 .. 128 rows go to the package's swapped-operand tcgen05 kernel
    # (with their neighbours fused into its epilogue) instead of the library product followed by
    # separate element-wise kernels.
    MID_QKV, MID_OUT, MID_GATE_UP, MID_DOWN, MID_HEAD = 1, 2, 4, 8, 16
    mid_batch_mask: int = MID_HEAD

    def mid_batch(self, n_rows: int, k: int, which: int) -> bool:
        """True if projection ``which`` (one of the MID_* bits) of n_rows rows with inner size k
        takes the swapped-operand kernel."""
        return (self.dtype == torch.bfloat16 and ops.SKINNY_ROWS < n_rows <= ops.SWAP_MAX_ROWS and k % 8 == 0
                and bool(self.mid_batch_mask & which))

    def swapped_gemm(self, n_rows: int, n_out: int, k: int, fused: bool = False) -> bool:
        """True if a plain product of 9..128 rows goes to the package's swapped-operand tcgen05 kernel:
        an output projection over a vocabulary (blocks stream several tiles each: 5.9 TB/s of weights
        against 5.7 for the library product)."""
        if self.dtype != torch.bfloat16 or not ops.SKINNY_ROWS < n_rows <= ops.SWAP_MAX_ROWS or k % 8:
            return False
        tiles = -(-n_out // 128)
        return tiles >= 4 * ops.sm_count(self.device) and bool(self.mid_batch_mask & self.MID_HEAD)

    def tensor_core_gemm(self, n_rows: int, k: int) -> bool:
        """True if a product with this many rows goes to the package's tcgen05 kernel (where
        its fused epilogue beats the library product followed by a separate kernel)."""
        return self.dtype == torch.bfloat16 and n_rows >= 256 and k % 8 == 0

    def workspace(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A persistent scratch tensor of at least ``numel`` elements, shared by all layers
        (they run one after the other on one stream).  ``zero``: zero-filled when created;
        its users leave it zero."""
        t = self._workspaces.get(name)
        if t is None or t.numel() < numel or t.dtype != dtype:
            if torch.cuda.is_current_stream_capturing():
                raise ops.KernelError(f"workspace '{name}' would have to grow during graph capture")
            n = max(numel, 2 * t.numel() if t is not None else 0)
            if t is not None:
                self._retired.append(t)   # captured graphs may still point at the smaller one
            t = (torch.zeros if zero else torch.empty)(n, dtype=dtype, device=self.device)
            self._workspaces[name] = t
        return t
