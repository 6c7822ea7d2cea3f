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

    # From how many (token, kv head) pairs on a step's single-token attention takes the kernel that
    # deals the keys evenly over a fixed grid (0: one pair per SM, set when the device is known), and
    # whether heads of 64 take it too.  Measured in the step (ms per step, split kernel / balanced):
    # heads of 128: 3B batch 32 3.78 / 3.65, 8B batch 64 at context 6,144 13.62 / 13.27, the continuous
    # workload (3B, contexts of all lengths) 5.65k / 6.46k generated tokens a second.  Heads of 64 with
    # equal contexts: batch 24 1.44 / 1.39, but batch 32 1.36 / 1.45 and batch 64 1.76 / 1.85 - there it
    # only wins when the contexts differ (alone, contexts from a quarter to all of 3,072: batch 32
    # 37.6 / 33.7 us, batch 64 65.1 / 56.9 us), which a replayed graph cannot know; so it is off for them.
    balanced_attention_pairs: int = 0
    balanced_attention_narrow_heads: bool = False

    def balanced_attention(self, n_tokens: int, n_kv_heads: int, head_dim: int) -> bool:
        return (n_tokens * n_kv_heads > self.balanced_attention_pairs
                and (head_dim > 64 or self.balanced_attention_narrow_heads))

    def __post_init__(self) -> None:
        import os
        if os.environ.get("NANOINFER_B200_MID_BATCH"):          # for measurements: which projections take the swapped kernel
            self.mid_batch_mask = int(os.environ["NANOINFER_B200_MID_BATCH"])
        if os.environ.get("NANOINFER_B200_WARM"):               # for measurements: "<product KiB>,<attention KiB>"
            a, b, c = os.environ["NANOINFER_B200_WARM"].split(",")
            self.warm_bytes, self.warm_attention_bytes, self.warm_mask = int(a) << 10, int(b) << 10, int(c)
        if os.environ.get("NANOINFER_B200_NORM_HANDOFF"):       # for measurements: 0 switches it off
            self.norm_handoff = bool(int(os.environ["NANOINFER_B200_NORM_HANDOFF"]))
        if os.environ.get("NANOINFER_B200_BALANCED"):           # for measurements: "<pairs>,<0|1: heads of 64 too>"
            a, b = os.environ["NANOINFER_B200_BALANCED"].split(",")
            self.balanced_attention_pairs, self.balanced_attention_narrow_heads = int(a), bool(int(b))
        self._workspaces = {}
        self._retired = []
        ops.require_cuda()
        if self.device.type != "cuda":
            raise ops.KernelError(f"device {self.device} is not a CUDA device; there is no CPU path")
        if self.balanced_attention_pairs <= 0:
            self.balanced_attention_pairs = ops.sm_count(self.device)

    def weight(self, t: torch.Tensor) -> torch.Tensor:
        """A matrix weight on the device in the compute dtype."""
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def gain(self, t: torch.Tensor) -> torch.Tensor:
        """A norm gain on the device; gains are applied in FP32."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    def empty(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, device=self.device, dtype=dtype or self.dtype)

    # Asking weights into L2 ahead of their kernel (single-token steps).  A kernel of a few
    # microseconds leaves the memory system idle while its last blocks merge and write and the next
    # kernel's blocks start.  The decode attention therefore asks for its output projection when it
    # starts and, once a block's own stream has ended, for the first warm_attention_bytes of the matrix
    # after that (a third of that for a lone token, whose attention is over too soon for more); the
    # output projection goes on from there for warm_bytes.  Measured on the 1B sizes at context 2,048
    # (ms per step, without / with): batch 1 0.801 / 0.791, 2 0.836 / 0.814, 4 0.854 / 0.829,
    # 8 0.865 / 0.838.  More does not help (32 MiB: 0.842; 40 MiB: 0.848), nor does the same request at
    # the end of gate/up (for the down projection: 0.855 - that kernel runs at its register limit and
    # is 6 % slower with the code in it) or of the down projection (for the next layer: 0.842).
    warm_bytes: int = 12 << 20
    warm_attention_bytes: int = 24 << 20
    warm_mask: int = 1          # which products ask: 1 a mixer's output projection, 2 gate/up, 4 down

    def warm(self, tensor, first: int, nbytes: Optional[int] = None, which: int = 0):
        """A hint (tensor, first byte, bytes) for a kernel's ``warm`` argument, or None."""
        nbytes = self.warm_bytes if nbytes is None else nbytes
        if which and not self.warm_mask & which:
            return None
        return (tensor, first, nbytes) if nbytes > 0 and tensor is not None else None

    def warm_after(self, ctx, skip: int = 0, which: int = 0):
        """The hint for the matrix that is read after the running part (ctx.read_after)."""
        nxt = ctx.read_after[0] if ctx is not None and ctx.read_after else None
        return self.warm(nxt, skip, which=which)

    def warm_attention(self, w_out, ctx):
        """The decode attention's two hints: its own output projection, the head of what follows."""
        if not ctx.decode_only or (self.warm_bytes <= 0 and self.warm_attention_bytes <= 0):
            return ()
        nxt = ctx.read_after[0] if ctx.read_after else None
        return (self.warm(w_out, 0, w_out.numel() * w_out.element_size()), self.warm(nxt, 0, self.attention_share(ctx)))

    def attention_share(self, ctx) -> int:
        """How much of the matrix after its output projection the decode attention of this step asks for."""
        return self.warm_attention_bytes // 3 if ctx.n_tokens == 1 else self.warm_attention_bytes

    # Handing a norm from the kernel that adds into the residual stream to the kernel that reads it
    # (steps of up to 8 rows): the adding product also stores bfloat16(h * gain) and partial sums of
    # h^2, the reading product takes that as its input and scales its results by 1/rms - so the
    # readers (gate/up, QKV) no longer read and normalise the FP32 stream themselves.  Measured on the
    # decode step with the readers' norm simply left out (an upper bound): batch 8 0.796 -> 0.719 ms.
    norm_handoff: bool = True

    @staticmethod
    def fuses_norm(norm) -> bool:
        """True if the skinny products can run this norm inside themselves (RMSNorm with gain and eps)."""
        return getattr(norm, "fused_kind", None) == "rmsnorm" and hasattr(norm, "gain") and hasattr(norm, "eps")

    def handoff(self, norm, n_rows: int, n_out: int, k: int):
        """A NormHandoff for ``norm`` to be filled by the product that adds [n_rows, n_out] into the
        stream (inner size k), or None where that is not possible."""
        if (not self.norm_handoff or norm is None or not self.fuses_norm(norm) or self.dtype != torch.bfloat16
                or not 0 < n_rows <= ops.HANDOFF_ROWS or k % 8 or not ops.gemv_reads_handoff(n_rows, n_out)):
            return None
        tiles = ops.gemv_out_tiles(n_rows, n_out, k)          # 0: the adding kernel for these sizes cannot prepare it
        return ops.NormHandoff(norm, norm.gain, norm.eps, n_rows, n_out, tiles, self.device) if tiles > 0 else None

    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
               residual: Optional[torch.Tensor] = None, warm=None, handoff=None) -> Optional[torch.Tensor]:
        """y[M, N] = x[M, K] . w[N, K]^T.  ``out_dtype`` float32 asks for FP32 results
        (logits); the default is the compute dtype.  With ``residual`` (the FP32 residual
        stream) the kernel MAY add the product into it and return None; otherwise the product
        is returned and the caller adds it.  ``warm``: a hint that the skinny kernel takes (see warm())."""
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
        return ops.linear_bf16(x, w, out_dtype, residual, warm, handoff)

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
