"""Matrix products of the decoder: ``y = x . W^T`` with ``W`` kept in the
checkpoint's ``[out, in]`` layout (the reference transposes to ``[in, out]``
for cuBLAS, infernum/src/weights ... generic_impl.rs:107-131; K-major rows are
what both the plain kernel and a tensor-core ``A . B^T`` tile want, so no
transpose is made here).

Which routine runs:
  * engine in float32, or a weight that is stored in 32-bit: the package's
    plain kernel, 32-bit fused multiply-adds in k order (no tensor cores, no
    reduced-precision mode);
  * bfloat16 activations and weights: the library GEMM (cuBLAS through
    ``torch.mm``, 32-bit accumulation), where the reference also calls cuBLAS
    (infernum-cuda/src/inner/cuda/ops/matmul.rs:92-116), or this package's own
    small-batch kernel when one is registered for the shape.
"""

from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..errors import KernelError
from ..ops import core

# Optional hand-written bf16 GEMM routes: callables (x, w, out, err) -> bool that
# return True when they took the product.  Filled by ops modules at import.
BF16_ROUTES: List[Callable[..., bool]] = []


def matmul_nt(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
              out: Optional[torch.Tensor] = None, err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [M, K] @ w [N, K]^T -> [M, N]`` in ``out_dtype`` (default: x's).
    ``err``: the device error word in which the package's tensor-core kernels
    report a wait that ran out (the engine's, so that its check sees it)."""
    core.require_cuda(x, w)
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise KernelError(f"matmul_nt: cannot multiply {tuple(x.shape)} by {tuple(w.shape)}^T")
    out_dtype = out_dtype or x.dtype
    M, N = x.shape[0], w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if not BF16_ROUTES:
            from ..ops import gemm_tc

            BF16_ROUTES.append(gemm_tc.route)
        for route in BF16_ROUTES:
            if route(x, w, out, err):
                return out
        if out_dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        else:
            out.copy_(torch.mm(x, w.t(), out_dtype=torch.float32))
        core.profile_mark("library_gemm")
        return out
    core.gemm_plain(x, w, out)
    return out


class Linear:
    """A weight and its product; ``parts`` own these, they are not parts."""

    def __init__(self, weight: torch.Tensor, rt=None):
        if weight.dim() != 2:
            raise KernelError("Linear: weight must be [out, in]")
        self.weight = weight.contiguous()
        self.rt = rt  # the owning part's Runtime: its error word is handed to the kernels

    @property
    def err(self) -> Optional[torch.Tensor]:
        return self.rt.error_word() if self.rt is not None else None

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    @property
    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return matmul_nt(x, self.weight, out_dtype, err=self.err)
