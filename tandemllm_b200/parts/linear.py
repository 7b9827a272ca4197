"""The one place a weight matrix is multiplied: `linear(runtime, x, w)` = x @ w^T (+ bias).

32-bit tensors go to the CUDA-core kernel (true 32-bit: no tensor-core mode is involved). bfloat16
tensors go to the runtime's tensor-core kernels when it has them, else to the same CUDA-core kernel
with 32-bit accumulation. The reference routes every product through one function for the same reason
(`lin`, engine/models/lfm2_moe/ref.py:99-103; engine.py:184-197).
"""

from __future__ import annotations

import torch

from ..kernels import ops


def linear(runtime, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    M, N = x.shape[0], w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or x.dtype, device=x.device)
    if M == 0:
        return out
    tc = runtime.tensorcore
    if tc is not None and x.dtype == torch.bfloat16 and tc.linear(x, w, bias, out):
        return out
    return ops.gemm_simt(x, w, bias, out)
