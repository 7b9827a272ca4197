"""The one place a weight matrix is multiplied: `linear(runtime, x, w)` = x @ w^T (+ bias).

32-bit tensors go to the CUDA-core kernel (true 32-bit: no tensor-core mode is involved). bfloat16
tensors go to the runtime's tensor-core kernels when it has them, else to the same CUDA-core kernel
with 32-bit accumulation. The reference routes every product through one function for the same reason
(`lin`, engine/models/lfm2_moe/ref.py:99-103; engine.py:184-197).

With `defer` (a branch's last product, whose result only goes into the residual) the result may come back as
`ops.PartialSums` instead of a tensor: partial sums that the consuming norm kernel adds itself. `defer="rounded"`
allows the same for a result of any precision, whose consumer adds the sums and rounds them as the product would
have. `ops.materialize` turns any such result into a plain tensor.
"""

from __future__ import annotations

import torch

from ..kernels import ops


def linear(runtime, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None, defer: bool = False):
    M, N = x.shape[0], w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or x.dtype, device=x.device)
    if M == 0:
        return out
    tc = runtime.tensorcore
    if tc is not None and x.dtype == torch.bfloat16:
        done = tc.linear(x, w, bias, out, defer=defer)
        if done is True:
            return out
        if done is not False:
            return done
    return ops.gemm_simt(x, w, bias, out)
