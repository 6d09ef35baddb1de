"""PyTorch custom operator for a linear layer over a bitmap-v3 weight.

    torch.ops.spmspm_b200.sparse_linear(x, vals, gtile, mtile, bitmap, max_nnz, M, bias, residual, activation, split_k)

computes residual + act(x @ W^T + bias) for W in bitmap-v3 form, with the element-wise steps folded into the SpMM's
own launches (spb_linear_bitmap_v3): the call FasterTransformer's OPT decoder makes around each of its four GEMMs
(third_party/ft_spinfer.patch:623-862, 1459-1573, 1704-1811).  `SparseLinear` is the module form.  The operator is
registered with a shape function, so it can be traced (FakeTensor) and captured in CUDA graphs; it is inference-only
(no autograd formula) and has no CPU implementation: without the CUDA library the call raises.
"""
from typing import Optional

import torch

from . import api

ACT_NONE, ACT_RELU = api.ACT_NONE, api.ACT_RELU


@torch.library.custom_op("spmspm_b200::sparse_linear", mutates_args=(), device_types="cuda")
def sparse_linear(x: torch.Tensor, vals: torch.Tensor, gtile: torch.Tensor, mtile: torch.Tensor, bitmap: torch.Tensor,
                  max_nnz: torch.Tensor, M: int, bias: Optional[torch.Tensor], residual: Optional[torch.Tensor],
                  activation: int, split_k: int) -> torch.Tensor:
    """x [N, K] fp16 -> [N, M] fp16.  split_k <= 0: let the library choose."""
    W = api.BitmapMatrix(M, x.shape[1], vals, gtile, mtile, bitmap, max_nnz)
    return api.linear(W, x, bias=bias, residual=residual, activation=activation, split_k=split_k if split_k > 0 else None)


@sparse_linear.register_fake
def _(x, vals, gtile, mtile, bitmap, max_nnz, M, bias, residual, activation, split_k):
    return x.new_empty((x.shape[0], M))


class SparseLinear(torch.nn.Module):
    """y = residual + act(x W^T + b) with W held in bitmap-v3 form (buffers, so that .to() and state_dict() carry
    them).  `weight`: an spmspm_b200.BitmapMatrix; `bias`: fp16 [M] or None."""

    def __init__(self, weight, bias=None, activation=ACT_NONE, split_k=0):
        super().__init__()
        self.M, self.K = weight.M, weight.K
        self.activation, self.split_k = int(activation), int(split_k)
        for name in ("vals", "gtile", "mtile", "bitmap", "max_nnz"):
            self.register_buffer(name, getattr(weight, name))
        self.register_buffer("bias", bias)

    def forward(self, x, residual=None):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.K).contiguous()
        r2 = residual.reshape(-1, self.M).contiguous() if residual is not None else None
        y = torch.ops.spmspm_b200.sparse_linear(x2, self.vals, self.gtile, self.mtile, self.bitmap, self.max_nnz, self.M,
                                                self.bias, r2, self.activation, self.split_k)
        return y.reshape(*lead, self.M)
