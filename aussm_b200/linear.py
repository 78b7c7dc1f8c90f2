"""Float32-accurate linear layers on the tensor cores.

The reference's blocks run their ``nn.Linear`` projections (in_proj, out_proj, x_proj, dt_proj; aussm.py:735-761,
:826-848) as float32 matrix products, which the library routes to SIMT SGEMM kernels (about 45 TFLOP/s on B200).
``SplitLinear`` is ``nn.Linear`` (same parameters, same ``state_dict`` keys) whose forward and backward products go
through the three-term split GEMM of this library (``aussm_b200_gemm_split3``: float32-level accuracy on tcgen05),
for CUDA float32 inputs whose feature sizes are multiples of 4; anything else takes ``F.linear``.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .variants import _gemm

__all__ = ["split_linear", "SplitLinear"]

# Below this many floating-point operations per product the library SGEMM is as fast (the split GEMM runs two
# passes over each operand to take its FP16 parts before the product starts).
MIN_FLOP = 2.0e10


class _SplitLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d: Tensor, weight: Tensor):
        rows, d_in = x2d.shape
        d_out = weight.shape[0]
        out = torch.empty(rows, d_out, device=x2d.device, dtype=torch.float32)
        # out (rows x d_out) = x (rows x d_in, K contiguous) * weight (d_out x d_in, K contiguous)
        _gemm(x2d, 0, 0, weight, 0, 0, out, rows, d_out, d_in, 1, 0)
        ctx.save_for_backward(x2d, weight)
        return out

    @staticmethod
    def backward(ctx, g: Tensor):
        x2d, weight = ctx.saved_tensors
        rows, d_in = x2d.shape
        d_out = weight.shape[0]
        g = g.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = torch.empty_like(x2d)
            # gx (rows x d_in) = g (rows x d_out, K contiguous) * weight^T: weight stored (K = d_out) x (N = d_in)
            _gemm(g, 0, 0, weight, 1, 0, gx, rows, d_in, d_out, 1, 0)
        if ctx.needs_input_grad[1]:
            # gw (d_out x d_in) = g^T x: both stored with the contraction index (rows) as the slow one.  The output
            # has few tiles and a very long contraction, so the rows are cut into `nb` slices that run as independent
            # batch entries (one partial product each) and are added afterwards.
            tiles = ((d_out + 127) // 128) * ((d_in + 255) // 256)
            nb = 1
            while tiles * nb < 148 and rows % (2 * nb) == 0 and rows // (2 * nb) >= 512:
                nb *= 2
            if nb == 1:
                gw = torch.empty_like(weight)
                _gemm(g, 1, 0, x2d, 1, 0, gw, d_out, d_in, rows, 1, 0)
            else:
                part = torch.empty(nb, d_out, d_in, device=weight.device, dtype=torch.float32)
                _gemm(g, 1, 1, x2d, 1, 1, part, d_out, d_in, rows // nb, nb, 0)
                gw = part.sum(0)
        return gx, gw


def split_linear(x: Tensor, weight: Tensor, bias: Tensor = None) -> Tensor:
    """``F.linear(x, weight, bias)`` with the product on the split GEMM when the layout allows."""
    d_out, d_in = weight.shape
    rows = x.numel() // max(1, d_in)
    ok = (x.is_cuda and x.dtype == torch.float32 and weight.dtype == torch.float32 and d_in % 4 == 0
          and d_out % 4 == 0 and x.numel() > 0 and 2.0 * rows * d_in * d_out >= MIN_FLOP)
    if not ok:
        return F.linear(x, weight, bias)
    x2d = x.reshape(-1, d_in).contiguous()
    out = _SplitLinear.apply(x2d, weight.contiguous())
    if bias is not None:
        out = out + bias
    return out.view(*x.shape[:-1], d_out)


class SplitLinear(nn.Linear):
    def forward(self, x: Tensor) -> Tensor:
        return split_linear(x, self.weight, self.bias)
