"""Real selective scan of the Mamba block on B200.

``selective_scan_fn`` has the signature and semantics of the function the
reference's ``MambaBlock.ssm_mamba`` imports from the third-party package
mamba-ssm (ai-modules/wavesAI/model/aussm.py:30, :791-802):

    out = selective_scan_fn(u, delta, A, B, C, D=None, z=None, delta_bias=None,
                            delta_softplus=False, return_last_state=False)

with ``u, delta, z`` of shape ``(b, d, l)``, ``A`` ``(d, n)``, ``B, C`` ``(b, n, l)``
(input-dependent, shared by all channels), ``D, delta_bias`` ``(d,)``.  All
arithmetic runs in libaussm_b200.so; CUDA float32 tensors only.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F
from torch import Tensor

from . import _lib
from .ops import _f32c, _ptr, _stream, _workspace

__all__ = ["selective_scan_fn"]


class _SelectiveScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, B, C, D, z, delta_bias, delta_softplus, want_state):
        b, d, l = u.shape
        n = A.shape[1]
        u, delta = _f32c("u", u, (b, d, l)), _f32c("delta", delta, (b, d, l))
        A = _f32c("A", A, (d, n))
        B, C = _f32c("B", B, (b, n, l)), _f32c("C", C, (b, n, l))
        D = None if D is None else _f32c("D", D, (d,))
        z = None if z is None else _f32c("z", z, (b, d, l))
        delta_bias = None if delta_bias is None else _f32c("delta_bias", delta_bias, (d,))
        pad = (-l) % 4                      # the kernels stage 16-byte pieces of the time axis
        if pad:
            u, delta, B, C = (F.pad(t, (0, pad)).contiguous() for t in (u, delta, B, C))
            z = None if z is None else F.pad(z, (0, pad)).contiguous()
        lp = l + pad
        lib = _lib.load()
        out = torch.empty_like(u)
        ckpt = torch.empty(lib.aussm_b200_selective_scan_ckpt_floats(b, d, n, lp), device=u.device,
                           dtype=torch.float32)
        last = torch.empty(b, d, n, device=u.device, dtype=torch.float32) if (want_state and not pad) else None
        with torch.cuda.device(u.device):
            rc = lib.aussm_b200_selective_scan_fwd(_ptr(u), _ptr(delta), _ptr(A), _ptr(B), _ptr(C), _ptr(D), _ptr(z),
                                                   _ptr(delta_bias), int(bool(delta_softplus)), _ptr(out), _ptr(ckpt),
                                                   _ptr(last), b, d, n, lp, _stream(u))
        _lib.check(rc, "selective_scan forward")
        if want_state and pad:
            raise RuntimeError("return_last_state needs a sequence length that is a multiple of 4")
        ctx.save_for_backward(u, delta, A, B, C, D, z, delta_bias, ckpt)
        ctx.meta = (b, d, n, l, lp, bool(delta_softplus))
        ctx.mark_non_differentiable(*([last] if last is not None else []))
        return out[..., :l] if pad else out, last

    @staticmethod
    def backward(ctx, gout, _glast):
        u, delta, A, B, C, D, z, delta_bias, ckpt = ctx.saved_tensors
        b, d, n, l, lp, softplus = ctx.meta
        lib = _lib.load()
        gout = _f32c("grad_out", gout, (b, d, l))
        if lp != l:
            gout = F.pad(gout, (0, lp - l)).contiguous()
        du, ddelta = torch.empty_like(u), torch.empty_like(u)
        dz = None if z is None else torch.empty_like(u)
        dA = torch.empty_like(A)
        dB, dC = torch.empty_like(B), torch.empty_like(C)
        dD = None if D is None else torch.empty_like(D)
        dbias = None if delta_bias is None else torch.empty_like(delta_bias)
        with torch.cuda.device(u.device):
            ws = _workspace(lib.aussm_b200_selective_scan_bwd_workspace_bytes(b, d, n, lp), u.device)
            rc = lib.aussm_b200_selective_scan_bwd(_ptr(gout), _ptr(u), _ptr(delta), _ptr(A), _ptr(B), _ptr(C), _ptr(D),
                                                   _ptr(z), _ptr(delta_bias), int(softplus), _ptr(ckpt), _ptr(du),
                                                   _ptr(ddelta), _ptr(dA), _ptr(dB), _ptr(dC), _ptr(dD), _ptr(dz),
                                                   _ptr(dbias), b, d, n, lp, _ptr(ws), ws.numel(), _stream(u))
        _lib.check(rc, "selective_scan backward")
        if lp != l:
            du, ddelta, dB, dC = du[..., :l], ddelta[..., :l], dB[..., :l], dC[..., :l]
            dz = None if dz is None else dz[..., :l]
        return du, ddelta, dA, dB, dC, dD, dz, dbias, None, None


def selective_scan_fn(u: Tensor, delta: Tensor, A: Tensor, B: Tensor, C: Tensor, D: Optional[Tensor] = None,
                      z: Optional[Tensor] = None, delta_bias: Optional[Tensor] = None, delta_softplus: bool = False,
                      return_last_state: bool = False):
    """Selective scan; returns ``out`` or ``(out, last_state)`` with ``last_state`` of shape ``(b, d, n)``."""
    out, last = _SelectiveScan.apply(u, delta, A, B, C, D, z, delta_bias, delta_softplus, return_last_state)
    return (out, last) if return_last_state else out
