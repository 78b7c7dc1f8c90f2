"""Complex and positive-real variants of the adaptive selective scan on B200.

The reference compiles kernels for these (csrc/cuda/ssm_adaptive_complex.cu,
ssm_adaptive_real.cu) but never registers or wraps them; what it does define is
their PyTorch loop references, whose signatures these functions take:

    ssm_adaptive_complex(u, dt, x, B, C, D, z)   x: (2, d, n, d) [rho, theta rows];  B, C complex (b, n, l)
    ssm_adaptive_preal(u, dt, x, B, C, D, z)     x: (d, n, d);                       B, C real (b, n, l)
    (extension-cpp/extension_cpp/ops.py:233-297 and :300-357)

Both are a projection (eigenvalue exponent = x . u, a dense contraction that
runs on the tcgen05 GEMM of the library) followed by the scan core
``scan_complex`` on the resulting (rho, theta).  Phase/log-magnitude tensors of
shape (b, d, n, l) are materialised for the whole sequence here (no time
windows yet).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F
from torch import Tensor

from . import _lib
from .ops import _f32c, _library, _ptr, _stream, _workspace

__all__ = ["scan_complex", "project", "ssm_adaptive_complex", "ssm_adaptive_preal"]


def _gemm(A, a_mn, a_b, B, b_mn, b_b, C, M, N, K, batches, reduce, beta=0):
    lib = _lib.load()
    with torch.cuda.device(C.device):
        ws = _workspace(lib.aussm_b200_gemm_split3_workspace_bytes(M, N, K, batches, a_mn, a_b, b_mn, b_b), C.device)
        rc = lib.aussm_b200_gemm_split3(_ptr(A), a_mn, a_b, _ptr(B), b_mn, b_b, _ptr(C), M, N, K, batches, reduce, beta,
                                        _ptr(ws), ws.numel(), _stream(C))
    _lib.check(rc, "gemm_split3")


class _Projection(torch.autograd.Function):
    """A[b] = W @ u[b]  with W (m, d), u (b, d, l) -> (b, m, l); d and l multiples of 4."""

    @staticmethod
    def forward(ctx, W, u):
        m, d = W.shape
        b, _, l = u.shape
        out = torch.empty(b, m, l, device=u.device, dtype=torch.float32)
        # W: (rows m, K = d) K-major, shared; u[b]: (K = d, cols l) stored with l contiguous -> MN-major, batched
        _gemm(W, 0, 0, u, 1, 1, out, m, l, d, b, 0)
        ctx.save_for_backward(W, u)
        return out

    @staticmethod
    def backward(ctx, g):
        W, u = ctx.saved_tensors
        m, d = W.shape
        b, _, l = u.shape
        g = g.contiguous()
        dW = torch.empty_like(W)
        du = torch.empty_like(u)
        # dW (m, d) = sum_b g[b] (m, K = l) . u[b] (d, K = l)^T : both K-major, reduced over the batch
        _gemm(g, 0, 1, u, 0, 1, dW, m, d, l, b, 1)
        # du[b] (d, l) = W^T g[b]: W stored (K = m, rows d) -> MN-major shared; g[b] stored (K = m, cols l) -> MN-major
        _gemm(W, 1, 0, g, 1, 1, du, d, l, m, b, 0)
        return dW, du


def project(W: Tensor, u: Tensor) -> Tensor:
    """``einsum('mr,brt->bmt')`` in float32 accuracy on the tensor cores (pads r and t to multiples of 4)."""
    W = _f32c("W", W)
    u = _f32c("u", u)
    m, d = W.shape
    b, d2, l = u.shape
    if d2 != d:
        raise RuntimeError(f"projection: W is {tuple(W.shape)}, u is {tuple(u.shape)}")
    pd, pl = (-d) % 4, (-l) % 4
    if pd or pl:
        W = F.pad(W, (0, pd)).contiguous()
        u = F.pad(u, (0, pl, 0, pd)).contiguous()
    out = _Projection.apply(W, u)
    return out[..., :l].contiguous() if pl else out


class _ScanComplex(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rho, theta, u, dt, z, B_re, B_im, C_re, C_im, D):
        b, d, l = u.shape
        n = B_re.shape[1]
        lib = _lib.load()
        y = torch.empty_like(u)
        ckpt = torch.empty(lib.aussm_b200_scan_complex_ckpt_floats(b, d, n, l), device=u.device, dtype=torch.float32)
        with torch.cuda.device(u.device):
            rc = lib.aussm_b200_scan_complex_fwd(_ptr(rho), _ptr(theta), _ptr(u), _ptr(dt), _ptr(z), _ptr(B_re),
                                                 _ptr(B_im), _ptr(C_re), _ptr(C_im), _ptr(D), _ptr(y), _ptr(ckpt), b, d,
                                                 n, l, _stream(u))
        _lib.check(rc, "scan_complex forward")
        ctx.save_for_backward(rho, theta, u, dt, z, B_re, B_im, C_re, C_im, D, ckpt)
        ctx.mark_non_differentiable(ckpt)
        return y, ckpt

    @staticmethod
    def backward(ctx, gy, _gck):
        rho, theta, u, dt, z, B_re, B_im, C_re, C_im, D, ckpt = ctx.saved_tensors
        b, d, l = u.shape
        n = B_re.shape[1]
        lib = _lib.load()
        gy = gy.contiguous()
        like = lambda t: None if t is None else torch.empty_like(t)
        drho, dtheta = like(rho), like(theta)
        du, ddt, dz = torch.empty_like(u), torch.empty_like(u), torch.empty_like(u)
        dBr, dBi, dCr, dCi = like(B_re), like(B_im), like(C_re), like(C_im)
        dD = torch.empty_like(D)
        with torch.cuda.device(u.device):
            ws = _workspace(lib.aussm_b200_scan_complex_bwd_workspace_bytes(b, d, n, l), u.device)
            rc = lib.aussm_b200_scan_complex_bwd(_ptr(gy), _ptr(rho), _ptr(theta), _ptr(u), _ptr(dt), _ptr(z),
                                                 _ptr(B_re), _ptr(B_im), _ptr(C_re), _ptr(C_im), _ptr(D), _ptr(ckpt),
                                                 _ptr(drho), _ptr(dtheta), _ptr(du), _ptr(ddt), _ptr(dz), _ptr(dBr),
                                                 _ptr(dBi), _ptr(dCr), _ptr(dCi), _ptr(dD), b, d, n, l, _ptr(ws),
                                                 ws.numel(), _stream(u))
        _lib.check(rc, "scan_complex backward")
        return drho, dtheta, du, ddt, dz, dBr, dBi, dCr, dCi, dD


def scan_complex(rho: Optional[Tensor], theta: Optional[Tensor], u: Tensor, dt: Tensor, z: Tensor, B_re: Tensor,
                 B_im: Optional[Tensor], C_re: Tensor, C_im: Optional[Tensor], D: Tensor, return_states: bool = False):
    """Scan core on a given eigenvalue ``exp(rho + i theta)``; ``rho, theta``: (b, d, n, l) or None (= 0),
    ``B_*, C_*``: (b, n, l) (imaginary parts may be None).  Returns ``y`` (b, d, l) [and the tile-start states]."""
    b, d, l = u.shape
    n = B_re.shape[1]
    pad = (-l) % 4

    def prep(name, t, shape):
        if t is None:
            return None
        t = _f32c(name, t, shape)
        return F.pad(t, (0, pad)).contiguous() if pad else t

    args = [prep("rho", rho, (b, d, n, l)), prep("theta", theta, (b, d, n, l)), prep("u", u, (b, d, l)),
            prep("dt", dt, (b, d, l)), prep("z", z, (b, d, l)), prep("B_re", B_re, (b, n, l)),
            prep("B_im", B_im, (b, n, l)), prep("C_re", C_re, (b, n, l)), prep("C_im", C_im, (b, n, l))]
    y, ckpt = _ScanComplex.apply(*args, _f32c("D", D, (d,)))
    y = y[..., :l] if pad else y
    if return_states:
        ntiles = (l + pad + 31) // 32
        return y, ckpt.view(b, d, n, ntiles, 2)
    return y


def ssm_adaptive_complex(u: Tensor, dt: Tensor, x: Tensor, B: Tensor, C: Tensor, D: Tensor, z: Tensor,
                         return_states: bool = False):
    """General complex eigenvalue: ``lambda = exp(x[0].u) * exp(i x[1].u)`` (ops.py:233-297)."""
    two, d, n, d2 = x.shape
    assert two == 2 and d2 == d
    b, _, l = u.shape
    A = project(x.reshape(2 * d * n, d), u).view(b, 2, d, n, l)
    B, C = B.contiguous(), C.contiguous()
    return scan_complex(A[:, 0].contiguous(), A[:, 1].contiguous(), u, dt, z, B.real.contiguous(),
                        B.imag.contiguous(), C.real.contiguous(), C.imag.contiguous(), D, return_states)


def ssm_adaptive_preal(u: Tensor, dt: Tensor, x: Tensor, B: Tensor, C: Tensor, D: Tensor, z: Tensor,
                       return_states: bool = False):
    """Positive real eigenvalue: ``lambda = exp(x.u)``, real ``B, C`` (ops.py:300-357)."""
    d, n, d2 = x.shape
    b, _, l = u.shape
    rho = project(x.reshape(d * n, d), u).view(b, d, n, l)
    return scan_complex(rho, None, u, dt, z, B, None, C, None, D, return_states)


# Operator names the reference's kernels were meant to be registered under (they are `m.impl`-ed for names that
# are never defined there: ssm_adaptive_complex.cu:749-752, ssm_adaptive_real.cu:565-568), with the argument lists
# of their host functions (complex.cu:296-306, real.cu:211-218).
_library.define("ssm_adaptive_complex(Tensor u, Tensor dt, Tensor x_rho, Tensor x_theta, Tensor B_r, Tensor B_theta, "
                "Tensor C_r, Tensor C_theta, Tensor D, Tensor z) -> (Tensor, Tensor)")
_library.define("ssm_adaptive_preal(Tensor u, Tensor dt, Tensor x_rho, Tensor B_r, Tensor C_r, Tensor D, Tensor z) "
                "-> (Tensor, Tensor)")


def _op_complex(u, dt, x_rho, x_theta, B_r, B_theta, C_r, C_theta, D, z):
    B = torch.polar(B_r, B_theta)
    C = torch.polar(C_r, C_theta)
    return ssm_adaptive_complex(u, dt, torch.stack([x_rho, x_theta]), B, C, D, z, return_states=True)


def _op_preal(u, dt, x_rho, B_r, C_r, D, z):
    return ssm_adaptive_preal(u, dt, x_rho, B_r, C_r, D, z, return_states=True)


_library.impl("ssm_adaptive_complex", _op_complex, "CompositeImplicitAutograd")
_library.impl("ssm_adaptive_preal", _op_preal, "CompositeImplicitAutograd")
