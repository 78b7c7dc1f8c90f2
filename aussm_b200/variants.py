"""Complex and positive-real variants of the adaptive selective scan on B200.

The reference compiles kernels for these (csrc/cuda/ssm_adaptive_complex.cu,
ssm_adaptive_real.cu) but never registers or wraps them; what it does define is
their PyTorch loop references, whose signatures these functions take:

    ssm_adaptive_complex(u, dt, x, B, C, D, z)   x: (2, d, n, d) [rho, theta rows];  B, C complex (b, n, l)
    ssm_adaptive_preal(u, dt, x, B, C, D, z)     x: (d, n, d);                       B, C real (b, n, l)
    (extension-cpp/extension_cpp/ops.py:233-297 and :300-357)

Both are a projection (eigenvalue exponent = x . u, a dense contraction that
runs on the tcgen05 GEMM of the library) followed by the scan; the library's
operators ``aussm_b200_complex_fwd / _bwd`` do both one time window at a time
(the reference's kernels loop chunks in-kernel, ssm_adaptive_complex.cu:228,
ssm_adaptive_real.cu:154), so the (b, d, n, l) exponent tensors are never
materialised.  ``scan_complex`` is the scan core on given exponents.
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
    """A[b] = W @ u[b]  with W (m, d), u (b, d, l) -> (b, m, l)."""

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
        du = torch.empty_like(u)
        # dW (m, d) = sum_b g[b] (m, K = l) . u[b] (d, K = l)^T : both K-major, reduced over the batch
        from .stages import _weight_grad
        dW = _weight_grad(g, 0, u, 0, m, d, l, b)
        # du[b] (d, l) = W^T g[b]: W stored (K = m, rows d) -> MN-major shared; g[b] stored (K = m, cols l) -> MN-major
        _gemm(W, 1, 0, g, 1, 1, du, d, l, m, b, 0)
        return dW, du


def project(W: Tensor, u: Tensor) -> Tensor:
    """``einsum('mr,brt->bmt')`` in float32 accuracy on the tensor cores."""
    W = _f32c("W", W)
    u = _f32c("u", u)
    if u.shape[1] != W.shape[1]:
        raise RuntimeError(f"projection: W is {tuple(W.shape)}, u is {tuple(u.shape)}")
    return _Projection.apply(W, u)


class _ScanComplex(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rho, theta, u, dt, z, B_re, B_im, C_re, C_im, D):
        b, d, l = u.shape
        n = B_re.shape[1]
        lib = _lib.load()
        y = torch.empty_like(u)
        states = torch.empty(lib.aussm_b200_scan_complex_states_floats(b, d, n, l), device=u.device,
                             dtype=torch.float32)
        with torch.cuda.device(u.device):
            rc = lib.aussm_b200_scan_complex_fwd(_ptr(rho), _ptr(theta), _ptr(u), _ptr(dt), _ptr(z), _ptr(B_re),
                                                 _ptr(B_im), _ptr(C_re), _ptr(C_im), _ptr(D), _ptr(y), _ptr(states), b,
                                                 d, n, l, _stream(u))
        _lib.check(rc, "scan_complex forward")
        ctx.save_for_backward(rho, theta, u, dt, z, B_re, B_im, C_re, C_im, D, states)
        return y, states

    @staticmethod
    def backward(ctx, gy, gstates):
        rho, theta, u, dt, z, B_re, B_im, C_re, C_im, D, states = ctx.saved_tensors
        b, d, l = u.shape
        n = B_re.shape[1]
        lib = _lib.load()
        gy = torch.zeros_like(u) if gy is None else gy.contiguous()
        gstates = None if gstates is None else gstates.contiguous()
        like = lambda t: None if t is None else torch.empty_like(t)
        drho, dtheta = like(rho), like(theta)
        du, ddt, dz = torch.empty_like(u), torch.empty_like(u), torch.empty_like(u)
        dBr, dBi, dCr, dCi = like(B_re), like(B_im), like(C_re), like(C_im)
        dD = torch.empty_like(D)
        with torch.cuda.device(u.device):
            ws = _workspace(lib.aussm_b200_scan_complex_bwd_workspace_bytes(b, d, n, l), u.device)
            rc = lib.aussm_b200_scan_complex_bwd(_ptr(gy), _ptr(gstates), _ptr(rho), _ptr(theta), _ptr(u), _ptr(dt),
                                                 _ptr(z), _ptr(B_re), _ptr(B_im), _ptr(C_re), _ptr(C_im), _ptr(D),
                                                 _ptr(states), _ptr(drho), _ptr(dtheta), _ptr(du), _ptr(ddt), _ptr(dz),
                                                 _ptr(dBr), _ptr(dBi), _ptr(dCr), _ptr(dCi), _ptr(dD), b, d, n, l,
                                                 _ptr(ws), ws.numel(), _stream(u))
        _lib.check(rc, "scan_complex backward")
        return drho, dtheta, du, ddt, dz, dBr, dBi, dCr, dCi, dD


def _pad4(name, t, shape, pad):
    if t is None:
        return None
    t = _f32c(name, t, shape)
    return F.pad(t, (0, pad)).contiguous() if pad else t


def _states_view(states: Tensor, b, d, n, lp):
    """(b, d, n, lp/16 + 1, 2): the state before every 16th step and after the last one (real, imaginary)."""
    return states.view(b, d, n, (lp + 15) // 16 + 1, 2)


def scan_complex(rho: Optional[Tensor], theta: Optional[Tensor], u: Tensor, dt: Tensor, z: Tensor, B_re: Tensor,
                 B_im: Optional[Tensor], C_re: Tensor, C_im: Optional[Tensor], D: Tensor, return_states: bool = False):
    """Scan core on a given eigenvalue ``exp(rho + i theta)``; ``rho, theta``: (b, d, n, l) or None (= 0),
    ``B_*, C_*``: (b, n, l) (imaginary parts may be None).  Returns ``y`` (b, d, l) [and the state record]."""
    b, d, l = u.shape
    n = B_re.shape[1]
    pad = (-l) % 4
    args = [_pad4("rho", rho, (b, d, n, l), pad), _pad4("theta", theta, (b, d, n, l), pad),
            _pad4("u", u, (b, d, l), pad), _pad4("dt", dt, (b, d, l), pad), _pad4("z", z, (b, d, l), pad),
            _pad4("B_re", B_re, (b, n, l), pad), _pad4("B_im", B_im, (b, n, l), pad),
            _pad4("C_re", C_re, (b, n, l), pad), _pad4("C_im", C_im, (b, n, l), pad)]
    y, states = _ScanComplex.apply(*args, _f32c("D", D, (d,)))
    y = y[..., :l] if pad else y
    if return_states:
        return y, _states_view(states, b, d, n, l + pad)
    return y


class _ComplexOp(torch.autograd.Function):
    """Projection + scan through the windowed C-ABI operators (aussm_b200_complex_fwd / _bwd): the eigenvalue
    exponents x . u exist one time window at a time only."""

    @staticmethod
    def forward(ctx, u, dt, x, B_re, B_im, C_re, C_im, D, z):
        b, d, l = u.shape
        n = B_re.shape[1]
        has_theta = 1 if x.dim() == 4 else 0
        lib = _lib.load()
        y = torch.empty_like(u)
        states = torch.empty(lib.aussm_b200_scan_complex_states_floats(b, d, n, l), device=u.device,
                             dtype=torch.float32)
        with torch.cuda.device(u.device):
            ws = _workspace(lib.aussm_b200_complex_workspace_bytes(b, d, n, l, has_theta), u.device)
            rc = lib.aussm_b200_complex_fwd(_ptr(u), _ptr(dt), _ptr(x), has_theta, _ptr(B_re), _ptr(B_im), _ptr(C_re),
                                            _ptr(C_im), _ptr(D), _ptr(z), _ptr(y), _ptr(states), b, d, n, l, _ptr(ws),
                                            ws.numel(), _stream(u))
        _lib.check(rc, "ssm_adaptive_complex" if has_theta else "ssm_adaptive_preal")
        ctx.save_for_backward(u, dt, x, B_re, B_im, C_re, C_im, D, z, states)
        return y, states

    @staticmethod
    def backward(ctx, gy, gstates):
        u, dt, x, B_re, B_im, C_re, C_im, D, z, states = ctx.saved_tensors
        gy = torch.zeros_like(u) if gy is None else gy
        return _complex_backward(gy, gstates, u, dt, x, B_re, B_im, C_re, C_im, D, z, states)


def _complex_backward(gy, gstates, u, dt, x, B_re, B_im, C_re, C_im, D, z, states):
    """(du, ddt, dx, dB_re, dB_im, dC_re, dC_im, dD, dz) through aussm_b200_complex_bwd."""
    b, d, l = u.shape
    n = B_re.shape[1]
    has_theta = 1 if x.dim() == 4 else 0
    lib = _lib.load()
    gy = _f32c("grad_y", gy, (b, d, l))
    gstates = None if gstates is None else _f32c("grad_h", gstates.reshape(-1), (states.numel(),))
    like = lambda t: None if t is None else torch.empty_like(t)
    du, ddt, dz = torch.empty_like(u), torch.empty_like(u), torch.empty_like(u)
    dx = torch.empty_like(x)
    dBr, dBi, dCr, dCi = like(B_re), like(B_im), like(C_re), like(C_im)
    dD = torch.empty_like(D)
    with torch.cuda.device(u.device):
        ws = _workspace(lib.aussm_b200_complex_workspace_bytes(b, d, n, l, has_theta), u.device)
        rc = lib.aussm_b200_complex_bwd(_ptr(gy), _ptr(gstates), _ptr(u), _ptr(dt), _ptr(x), has_theta, _ptr(B_re),
                                        _ptr(B_im), _ptr(C_re), _ptr(C_im), _ptr(D), _ptr(z), _ptr(states), _ptr(du),
                                        _ptr(ddt), _ptr(dx), _ptr(dBr), _ptr(dBi), _ptr(dCr), _ptr(dCi), _ptr(dD),
                                        _ptr(dz), b, d, n, l, _ptr(ws), ws.numel(), _stream(u))
    _lib.check(rc, "ssm_adaptive_backward_complex" if has_theta else "ssm_adaptive_backward_preal")
    return du, ddt, dx, dBr, dBi, dCr, dCi, dD, dz


def _complex_call(u, dt, x, B_re, B_im, C_re, C_im, D, z, return_states):
    b, d, l = u.shape
    n = B_re.shape[1]
    pad = (-l) % 4
    y, states = _ComplexOp.apply(_pad4("u", u, (b, d, l), pad), _pad4("dt", dt, (b, d, l), pad), _f32c("x", x),
                                 _pad4("B_re", B_re, (b, n, l), pad), _pad4("B_im", B_im, (b, n, l), pad),
                                 _pad4("C_re", C_re, (b, n, l), pad), _pad4("C_im", C_im, (b, n, l), pad),
                                 _f32c("D", D, (d,)), _pad4("z", z, (b, d, l), pad))
    y = y[..., :l] if pad else y
    if return_states:
        return y, _states_view(states, b, d, n, l + pad)
    return y


def ssm_adaptive_complex(u: Tensor, dt: Tensor, x: Tensor, B: Tensor, C: Tensor, D: Tensor, z: Tensor,
                         return_states: bool = False):
    """General complex eigenvalue: ``lambda = exp(x[0].u) * exp(i x[1].u)`` (ops.py:233-297);
    ``x``: (2, d, n, d), ``B, C``: complex (b, n, l)."""
    two, d, n, d2 = x.shape
    assert two == 2 and d2 == d
    return _complex_call(u, dt, x, B.real, B.imag, C.real, C.imag, D, z, return_states)


def ssm_adaptive_preal(u: Tensor, dt: Tensor, x: Tensor, B: Tensor, C: Tensor, D: Tensor, z: Tensor,
                       return_states: bool = False):
    """Positive real eigenvalue: ``lambda = exp(x.u)``, real ``B, C`` (ops.py:300-357); ``x``: (d, n, d)."""
    d, n, d2 = x.shape
    assert d2 == d
    return _complex_call(u, dt, x, B, None, C, None, D, z, return_states)


# ---------------------------------------------------------------------------
# The four operator names the reference's kernels were meant to be registered under.  There they are
# `m.impl`-ed for names that are never defined (ssm_adaptive_complex.cu:749-752, ssm_adaptive_real.cu:565-568);
# here they exist, with the argument lists of the reference's host functions: forwards complex.cu:296-306 and
# real.cu:211-218, backwards complex.cu:662-676 and real.cu:490-501 (grad_y, grad_h, the forward's inputs,
# hidden_states -> one gradient per input).  B and C arrive as radius / angle pairs (b, n, l).
# `hidden_states` is this library's state record: (b, d, n, l/16 + 1, 2).
# ---------------------------------------------------------------------------
_library.define("ssm_adaptive_complex(Tensor u, Tensor dt, Tensor x_rho, Tensor x_theta, Tensor B_r, Tensor B_theta, "
                "Tensor C_r, Tensor C_theta, Tensor D, Tensor z) -> (Tensor, Tensor)")
_library.define("ssm_adaptive_backward_complex(Tensor grad_y, Tensor grad_h, Tensor u, Tensor dt, Tensor x_rho, "
                "Tensor x_theta, Tensor B_r, Tensor B_theta, Tensor C_r, Tensor C_theta, Tensor D, Tensor z, "
                "Tensor hidden_states) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, "
                "Tensor)")
_library.define("ssm_adaptive_preal(Tensor u, Tensor dt, Tensor x_rho, Tensor B_r, Tensor C_r, Tensor D, Tensor z) "
                "-> (Tensor, Tensor)")
_library.define("ssm_adaptive_backward_preal(Tensor grad_y, Tensor grad_h, Tensor u, Tensor dt, Tensor x_rho, "
                "Tensor B_r, Tensor C_r, Tensor D, Tensor z, Tensor hidden_states) -> (Tensor, Tensor, Tensor, "
                "Tensor, Tensor, Tensor, Tensor)")


def _need4(l):
    if l % 4:
        raise RuntimeError(f"the registered operators need a sequence length that is a multiple of 4, got {l} "
                           "(aussm_b200.ssm_adaptive_complex / ssm_adaptive_preal pad for you)")


def _op_complex(u, dt, x_rho, x_theta, B_r, B_theta, C_r, C_theta, D, z):
    b, d, l = u.shape
    n = B_r.shape[1]
    _need4(l)
    x = torch.stack([x_rho, x_theta]).contiguous()
    Bc, Cc = torch.polar(B_r, B_theta), torch.polar(C_r, C_theta)
    lib = _lib.load()
    y = torch.empty_like(u)
    states = torch.empty(lib.aussm_b200_scan_complex_states_floats(b, d, n, l), device=u.device, dtype=torch.float32)
    args = [_f32c("u", u, (b, d, l)), _f32c("dt", dt, (b, d, l)), _f32c("x", x, (2, d, n, d)),
            _f32c("B_re", Bc.real, (b, n, l)), _f32c("B_im", Bc.imag, (b, n, l)), _f32c("C_re", Cc.real, (b, n, l)),
            _f32c("C_im", Cc.imag, (b, n, l)), _f32c("D", D, (d,)), _f32c("z", z, (b, d, l))]
    with torch.cuda.device(u.device):
        ws = _workspace(lib.aussm_b200_complex_workspace_bytes(b, d, n, l, 1), u.device)
        rc = lib.aussm_b200_complex_fwd(_ptr(args[0]), _ptr(args[1]), _ptr(args[2]), 1, _ptr(args[3]), _ptr(args[4]),
                                        _ptr(args[5]), _ptr(args[6]), _ptr(args[7]), _ptr(args[8]), _ptr(y),
                                        _ptr(states), b, d, n, l, _ptr(ws), ws.numel(), _stream(u))
    _lib.check(rc, "ssm_adaptive_complex")
    return y, _states_view(states, b, d, n, l)


def _polar_grads(r, th, g_re, g_im):
    """Gradients of (radius, angle) from the gradients of the real and imaginary parts of r exp(i th)."""
    c, s = torch.cos(th), torch.sin(th)
    return g_re * c + g_im * s, r * (g_im * c - g_re * s)


def _op_backward_complex(grad_y, grad_h, u, dt, x_rho, x_theta, B_r, B_theta, C_r, C_theta, D, z, hidden_states):
    _need4(u.shape[-1])
    x = torch.stack([x_rho, x_theta]).contiguous()
    Bc, Cc = torch.polar(B_r, B_theta), torch.polar(C_r, C_theta)
    du, ddt, dx, dBr, dBi, dCr, dCi, dD, dz = _complex_backward(
        grad_y, grad_h, u.contiguous(), dt.contiguous(), x, Bc.real.contiguous(), Bc.imag.contiguous(),
        Cc.real.contiguous(), Cc.imag.contiguous(), D.contiguous(), z.contiguous(), hidden_states.contiguous().view(-1))
    gBr, gBt = _polar_grads(B_r, B_theta, dBr, dBi)
    gCr, gCt = _polar_grads(C_r, C_theta, dCr, dCi)
    return du, ddt, dx[0], dx[1], gBr, gBt, gCr, gCt, dD, dz


def _op_preal(u, dt, x_rho, B_r, C_r, D, z):
    b, d, l = u.shape
    n = B_r.shape[1]
    _need4(l)
    lib = _lib.load()
    y = torch.empty_like(u)
    states = torch.empty(lib.aussm_b200_scan_complex_states_floats(b, d, n, l), device=u.device, dtype=torch.float32)
    args = [_f32c("u", u, (b, d, l)), _f32c("dt", dt, (b, d, l)), _f32c("x_rho", x_rho, (d, n, d)),
            _f32c("B_r", B_r, (b, n, l)), _f32c("C_r", C_r, (b, n, l)), _f32c("D", D, (d,)), _f32c("z", z, (b, d, l))]
    with torch.cuda.device(u.device):
        ws = _workspace(lib.aussm_b200_complex_workspace_bytes(b, d, n, l, 0), u.device)
        rc = lib.aussm_b200_complex_fwd(_ptr(args[0]), _ptr(args[1]), _ptr(args[2]), 0, _ptr(args[3]), None,
                                        _ptr(args[4]), None, _ptr(args[5]), _ptr(args[6]), _ptr(y), _ptr(states), b, d,
                                        n, l, _ptr(ws), ws.numel(), _stream(u))
    _lib.check(rc, "ssm_adaptive_preal")
    return y, _states_view(states, b, d, n, l)


def _op_backward_preal(grad_y, grad_h, u, dt, x_rho, B_r, C_r, D, z, hidden_states):
    _need4(u.shape[-1])
    du, ddt, dx, dBr, _, dCr, _, dD, dz = _complex_backward(
        grad_y, grad_h, u.contiguous(), dt.contiguous(), x_rho.contiguous(), B_r.contiguous(), None, C_r.contiguous(),
        None, D.contiguous(), z.contiguous(), hidden_states.contiguous().view(-1))
    return du, ddt, dx, dBr, dCr, dD, dz


_library.impl("ssm_adaptive_complex", _op_complex, "CUDA")
_library.impl("ssm_adaptive_backward_complex", _op_backward_complex, "CUDA")
_library.impl("ssm_adaptive_preal", _op_preal, "CUDA")
_library.impl("ssm_adaptive_backward_preal", _op_backward_preal, "CUDA")


def _fake_fwd_states(u, B_r):
    b, d, l = u.shape
    return torch.empty_like(u), u.new_empty(b, d, B_r.shape[1], (l + 15) // 16 + 1, 2)


@torch.library.register_fake("extension_cpp::ssm_adaptive_complex")
def _fake_complex(u, dt, x_rho, x_theta, B_r, B_theta, C_r, C_theta, D, z):
    return _fake_fwd_states(u, B_r)


@torch.library.register_fake("extension_cpp::ssm_adaptive_preal")
def _fake_preal(u, dt, x_rho, B_r, C_r, D, z):
    return _fake_fwd_states(u, B_r)


@torch.library.register_fake("extension_cpp::ssm_adaptive_backward_complex")
def _fake_backward_complex(grad_y, grad_h, u, dt, x_rho, x_theta, B_r, B_theta, C_r, C_theta, D, z, hidden_states):
    return tuple(torch.empty_like(t) for t in (u, dt, x_rho, x_theta, B_r, B_theta, C_r, C_theta, D, z))


@torch.library.register_fake("extension_cpp::ssm_adaptive_backward_preal")
def _fake_backward_preal(grad_y, grad_h, u, dt, x_rho, B_r, C_r, D, z, hidden_states):
    return tuple(torch.empty_like(t) for t in (u, dt, x_rho, B_r, C_r, D, z))


# autograd: the forwards save their inputs and the state record, the backward is the second operator of each
# pair, as for the unitary pair (extension_cpp/ops.py:109-154)
def _setup_ctx(ctx, inputs, output):
    ctx.save_for_backward(*inputs, output[1])


def _zeros_if_none(g, like):
    return torch.zeros_like(like) if g is None else g


def _autograd_complex(ctx, grad_y, grad_h):
    *inputs, states = ctx.saved_tensors
    grad_h = _zeros_if_none(grad_h, states)
    return torch.ops.extension_cpp.ssm_adaptive_backward_complex.default(_zeros_if_none(grad_y, inputs[0]), grad_h,
                                                                         *inputs, states)


def _autograd_preal(ctx, grad_y, grad_h):
    *inputs, states = ctx.saved_tensors
    grad_h = _zeros_if_none(grad_h, states)
    return torch.ops.extension_cpp.ssm_adaptive_backward_preal.default(_zeros_if_none(grad_y, inputs[0]), grad_h,
                                                                       *inputs, states)


torch.library.register_autograd("extension_cpp::ssm_adaptive_complex", _autograd_complex, setup_context=_setup_ctx)
torch.library.register_autograd("extension_cpp::ssm_adaptive_preal", _autograd_preal, setup_context=_setup_ctx)
