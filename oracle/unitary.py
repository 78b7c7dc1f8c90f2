"""CPU restatement of the adaptive *unitary* selective scan (test oracle).

TEST INFRASTRUCTURE ONLY - the shipped package never imports this module.

Shapes (reference convention): ``u, dt, z, y`` are ``(b, d, l)``; ``x`` is
``(d, n, d)`` indexed ``[i][j][r]``; ``x_bias`` is ``(d, n)``; ``D`` is
``(d,)``; the hidden state is ``(b, d, n)`` complex, passed as two real
tensors.  Every function works in whatever floating dtype it is given
(float32 for the timed CPU baseline, float64 for parity "truth") and is
differentiable through autograd, which is how gradient parity is checked.

Math of one operator call, for every ``(b, i, j)`` and ``t = 0 .. l-1``::

    theta_t = sum_r x[i,j,r] * u[b,r,t] + x_bias[i,j]
    h_t     = exp(1j*theta_t) * h_{t-1} + Bc_j * dt[b,i,t] * silu(u[b,i,t])
    y[b,i,t] = silu(z[b,i,t]) * (D[i]*silu(u[b,i,t]) + sum_j Re(Cc_j * h_t))

with ``Bc_j = B_r[j]*exp(1j*B_theta[j])`` and likewise ``Cc_j``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

TWO_PI = 2.0 * math.pi


def phase_projection(u: torch.Tensor, x: torch.Tensor, x_bias: torch.Tensor) -> torch.Tensor:
    """theta[b,i,j,t] = sum_r x[i,j,r] u[b,r,t] + x_bias[i,j]   -> (b, d, n, l).

    Follows extension-cpp/extension_cpp/ops.py:672 (einsum) and :680 (bias);
    the CUDA reference builds the same sum row by row in
    csrc/cuda/ssm_adaptive_unitary_forward.cu:83-110.
    """
    return torch.einsum("ijr,brt->bijt", x, u) + x_bias[None, :, :, None]


def scan_unitary_cumsum(theta, u, dt, z, B_r, B_theta, C_r, C_theta, D, h0_re=None, h0_im=None):
    """Scan core on a given phase tensor, in the reference's cumulative-sum form.

    ``theta`` is ``(b, d, n, l)``.  Returns ``(y, h_re, h_im)`` with the state
    after the last step.  Steps follow extension-cpp/extension_cpp/ops.py:
    :690 running phase, :696 reduction mod 2*pi, :719-720 rotated drive,
    :729-730 its running sum, :744 projection on C, :756 skip term, :760 gate;
    the previous hidden state enters as in
    csrc/cuda/ssm_adaptive_unitary_forward.cu:161-162 and the next one leaves
    as in :173-181.
    """
    b, d, n, l = theta.shape
    if h0_re is None:
        h0_re = theta.new_zeros(b, d, n)
    if h0_im is None:
        h0_im = theta.new_zeros(b, d, n)
    G = torch.remainder(torch.cumsum(theta, dim=-1), TWO_PI)            # (b,d,n,l)
    v = F.silu(u)                                                        # (b,d,l)
    drive = (dt * v)[:, :, None, :]                                      # (b,d,1,l)
    Br = B_r.reshape(1, 1, n, 1)
    Bt = B_theta.reshape(1, 1, n, 1)
    Cr = C_r.reshape(1, 1, n, 1)
    Ct = C_theta.reshape(1, 1, n, 1)
    re = torch.cumsum(Br * torch.cos(Bt - G) * drive, dim=-1) + h0_re[..., None]
    im = torch.cumsum(Br * torch.sin(Bt - G) * drive, dim=-1) + h0_im[..., None]
    proj = (Cr * (torch.cos(Ct + G) * re - torch.sin(Ct + G) * im)).sum(dim=2)   # (b,d,l)
    y = (proj + v * D.reshape(1, d, 1)) * F.silu(z)
    Gl, rel, iml = G[..., -1], re[..., -1], im[..., -1]
    h_re = torch.cos(Gl) * rel - torch.sin(Gl) * iml
    h_im = torch.sin(Gl) * rel + torch.cos(Gl) * iml
    return y, h_re, h_im


def scan_unitary_recurrence(theta, u, dt, z, B_r, B_theta, C_r, C_theta, D, h0_re=None, h0_im=None):
    """The same operator as a plain time loop (independent cross-check).

    This is the sequential recurrence that the cumulative-sum form above is
    algebraically equal to; it never forms an unbounded running phase, so in
    float64 it is the reference "truth" for long sequences.
    """
    b, d, n, l = theta.shape
    hr = theta.new_zeros(b, d, n) if h0_re is None else h0_re
    hi = theta.new_zeros(b, d, n) if h0_im is None else h0_im
    v = F.silu(u)
    drive = dt * v
    bre = (B_r * torch.cos(B_theta)).reshape(1, 1, n)
    bim = (B_r * torch.sin(B_theta)).reshape(1, 1, n)
    cre = (C_r * torch.cos(C_theta)).reshape(1, 1, n)
    cim = (C_r * torch.sin(C_theta)).reshape(1, 1, n)
    # per-step views through unbind: one autograd node per tensor instead of one full-size gradient per step
    cs, sn = torch.cos(theta).unbind(-1), torch.sin(theta).unbind(-1)
    drv = drive.unsqueeze(-1).unbind(2)
    out = []
    for t in range(l):
        c, s, s_t = cs[t], sn[t], drv[t]
        hr, hi = c * hr - s * hi + bre * s_t, s * hr + c * hi + bim * s_t
        out.append((cre * hr - cim * hi).sum(-1))
    proj = torch.stack(out, dim=-1)
    y = (proj + v * D.reshape(1, d, 1)) * F.silu(z)
    return y, hr, hi


def op_unitary(u, dt, x, x_bias, B_r, B_theta, C_r, C_theta, D, z, h0_re, h0_im, recurrence=False):
    """The registered operator ``extension_cpp::ssm_adaptive_unitary``.

    Argument order and meaning are those of the schema in
    csrc/cuda/ssm_adaptive_unitary_forward.cu:284; returns ``(y, h_re, h_im)``.
    """
    theta = phase_projection(u, x, x_bias)
    fn = scan_unitary_recurrence if recurrence else scan_unitary_cumsum
    return fn(theta, u, dt, z, B_r, B_theta, C_r, C_theta, D, h0_re, h0_im)


def polar_cumsum_unitary(u, dt, x, x_bias, B, C, D, z):
    """Restatement of ``reference_ssm_adaptive_unitary_optimized_polar`` for
    constant complex ``B, C`` of shape ``(n,)``
    (extension-cpp/extension_cpp/ops.py:614-769; the radius goes through a
    softplus at :706 and :738, the angle is the imaginary part, :705 / :737).
    This is the function the reference's tests compare the CUDA kernels with
    (extension-cpp/test/test_extension.py:87, :122).
    """
    y, _, _ = op_unitary(u, dt, x, x_bias, F.softplus(B.real), B.imag, F.softplus(C.real), C.imag, D, z,
                         None, None)
    return y


def interface_unitary(u, dt, x, x_bias, B, C, D, z, max_parallel_length=2048, recurrence=False):
    """Restatement of the front end ``ssm_adaptive_interface(..., unitary=True)``
    (extension-cpp/extension_cpp/ops.py:28-93): zero-pad the time axis to a
    multiple of 16 (:36-41), split B and C into softplus radius and angle
    (:55-58), run the operator over chunks of ``max_parallel_length`` steps
    carrying the complex hidden state (:72-85), cut the padding off (:91).
    """
    l0 = u.shape[-1]
    pad = (-l0) % 16
    if pad:
        u, dt, z = (F.pad(t, (0, pad)) for t in (u, dt, z))
    b, d, l = u.shape
    n = x.shape[1]
    B_r, B_theta = F.softplus(B.real), B.imag
    C_r, C_theta = F.softplus(C.real), C.imag
    h_re = u.new_zeros(b, d, n)
    h_im = u.new_zeros(b, d, n)
    pieces = []
    for s in range(0, l, max_parallel_length):
        e = min(s + max_parallel_length, l)
        y_c, h_re, h_im = op_unitary(u[..., s:e], dt[..., s:e], x, x_bias, B_r, B_theta, C_r, C_theta, D,
                                     z[..., s:e], h_re, h_im, recurrence=recurrence)
        pieces.append(y_c)
    return torch.cat(pieces, dim=-1)[..., :l0]
