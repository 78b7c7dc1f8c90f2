"""CPU restatements of the reference's loop references for the complex and
positive-real recurrences.  TEST INFRASTRUCTURE ONLY.

Pinned against outputs of the reference's own functions stored in
tests/golden/loop_variants.npz (made by tests/golden/make_golden.py).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def scan_complex_ref(rho, theta, u, dt, z, B, C, D):
    """h_t = exp(rho_t + i theta_t) h_{t-1} + B[b,j,t] dt_t silu(u_t);  y = silu(z)(Re sum_j C h + D silu(u)).
    rho, theta: (b, d, n, l) or None; B, C: (b, n, l) real or complex."""
    b, d, l = u.shape
    n = B.shape[1]
    cdt = torch.complex128 if u.dtype == torch.float64 else torch.complex64
    zero = u.new_zeros(b, d, n, l)
    lam = torch.polar(torch.exp(zero if rho is None else rho), zero if theta is None else theta)
    v = F.silu(u)
    drive = dt * v
    h = torch.zeros(b, d, n, dtype=cdt)
    # per-step views through unbind: one autograd node per tensor instead of one full-size gradient per step
    lam_t = lam.unbind(-1)
    drv_t = drive.unsqueeze(-1).unbind(2)                     # (b, d, 1) each
    B_t, C_t = B.to(cdt).unsqueeze(1).unbind(-1), C.to(cdt).unsqueeze(1).unbind(-1)   # (b, 1, n) each
    ys = []
    for t in range(l):
        h = lam_t[t] * h + drv_t[t] * B_t[t]
        ys.append((h * C_t[t]).sum(-1).real)
    y = torch.stack(ys, dim=-1)
    return (y + v * D[None, :, None]) * F.silu(z)


def complex_ref(u, dt, x, B, C, D, z):
    """extension-cpp/extension_cpp/ops.py:233-297: x is (2, d, n, d); eigenvalue exp(x[0].u) * exp(i x[1].u)."""
    A = torch.einsum("pijr,brt->pbijt", x, u)
    return scan_complex_ref(A[0], A[1], u, dt, z, B, C, D)


def preal_ref(u, dt, x, B, C, D, z):
    """extension-cpp/extension_cpp/ops.py:300-357: x is (d, n, d); eigenvalue exp(x.u); real B, C."""
    return scan_complex_ref(torch.einsum("ijr,brt->bijt", x, u), None, u, dt, z, B, C, D)
