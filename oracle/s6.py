"""CPU oracle of the real selective scan of the Mamba block.  TEST INFRASTRUCTURE ONLY.

Parity unpinned: the algorithm lives in the third-party package mamba-ssm
(version not pinned by the reference: requirements.txt does not list it, the
Makefile installs the latest, Makefile:9,14), which is absent from the reference
tree and from this machine, and the reference holds no test or golden vector at
this boundary.  This is the published S6 recurrence of the Mamba paper written
from the math, with the argument meaning of the reference's call site
(ai-modules/wavesAI/model/aussm.py:788-802: A = -exp(A_log), delta_bias,
delta_softplus=True, D skip, gate z through silu).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def selective_scan_ref(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False,
                       return_last_state=False):
    """u, delta, z: (b, d, l); A: (d, n); B, C: (b, n, l); D, delta_bias: (d,)."""
    b, d, l = u.shape
    n = A.shape[1]
    dlt = delta if delta_bias is None else delta + delta_bias[None, :, None]
    if delta_softplus:
        dlt = F.softplus(dlt)
    h = u.new_zeros(b, d, n)
    # per-step views through unbind: one autograd node per tensor instead of one full-size gradient per step
    dl_t = dlt.unsqueeze(-1).unbind(2)                        # (b, d, 1) each
    du_t = (dlt * u).unsqueeze(-1).unbind(2)
    B_t, C_t = B.unsqueeze(1).unbind(-1), C.unsqueeze(1).unbind(-1)      # (b, 1, n) each
    ys = []
    for t in range(l):
        a = torch.exp(dl_t[t] * A[None])                                  # (b, d, n)
        h = a * h + du_t[t] * B_t[t]
        ys.append((h * C_t[t]).sum(-1))
    y = torch.stack(ys, dim=-1)
    if D is not None:
        y = y + u * D[None, :, None]
    if z is not None:
        y = y * F.silu(z)
    return (y, h) if return_last_state else y
