"""Shared helpers of the test-suite: golden loading, seeded inputs, error reports."""
from __future__ import annotations

import math
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAMES = ["u", "dt", "x", "x_bias", "B", "C", "D", "z"]


def load_golden(name):
    blob = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: torch.from_numpy(blob[k]) for k in blob.files}


def model_like_inputs(seed, b, d, n, l, device="cpu", dtype=torch.float32):
    """Benchmark-configuration distributions (same recipe as tests/golden/make_golden.py)."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    u, z = r(b, d, l), r(b, d, l)
    dt = torch.nn.functional.softplus(r(b, d, l))
    x = r(d, n, d) / math.sqrt(d)
    x_bias = (torch.rand(d, n, generator=g) * 2 - 1) * math.pi
    sc = 1.0 / math.sqrt(n)
    B = torch.complex(r(n) * sc, r(n) * sc)
    C = torch.complex(r(n) * sc, r(n) * sc)
    D = r(d)
    gy = r(b, d, l)
    out = dict(u=u, dt=dt, x=x, x_bias=x_bias, B=B, C=C, D=D, z=z, gy=gy)
    for k, v in out.items():
        if v.is_complex():
            v = v.to(torch.complex64 if dtype == torch.float32 else torch.complex128)
        else:
            v = v.to(dtype)
        out[k] = v.to(device)
    return out


def scan_core_inputs(seed, b, d, n, l, device="cpu", dtype=torch.float32, with_state=True):
    """Inputs of the scan core: phase theta ~ U(-pi, pi) given directly."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    out = dict(
        theta=(torch.rand(b, d, n, l, generator=g) * 2 - 1) * math.pi,
        u=r(b, d, l), dt=torch.nn.functional.softplus(r(b, d, l)), z=r(b, d, l),
        B_r=torch.nn.functional.softplus(r(n) / math.sqrt(n)), B_theta=r(n) / math.sqrt(n),
        C_r=torch.nn.functional.softplus(r(n) / math.sqrt(n)), C_theta=r(n) / math.sqrt(n),
        D=r(d), gy=r(b, d, l),
        h0_re=r(b, d, n) if with_state else torch.zeros(b, d, n),
        h0_im=r(b, d, n) if with_state else torch.zeros(b, d, n),
        gh_re=r(b, d, n) if with_state else torch.zeros(b, d, n),
        gh_im=r(b, d, n) if with_state else torch.zeros(b, d, n),
    )
    return {k: v.to(dtype).to(device) for k, v in out.items()}


def outside_fraction(got, truth, atol, rtol):
    got = got.detach().double().cpu()
    truth = truth.detach().double().cpu()
    err = (got - truth).abs()
    return float((err > atol + rtol * truth.abs()).double().mean()), float(err.max())


def scaled_error(got, truth):
    """max |got - truth| / max |truth| : an error measure that does not blow up
    on the elements of a sum that happen to cancel."""
    got = got.detach().double().cpu()
    truth = truth.detach().double().cpu()
    return float((got - truth).abs().max() / truth.abs().max().clamp_min(1e-300))
