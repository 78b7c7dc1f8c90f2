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


def parity_report(name, got, truth, ref32=None, atol=1e-5, rtol=1e-4):
    """Error of `got` against the float64 truth, next to the float32 oracle's own error."""
    fo, mx = outside_fraction(got, truth, atol, rtol)
    line = f"{name}: max|err|={mx:.3e} scaled={scaled_error(got, truth):.3e} outside(atol={atol},rtol={rtol})={fo:.4%}"
    if ref32 is not None:
        fo32, mx32 = outside_fraction(ref32, truth, atol, rtol)
        line += f" | fp32 oracle: max|err|={mx32:.3e} outside={fo32:.4%}"
    print(line)
    return fo, mx


# every assert_parity call of the session: (test id, tensor, branch, fraction outside, max error, note);
# tests/conftest.py prints a summary of it at the end of the run
PARITY_LOG = []


def _record(name, branch, fo, mx, note=""):
    test = os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]
    PARITY_LOG.append((test, name, branch, fo, mx, note))
    print(f"    parity[{name}]: {branch} {note}")
    return branch


def assert_parity(name, got, truth, ref32=None, atol=1e-5, rtol=1e-4, scaled_tol=None):
    """Parity rule of this suite.

    Pass if every element is within ``atol + rtol*|truth|`` of the float64
    truth ("strict").  Float32 arithmetic cannot guarantee that for long
    sequences (the reference's own float32 oracle does not meet it either), so
    otherwise the result must be at least as close to the truth as the float32
    oracle is: no larger a fraction of elements outside the tolerance, and a
    largest error of at most twice the oracle's ("no worse than the float32
    oracle"); or - when no float32 oracle result is at hand - within
    ``scaled_tol`` of the truth relative to the largest magnitude of the tensor
    ("scaled").  The branch that let the case pass is printed and returned, so
    that a test log shows it per tensor.
    """
    fo, mx = parity_report(name, got, truth, ref32, atol, rtol)
    if fo == 0.0:
        return _record(name, "strict", fo, mx)
    if ref32 is not None:
        fo32, mx32 = outside_fraction(ref32, truth, atol, rtol)
        # a float32 oracle with nothing outside leaves no room: only the strict branch passes then
        bound = 0.0 if fo32 == 0.0 else max(fo32, 1e-3)
        assert fo <= bound, f"{name}: {fo:.4%} of elements outside tolerance, float32 oracle {fo32:.4%}"
        assert mx <= max(2.0 * mx32, atol), f"{name}: max error {mx:.3e} vs float32 oracle {mx32:.3e}"
        return _record(name, "float32-oracle", fo, mx, f"oracle32 outside {fo32:.4%} max|err| {mx32:.3e}")
    assert scaled_tol is not None, f"{name}: {fo:.4%} of elements outside atol={atol} rtol={rtol}"
    se = scaled_error(got, truth)
    assert se <= scaled_tol, f"{name}: scaled error {se:.3e} > {scaled_tol:.1e}"
    return _record(name, "scaled", fo, mx, f"scaled error {se:.3e} <= {scaled_tol:.1e}")
