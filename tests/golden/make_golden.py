"""Generate the golden vectors in this directory from the REFERENCE's own
Python oracles.  Run it where a checkout of arjunkaruvally/AUSSM is available:

    python tests/golden/make_golden.py /path/to/AUSSM

It loads ``extension-cpp/extension_cpp/ops.py`` from that checkout by path.
That file registers autograd for ``extension_cpp::ssm_adaptive_unitary`` when
it is imported (ops.py:153-154), so the two operator schemas
(csrc/cuda/ssm_adaptive_unitary_forward.cu:284-285) are defined first, empty.
The outputs are ``*.npz`` files holding the seeded inputs and what the
reference functions returned for them; the tests never need the checkout.
"""
from __future__ import annotations

import contextlib
import importlib.util
import io
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

FWD_SCHEMA = ("ssm_adaptive_unitary(Tensor u,Tensor dt,Tensor x, Tensor x_bias, Tensor B_r, Tensor B_theta, "
              "Tensor C_r, Tensor C_theta, Tensor D, Tensor z, Tensor prev_hid_real, "
              "Tensor prev_hidden_state_imag) -> (Tensor, Tensor, Tensor)")
BWD_SCHEMA = ("ssm_adaptive_backward_unitary(Tensor grad_y,Tensor grad_next_hid_real,Tensor grad_next_hid_imag,"
              "Tensor u,Tensor dt,Tensor x,Tensor x_bias,Tensor B_r,Tensor B_theta,Tensor C_r,Tensor C_theta,"
              "Tensor D,Tensor z, Tensor prev_hid_real, Tensor prev_hid_imag) -> (Tensor, Tensor, Tensor, Tensor, "
              "Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")


def load_reference_ops(root: str):
    lib = torch.library.Library("extension_cpp", "DEF")
    lib.define(FWD_SCHEMA)
    lib.define(BWD_SCHEMA)
    path = os.path.join(root, "extension-cpp", "extension_cpp", "ops.py")
    spec = importlib.util.spec_from_file_location("_reference_ops", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod._keepalive = lib
    return mod


def inputs_reference_test(b=16, d=16, n=16, l=14):
    """The fixture of extension-cpp/test/test_extension.py:31-70 (seed 10,
    binary u, un-softplussed dt), on the CPU."""
    torch.manual_seed(10)
    u = torch.randint(0, 2, size=(b, d, l)).float()
    dt = torch.randn(b, d, l)
    x = torch.randn(d, n, d)
    x_bias = torch.randn(d, n)
    B = torch.randn(n, dtype=torch.complex64)
    C = torch.randn(n, dtype=torch.complex64)
    D = torch.randn(d)
    z = torch.randn(b, d, l)
    gy = torch.randn(b, d, l)
    return dict(u=u, dt=dt, x=x, x_bias=x_bias, B=B, C=C, D=D, z=z, gy=gy)


def inputs_model_like(seed, b, d, n, l):
    """Distributions of the benchmark configurations: u, z ~ N(0,1); dt =
    softplus(N(0,1)); x ~ N(0,1)/sqrt(d) and x_bias ~ U(-pi,pi) as the model
    initialises them (ai-modules/wavesAI/model/aussm.py:834, :891); B, C
    complex with N(0,1/n) parts; D ~ N(0,1); upstream gradient ~ N(0,1)."""
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
    return dict(u=u, dt=dt, x=x, x_bias=x_bias, B=B, C=C, D=D, z=z, gy=gy)


NAMES = ["u", "dt", "x", "x_bias", "B", "C", "D", "z"]


def run_unitary(ops, inp, dtype):
    cd = torch.complex64 if dtype == torch.float32 else torch.complex128
    args = []
    for k in NAMES:
        t = inp[k].to(cd if inp[k].is_complex() else dtype).clone().requires_grad_(True)
        args.append(t)
    y, diag = ops.reference_ssm_adaptive_unitary_optimized_polar(*args, diagnostic=True)
    (y * inp["gy"].to(dtype)).sum().backward()
    h_last = diag["h"][:, -1]                      # (b, d, n) complex, state after the last step
    out = {"y": y.detach(), "h_last": h_last.detach()}
    for k, t in zip(NAMES, args):
        out["grad_" + k] = t.grad.detach()
    return out


def to_np(t):
    return t.detach().cpu().numpy()


def save_unitary_case(ops, name, inp):
    r32 = run_unitary(ops, inp, torch.float32)
    r64 = run_unitary(ops, inp, torch.float64)
    blob = {"in_" + k: to_np(v) for k, v in inp.items()}
    blob["y_ref32"] = to_np(r32["y"])
    blob["y_ref64"] = to_np(r64["y"])
    blob["h_last_ref64"] = to_np(r64["h_last"])
    for k in NAMES:
        blob["grad32_" + k] = to_np(r32["grad_" + k])
        # float64 gradients rounded to float32 storage (6e-8 relative, far below the 1e-3 tolerance)
        g = r64["grad_" + k]
        blob["grad64_" + k] = to_np(g.to(torch.complex64 if g.is_complex() else torch.float32))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
    print(name, {k: v.shape for k, v in blob.items() if k.startswith("in_")})


def save_loop_variants(ops):
    """Small cases of the loop references for the positive-real and general
    complex recurrences (ops.py:300-357 and :233-297)."""
    g = torch.Generator().manual_seed(77)
    b, d, n, l = 2, 4, 4, 24
    r = lambda *s: torch.randn(*s, generator=g)
    u, z = r(b, d, l), r(b, d, l)
    dt = torch.nn.functional.softplus(r(b, d, l))
    D = r(d)
    x_rho = -torch.nn.functional.softplus(r(d, n, d)) * 0.1
    x_theta = r(d, n, d) / math.sqrt(d)
    Br, Cr = r(b, n, l), r(b, n, l)
    Bc = torch.complex(r(b, n, l), r(b, n, l))
    Cc = torch.complex(r(b, n, l), r(b, n, l))
    sink = io.StringIO()
    with contextlib.redirect_stdout(sink), contextlib.redirect_stderr(sink):
        y_preal = ops.reference_ssm_adaptive_preal(u, dt, x_rho, Br, Cr, D, z)
        y_cplx = ops.reference_ssm_adaptive_complex(u, dt, torch.stack([x_rho, x_theta]), Bc, Cc, D, z)
    np.savez_compressed(os.path.join(HERE, "loop_variants.npz"), u=to_np(u), dt=to_np(dt), z=to_np(z), D=to_np(D),
                        x_rho=to_np(x_rho), x_theta=to_np(x_theta), B_real=to_np(Br), C_real=to_np(Cr),
                        B_complex=to_np(Bc), C_complex=to_np(Cc), y_preal=to_np(y_preal), y_complex=to_np(y_cplx))
    print("loop_variants", tuple(u.shape))


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AUSSM_REFERENCE_ROOT", "")
    if not root or not os.path.isdir(root):
        raise SystemExit("usage: make_golden.py <path to an AUSSM checkout>")
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    ops = load_reference_ops(root)
    save_unitary_case(ops, "unitary_reference_test_shape", inputs_reference_test())
    save_unitary_case(ops, "unitary_config0", inputs_model_like(1234, 8, 16, 4, 256))
    save_unitary_case(ops, "unitary_ragged", inputs_model_like(4321, 2, 3, 5, 37))
    save_loop_variants(ops)


if __name__ == "__main__":
    main()
