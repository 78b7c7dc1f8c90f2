"""Parity of the CUDA scan core (phase tensor given) with the CPU oracle.
All calls go through the C ABI of libaussm_b200.so."""
import pytest
import torch

import aussm_b200
from aussm_b200 import _lib
from oracle import unitary as O
from tests.helpers import assert_parity, scaled_error, scan_core_inputs

pytestmark = pytest.mark.gpu

KEYS = ["theta", "u", "dt", "z", "B_r", "B_theta", "C_r", "C_theta", "D", "h0_re", "h0_im"]

# (b, d, n, l): ragged lengths take the plain-load path, multiples of 4 the bulk-copy path
SHAPES = [
    (2, 3, 4, 37), (8, 16, 4, 256), (16, 16, 16, 14), (16, 16, 16, 16), (2, 5, 16, 1000), (3, 7, 16, 192),
    (1, 2, 32, 64), (2, 2, 64, 128), (1, 1, 128, 96), (1, 3, 5, 40), (1, 1, 1, 4), (1, 1, 2, 1), (2, 9, 8, 260),
    (1, 33, 16, 4096),
]


def _oracle(inp, dtype, recurrence=True):
    a = [inp[k].to(dtype).cpu().clone().requires_grad_(True) for k in KEYS]
    fn = O.scan_unitary_recurrence if recurrence else O.scan_unitary_cumsum
    y, hr, hi = fn(*a)
    return a, y, hr, hi


def _gpu(inp):
    a = [inp[k].cuda().clone().requires_grad_(True) for k in KEYS]
    y, hr, hi = aussm_b200.scan_unitary(*a)
    return a, y, hr, hi


@pytest.mark.parametrize("shape", SHAPES)
def test_forward_matches_oracle(shape):
    inp = scan_core_inputs(100 + sum(shape), *shape)
    _, y64, hr64, hi64 = _oracle(inp, torch.float64)
    _, y32, hr32, hi32 = _oracle(inp, torch.float32, recurrence=False)   # the reference's float32 formulation
    _, y, hr, hi = _gpu(inp)
    assert aussm_b200.device_status() == 0
    assert_parity("y", y, y64, y32)
    assert_parity("h_re", hr, hr64, hr32)
    assert_parity("h_im", hi, hi64, hi32)


@pytest.mark.parametrize("shape", SHAPES)
def test_backward_matches_oracle(shape):
    inp = scan_core_inputs(200 + sum(shape), *shape)
    outs = {}
    for tag, dtype in (("t", torch.float64), ("r", torch.float32)):
        a, y, hr, hi = _oracle(inp, dtype, recurrence=(tag == "t"))
        loss = (y * inp["gy"].to(dtype)).sum() + (hr * inp["gh_re"].to(dtype)).sum() + (hi * inp["gh_im"].to(dtype)).sum()
        loss.backward()
        outs[tag] = [t.grad for t in a]
    a, y, hr, hi = _gpu(inp)
    loss = (y * inp["gy"].cuda()).sum() + (hr * inp["gh_re"].cuda()).sum() + (hi * inp["gh_im"].cuda()).sum()
    loss.backward()
    assert aussm_b200.device_status() == 0
    for k, t, g64, g32 in zip(KEYS, a, outs["t"], outs["r"]):
        # gradients: relative 1e-3 (plus a small absolute floor scaled to the tensor)
        floor = 1e-5 * float(g64.abs().max())
        assert_parity("grad_" + k, t.grad, g64, g32, atol=max(floor, 1e-7), rtol=1e-3)


def test_two_calls_chain_like_one():
    """State hand-over: one call over l steps == two calls chained through the state."""
    b, d, n, l = 2, 6, 16, 512
    inp = scan_core_inputs(7, b, d, n, l)
    g = {k: v.cuda() for k, v in inp.items()}
    y, hr, hi = aussm_b200.scan_unitary(*[g[k] for k in KEYS])
    cut = 192
    first = [g["theta"][..., :cut].contiguous(), g["u"][..., :cut].contiguous(), g["dt"][..., :cut].contiguous(),
             g["z"][..., :cut].contiguous()] + [g[k] for k in KEYS[4:]]
    y1, h1r, h1i = aussm_b200.scan_unitary(*first)
    second = [g["theta"][..., cut:].contiguous(), g["u"][..., cut:].contiguous(), g["dt"][..., cut:].contiguous(),
              g["z"][..., cut:].contiguous()] + [g[k] for k in KEYS[4:9]] + [h1r, h1i]
    y2, h2r, h2i = aussm_b200.scan_unitary(*second)
    # float32 rounding differs between the two decompositions: compare on the scale of the tensor
    assert scaled_error(torch.cat([y1, y2], -1), y) < 5e-6
    assert scaled_error(h2r, hr) < 5e-6
    assert scaled_error(h2i, hi) < 5e-6


def test_deterministic():
    b, d, n, l = 2, 8, 16, 768
    inp = scan_core_inputs(11, b, d, n, l)

    def run():
        a, y, hr, hi = _gpu(inp)
        ((y * inp["gy"].cuda()).sum() + hr.sum() - hi.sum()).backward()
        return [y.detach(), hr.detach(), hi.detach()] + [t.grad for t in a]

    ref = run()
    again = run()
    for p, q in zip(ref, again):
        assert torch.equal(p, q), "two identical launches differ"
    assert aussm_b200.device_status() == 0


def test_zero_input_gain_takes_the_general_path():
    """B_r == 0 disables the state normalisation (division by Bc)."""
    b, d, n, l = 2, 4, 8, 64
    inp = scan_core_inputs(13, b, d, n, l)
    inp["B_r"][3] = 0.0
    _, y64, hr64, hi64 = _oracle(inp, torch.float64)
    a64, y64g, hr64g, hi64g = _oracle(inp, torch.float64)
    ((y64g * inp["gy"].double()).sum() + (hr64g * inp["gh_re"].double()).sum()).backward()
    a, y, hr, hi = _gpu(inp)
    ((y * inp["gy"].cuda()).sum() + (hr * inp["gh_re"].cuda()).sum()).backward()
    assert_parity("y", y, y64, scaled_tol=1e-5)
    assert_parity("h_re", hr, hr64, scaled_tol=1e-5)
    for k, t, r in zip(KEYS, a, a64):
        assert_parity("grad_" + k, t.grad, r.grad, atol=1e-6 * float(r.grad.abs().max()) + 1e-9, rtol=1e-3,
                      scaled_tol=1e-4)


def test_plain_load_path_agrees_with_the_bulk_copy_path():
    """Rows that are not 16-byte aligned (here: a view that starts one float into a buffer) take plain loads
    and stores; same arithmetic, same results."""
    b, d, n, l = 2, 8, 16, 768
    inp = {k: v.cuda() for k, v in scan_core_inputs(11, b, d, n, l).items()}
    lib = _lib.load()
    P = lambda t: t.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream

    def shifted(t):
        return torch.empty(t.numel() + 1, device="cuda")[1:].view(t.shape).copy_(t)

    outs = []
    for shift in (False, True):
        g = {k: (shifted(v) if shift and v.dim() >= 3 and v.shape[-1] == l else v) for k, v in inp.items()}
        y = torch.empty(b * d * l + 1, device="cuda")[1 if shift else 0:][: b * d * l].view(b, d, l)
        hr, hi = torch.empty(b, d, n, device="cuda"), torch.empty(b, d, n, device="cuda")
        rc = lib.aussm_b200_scan_unitary_fwd(P(g["theta"]), P(g["u"]), P(g["dt"]), P(g["z"]), P(g["B_r"]),
                                             P(g["B_theta"]), P(g["C_r"]), P(g["C_theta"]), P(g["D"]), P(g["h0_re"]),
                                             P(g["h0_im"]), P(y), P(hr), P(hi), b, d, n, l, stream)
        _lib.check(rc, "forward")
        outs.append((y.clone(), hr, hi))
    assert outs[1][0].data_ptr() != 0
    for p, q in zip(outs[0], outs[1]):
        torch.testing.assert_close(p, q, rtol=1e-6, atol=1e-6)
    assert aussm_b200.device_status() == 0


def test_bad_arguments_are_rejected():
    lib = _lib.load()
    assert lib.aussm_b200_scan_unitary_fwd(*([None] * 14), 1, 1, 1, 1, None) != 0
    assert b"null" in lib.aussm_b200_last_error()
    t = torch.zeros(4, device="cuda")
    p = t.data_ptr()
    assert lib.aussm_b200_scan_unitary_fwd(*([p] * 14), 1, 1, 1000, 1, None) != 0      # too many states
    assert lib.aussm_b200_scan_unitary_fwd(*([p] * 14), 0, 1, 1, 1, None) != 0         # empty batch
    with pytest.raises(RuntimeError):
        aussm_b200.scan_unitary(torch.zeros(1, 1, 1, 4), *[torch.zeros(1, 1, 4)] * 3, *[torch.zeros(1)] * 5)


def test_full_size_properties():
    """The benchmark workload (batch 16, d_inner 1024, d_state 16, 16384 steps; 17 GB of phases) is too large for the
    oracle, so it is checked through properties that do not depend on the size:
    * with no input (dt = 0) every step only rotates the state: |h| after 16384 steps equals |h| before (this is the
      accuracy of the sine / cosine evaluation and of the recurrence, paid 16384 times);
    * the backward pass is linear in the upstream gradient: doubling grad_y doubles every gradient bit for bit;
    * the gradient of the initial state has the norm of the gradient of the final state when nothing else feeds in
      (the adjoint recurrence is a rotation too)."""
    free, _total = torch.cuda.mem_get_info()
    if free < 70 * 2**30:
        pytest.skip("needs about 60 GB of device memory")
    b, d, n, l = 16, 1024, 16, 16384
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(2024)
    lib = _lib.load()
    P = lambda t: None if t is None else t.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    theta = torch.empty(b, d, n, l, device=dev).uniform_(-3.2, 3.2, generator=gen)
    u = torch.randn(b, d, l, device=dev, generator=gen)
    z = torch.randn(b, d, l, device=dev, generator=gen)
    dt0 = torch.zeros(b, d, l, device=dev)
    par = {k: torch.rand(n, device=dev, generator=gen) + 0.5 for k in ("B_r", "B_theta", "C_r", "C_theta")}
    Dsk = torch.randn(d, device=dev, generator=gen)
    h0_re = torch.randn(b, d, n, device=dev, generator=gen)
    h0_im = torch.randn(b, d, n, device=dev, generator=gen)
    y = torch.empty_like(u)
    h1_re, h1_im = torch.empty_like(h0_re), torch.empty_like(h0_im)

    def fwd(dt):
        _lib.check(lib.aussm_b200_scan_unitary_fwd(P(theta), P(u), P(dt), P(z), P(par["B_r"]), P(par["B_theta"]),
                                                   P(par["C_r"]), P(par["C_theta"]), P(Dsk), P(h0_re), P(h0_im), P(y),
                                                   P(h1_re), P(h1_im), b, d, n, l, stream), "forward")

    fwd(dt0)
    n0 = torch.sqrt(h0_re.double() ** 2 + h0_im.double() ** 2)
    n1 = torch.sqrt(h1_re.double() ** 2 + h1_im.double() ** 2)
    drift = ((n1 - n0).abs() / n0.clamp_min(1e-3)).max().item()
    assert drift < 1e-4, f"norm drift over {l} steps: {drift:.3e}"

    # backward: gy = 0 and a gradient on the final state only -> the state gradient is rotated back, norm kept
    ws = torch.empty(lib.aussm_b200_scan_unitary_bwd_workspace_bytes(b, d, n, l), dtype=torch.uint8, device=dev)
    dtheta = torch.empty_like(theta)
    outs = {k: torch.empty_like(u) for k in ("du", "ddt", "dz")}
    small = {k: torch.empty(n, device=dev) for k in ("dB_r", "dB_t", "dC_r", "dC_t")}
    dD = torch.empty(d, device=dev)
    dh_re, dh_im = torch.empty_like(h0_re), torch.empty_like(h0_im)
    g_re = torch.randn(b, d, n, device=dev, generator=gen)
    g_im = torch.randn(b, d, n, device=dev, generator=gen)

    def bwd(gy, gre, gim, dt):
        _lib.check(lib.aussm_b200_scan_unitary_bwd(
            P(gy), P(gre), P(gim), P(theta), P(u), P(dt), P(z), P(par["B_r"]), P(par["B_theta"]), P(par["C_r"]),
            P(par["C_theta"]), P(Dsk), P(h1_re), P(h1_im), P(dtheta), P(outs["du"]), P(outs["ddt"]), P(outs["dz"]),
            P(small["dB_r"]), P(small["dB_t"]), P(small["dC_r"]), P(small["dC_t"]), P(dD), P(dh_re), P(dh_im), b, d, n,
            l, P(ws), ws.numel(), stream), "backward")

    gy0 = torch.zeros_like(u)
    bwd(gy0, g_re, g_im, dt0)
    gn1 = torch.sqrt(g_re.double() ** 2 + g_im.double() ** 2)
    gn0 = torch.sqrt(dh_re.double() ** 2 + dh_im.double() ** 2)
    gdrift = ((gn0 - gn1).abs() / gn1.clamp_min(1e-3)).max().item()
    assert gdrift < 1e-4, f"adjoint norm drift over {l} steps: {gdrift:.3e}"
    del gy0

    # linearity in grad_y, with input (dt > 0)
    dt = torch.rand(b, d, l, device=dev, generator=gen) * 0.1
    fwd(dt)
    gy = torch.randn(b, d, l, device=dev, generator=gen)
    bwd(gy, None, None, dt)
    ref = {k: v.clone() for k, v in outs.items()}
    ref_dth = dtheta[:, ::97, :, ::13].clone()
    ref_small = {k: v.clone() for k, v in small.items()}
    gy *= 2
    bwd(gy, None, None, dt)
    for k in outs:
        assert torch.equal(outs[k], 2 * ref[k]), k
    assert torch.equal(dtheta[:, ::97, :, ::13], 2 * ref_dth)
    for k in small:
        assert torch.allclose(small[k], 2 * ref_small[k], rtol=1e-5, atol=0), k     # summed in float32 after a polar map
    assert aussm_b200.device_status() == 0


@pytest.mark.parametrize("shape", [(1, 6, 16, 4096), (2, 3, 4, 2048), (1, 2, 32, 8192), (1, 40, 16, 1024)])
def test_time_axis_split_agrees_with_the_sequential_scan(shape):
    """Few channels: the launch is cut into time segments (aggregate pass, chain over the segments, real pass).
    Forward and backward must agree with the unsplit kernels to float32 rounding, and with the float64 oracle."""
    b, d, n, l = shape
    lib = _lib.load()
    assert lib.aussm_b200_scan_unitary_fwd_workspace_bytes(b, d, n, l) > 0, "this shape should be split"
    inp = scan_core_inputs(300 + sum(shape), *shape)

    def run():
        a, y, hr, hi = _gpu(inp)
        ((y * inp["gy"].cuda()).sum() + (hr * inp["gh_re"].cuda()).sum() + (hi * inp["gh_im"].cuda()).sum()).backward()
        return [y.detach(), hr.detach(), hi.detach()] + [t.grad for t in a]

    split = run()
    try:
        _lib.set_option("time_split", 0)
        assert lib.aussm_b200_scan_unitary_fwd_workspace_bytes(b, d, n, l) == 0
        plain = run()
    finally:
        _lib.set_option("time_split", 1)
    names = ["y", "h_re", "h_im"] + ["grad_" + k for k in KEYS]
    for name, p, q in zip(names, split, plain):
        assert scaled_error(p, q) < 2e-5, name
    a64, y64, hr64, hi64 = _oracle(inp, torch.float64)
    ((y64 * inp["gy"].double()).sum() + (hr64 * inp["gh_re"].double()).sum() + (hi64 * inp["gh_im"].double()).sum()).backward()
    assert_parity("y (split)", split[0], y64, scaled_tol=2e-5)
    for k, g, t in zip(KEYS, split[3:], a64):
        assert_parity("grad_" + k + " (split)", g, t.grad, atol=1e-5 * float(t.grad.abs().max()) + 1e-9, rtol=1e-3,
                      scaled_tol=1e-4)
    assert aussm_b200.device_status() == 0


def test_time_axis_split_in_the_drop_in_operator():
    """The windowed operator splits its scans too (few channels, long windows); same result as without."""
    from tests.helpers import NAMES, model_like_inputs
    inp = model_like_inputs(55, 1, 8, 16, 2048)

    def run():
        args = [inp[k].cuda().clone().requires_grad_(True) for k in NAMES]
        y = aussm_b200.ssm_adaptive_interface(*args, unitary=True)
        (y * inp["gy"].cuda()).sum().backward()
        return [y.detach()] + [a.grad for a in args]

    split = run()
    try:
        _lib.set_option("time_split", 0)
        plain = run()
    finally:
        _lib.set_option("time_split", 1)
    for name, p, q in zip(["y"] + NAMES, split, plain):
        if p.is_complex():
            p, q = torch.view_as_real(p), torch.view_as_real(q)
        assert scaled_error(p, q) < 5e-5, name
    assert aussm_b200.device_status() == 0
