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


def test_deterministic_and_path_independent():
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
    try:
        _lib.set_option("force_plain", 1)
        plain = run()
    finally:
        _lib.set_option("force_plain", 0)
    for p, q in zip(ref, plain):
        torch.testing.assert_close(p, q, rtol=1e-6, atol=1e-6)
    for variant in (1, 2, 3):
        try:
            _lib.set_option("variant", variant)
            other = run()
        finally:
            _lib.set_option("variant", 0)
        for p, q in zip(ref, other):
            assert scaled_error(p, q) < 1e-5
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


def test_fast_trig_option_is_close():
    b, d, n, l = 2, 4, 16, 256
    inp = scan_core_inputs(17, b, d, n, l)
    _, y64, _, _ = _oracle(inp, torch.float64)
    try:
        _lib.set_option("fast_trig", 1)
        _, y, _, _ = _gpu(inp)
    finally:
        _lib.set_option("fast_trig", 0)
    assert_parity("y(fast trig)", y, y64, scaled_tol=1e-4)


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
