"""Real selective scan (Mamba block) against the CPU oracle, through the C ABI."""
import math

import pytest
import torch

import aussm_b200
from aussm_b200.s6 import selective_scan_fn
from oracle.s6 import selective_scan_ref
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu
KEYS = ["u", "delta", "A", "B", "C", "D", "z", "delta_bias"]


def _inputs(seed, b, d, n, l):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    return dict(u=r(b, d, l), delta=r(b, d, l) * 0.5, A=-torch.exp(r(d, n)), B=r(b, n, l) / math.sqrt(n),
                C=r(b, n, l) / math.sqrt(n), D=r(d), z=r(b, d, l), delta_bias=r(d) * 0.5, gy=r(b, d, l))


# The kernels for N <= 16 give a channel 1, 2 or 4 lanes depending on how many warps the channels make: the two wide
# cases are the sizes at which the forward kernel runs with one lane (8 x 7109 channels) and with two (8 x 4001); all
# small cases run with four; the backward kernel uses two lanes at the wide sizes and four at the small ones.
@pytest.mark.parametrize("shape", [(2, 6, 16, 64), (3, 5, 16, 100), (1, 7, 4, 37), (2, 16, 8, 256), (1, 3, 32, 96),
                                   (2, 256, 16, 720), (1, 2, 5, 8), (8, 7109, 16, 48), (8, 4001, 12, 40),
                                   (1, 40, 20, 72)])
@pytest.mark.parametrize("full", [True, False])
def test_selective_scan_matches_oracle(shape, full):
    inp = _inputs(sum(shape), *shape)
    if not full:                       # no gate, no skip, no bias, no softplus
        inp["z"] = inp["D"] = inp["delta_bias"] = None
        inp["delta"] = torch.nn.functional.softplus(inp["delta"])
    outs = {}
    for tag, dtype, dev in (("t", torch.float64, "cpu"), ("r", torch.float32, "cpu"), ("g", torch.float32, "cuda")):
        a = [None if inp[k] is None else inp[k].to(dtype).to(dev).clone().requires_grad_(True) for k in KEYS]
        fn = selective_scan_fn if tag == "g" else selective_scan_ref
        y = fn(*a, delta_softplus=full)
        (y * inp["gy"].to(dtype).to(dev)).sum().backward()
        outs[tag] = (y.detach(), [None if t is None else t.grad for t in a])
    assert_parity("out", outs["g"][0], outs["t"][0], outs["r"][0])
    for k, g, t, r in zip(KEYS, outs["g"][1], outs["t"][1], outs["r"][1]):
        if g is None:
            continue
        assert_parity("grad_" + k, g, t, r, atol=1e-5 * float(t.abs().max()) + 1e-9, rtol=1e-3)
    assert aussm_b200.device_status() == 0


def test_last_state_and_errors():
    inp = _inputs(3, 2, 4, 16, 64)
    a = [inp[k].cuda() for k in KEYS]
    y, last = selective_scan_fn(*a, delta_softplus=True, return_last_state=True)
    y64, last64 = selective_scan_ref(*[inp[k].double() for k in KEYS], delta_softplus=True, return_last_state=True)
    assert_parity("out", y, y64, scaled_tol=1e-5)
    assert_parity("last_state", last, last64, scaled_tol=1e-5)
    with pytest.raises(RuntimeError):
        selective_scan_fn(*[inp[k] for k in KEYS])                       # CPU tensors
    lib = aussm_b200._lib.load()
    assert lib.aussm_b200_selective_scan_fwd(*([None] * 8), 0, *([None] * 3), 1, 1, 64, 4, None) != 0   # N > 32
