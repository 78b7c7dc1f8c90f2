"""Complex / positive-real variants against the oracle and the reference's golden outputs."""
import math

import pytest
import torch

import aussm_b200
from oracle import variants as V
from tests.helpers import assert_parity, load_golden

pytestmark = pytest.mark.gpu


def _rand(seed, b, d, n, l):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    sp = torch.nn.functional.softplus
    return dict(u=r(b, d, l), dt=sp(r(b, d, l)), z=r(b, d, l), D=r(d), x_rho=-sp(r(d, n, d)) * 0.2 / math.sqrt(d),
                x_theta=r(d, n, d) / math.sqrt(d), Br=r(b, n, l) / math.sqrt(n), Bi=r(b, n, l) / math.sqrt(n),
                Cr=r(b, n, l) / math.sqrt(n), Ci=r(b, n, l) / math.sqrt(n), gy=r(b, d, l))


def test_golden_outputs_of_the_reference_loop_functions():
    g = load_golden("loop_variants")
    c = {k: v.cuda() for k, v in g.items()}
    y = aussm_b200.ssm_adaptive_preal(c["u"], c["dt"], c["x_rho"], c["B_real"], c["C_real"], c["D"], c["z"])
    torch.testing.assert_close(y.cpu(), g["y_preal"], rtol=1e-4, atol=2e-5)
    x = torch.stack([c["x_rho"], c["x_theta"]])
    y = aussm_b200.ssm_adaptive_complex(c["u"], c["dt"], x, c["B_complex"], c["C_complex"], c["D"], c["z"])
    torch.testing.assert_close(y.cpu(), g["y_complex"], rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("shape", [(2, 4, 4, 24), (2, 8, 16, 100), (1, 6, 5, 37), (3, 12, 8, 130), (1, 4, 32, 64)])
@pytest.mark.parametrize("kind", ["complex", "preal"])
def test_variants_match_oracle(shape, kind):
    inp = _rand(sum(shape) + len(kind), *shape)

    def run(dtype, dev, gpu):
        t = {k: v.to(dtype).to(dev).clone().requires_grad_(True) for k, v in inp.items() if k != "gy"}
        if kind == "complex":
            x = torch.stack([t["x_rho"], t["x_theta"]])
            B, C = torch.complex(t["Br"], t["Bi"]), torch.complex(t["Cr"], t["Ci"])
            fn = aussm_b200.ssm_adaptive_complex if gpu else V.complex_ref
            names = ["u", "dt", "z", "D", "x_rho", "x_theta", "Br", "Bi", "Cr", "Ci"]
        else:
            x, B, C = t["x_rho"], t["Br"], t["Cr"]
            fn = aussm_b200.ssm_adaptive_preal if gpu else V.preal_ref
            names = ["u", "dt", "z", "D", "x_rho", "Br", "Cr"]
        y = fn(t["u"], t["dt"], x, B, C, t["D"], t["z"])
        (y * inp["gy"].to(dtype).to(dev)).sum().backward()
        return y.detach(), {k: t[k].grad for k in names}

    y64, g64 = run(torch.float64, "cpu", False)
    y32, g32 = run(torch.float32, "cpu", False)
    yg, gg = run(torch.float32, "cuda", True)
    assert_parity("y", yg, y64, y32)
    for k in gg:
        assert_parity("grad_" + k, gg[k], g64[k], g32[k], atol=1e-5 * float(g64[k].abs().max()) + 1e-9, rtol=1e-3)


def test_registered_operator_names():
    inp = _rand(1, 2, 4, 4, 32)
    c = {k: v.cuda() for k, v in inp.items()}
    y, states = torch.ops.extension_cpp.ssm_adaptive_preal(c["u"], c["dt"], c["x_rho"], c["Br"], c["Cr"], c["D"], c["z"])
    assert y.shape == (2, 4, 32) and states.shape == (2, 4, 4, 1, 2)
    ref = V.preal_ref(inp["u"].double(), inp["dt"].double(), inp["x_rho"].double(), inp["Br"].double(),
                      inp["Cr"].double(), inp["D"].double(), inp["z"].double())
    assert_parity("y", y, ref, scaled_tol=1e-5)
    Bc = torch.complex(inp["Br"], inp["Bi"]); Cc = torch.complex(inp["Cr"], inp["Ci"])
    y, _ = torch.ops.extension_cpp.ssm_adaptive_complex(c["u"], c["dt"], c["x_rho"], c["x_theta"], Bc.abs().cuda(),
                                                        Bc.angle().cuda(), Cc.abs().cuda(), Cc.angle().cuda(), c["D"],
                                                        c["z"])
    ref = V.complex_ref(inp["u"].double(), inp["dt"].double(), torch.stack([inp["x_rho"], inp["x_theta"]]).double(),
                        Bc.to(torch.complex128), Cc.to(torch.complex128), inp["D"].double(), inp["z"].double())
    assert_parity("y", y, ref, scaled_tol=1e-5)
