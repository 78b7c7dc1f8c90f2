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
    assert y.shape == (2, 4, 32) and states.shape == (2, 4, 4, 3, 2)
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


def _op_args(inp, kind):
    c = {k: v.cuda() for k, v in inp.items()}
    if kind == "complex":
        Bc, Cc = torch.complex(c["Br"], c["Bi"]), torch.complex(c["Cr"], c["Ci"])
        return [c["u"], c["dt"], c["x_rho"], c["x_theta"], Bc.abs(), Bc.angle(), Cc.abs(), Cc.angle(), c["D"], c["z"]]
    return [c["u"], c["dt"], c["x_rho"], c["Br"], c["Cr"], c["D"], c["z"]]


@pytest.mark.parametrize("kind", ["complex", "preal"])
def test_backward_operators_by_name_match_autograd_through_the_oracle(kind):
    """extension_cpp::ssm_adaptive_backward_complex / _preal called directly with the reference host functions'
    argument lists (grad_y, grad_h, inputs..., hidden_states), against float64 autograd through the loop oracle
    in the operators' own parametrisation (B, C as radius and angle)."""
    shape = (2, 8, 16, 96)
    inp = _rand(11, *shape)
    args = _op_args(inp, kind)
    fwd = getattr(torch.ops.extension_cpp, "ssm_adaptive_" + kind)
    bwd = getattr(torch.ops.extension_cpp, "ssm_adaptive_backward_" + kind)
    y, states = fwd(*args)
    gy = inp["gy"].cuda()
    grads = bwd(gy, torch.zeros_like(states), *args, states)
    assert len(grads) == len(args)
    a64 = [a.double().cpu().requires_grad_(True) for a in args]
    if kind == "complex":
        u, dt, xr, xt, Br, Bt, Cr, Ct, D, z = a64
        ref = V.complex_ref(u, dt, torch.stack([xr, xt]), torch.polar(Br, Bt), torch.polar(Cr, Ct), D, z)
    else:
        u, dt, xr, Br, Cr, D, z = a64
        ref = V.preal_ref(u, dt, xr, Br, Cr, D, z)
    (ref * inp["gy"].double()).sum().backward()
    assert_parity("y", y, ref.detach(), scaled_tol=1e-5)
    for i, (g, a) in enumerate(zip(grads, a64)):
        assert_parity(f"{kind} grad of input {i}", g, a.grad, atol=1e-5 * float(a.grad.abs().max()) + 1e-9, rtol=1e-3,
                      scaled_tol=1e-4)
    # the same gradients through autograd of the forward operator
    leaves = [a.clone().requires_grad_(True) for a in args]
    y2, _ = fwd(*leaves)
    (y2 * gy).sum().backward()
    for g, l in zip(grads, leaves):
        # dB / dC are summed with float atomics: the order, and so the last bits, differ from call to call
        torch.testing.assert_close(l.grad, g, rtol=1e-4, atol=1e-5 * float(g.abs().max()) + 1e-7)


@pytest.mark.parametrize("kind", ["complex", "preal"])
def test_time_windows_do_not_change_the_result(kind):
    """The operators walk the time axis in windows (bounded workspace); six windows must agree with one."""
    from aussm_b200 import _lib
    shape = (2, 8, 16, 336)
    inp = _rand(5, *shape)

    def run():
        leaves = [a.clone().requires_grad_(True) for a in _op_args(inp, kind)]
        y, states = getattr(torch.ops.extension_cpp, "ssm_adaptive_" + kind)(*leaves)
        (y * inp["gy"].cuda()).sum().backward()
        return [y.detach(), states.detach()] + [l.grad for l in leaves]

    one = run()
    try:
        _lib.set_option("window_steps", 64)
        lib = _lib.load()
        # bounded workspace: it does not grow with the sequence length
        assert (lib.aussm_b200_complex_workspace_bytes(*shape, 1)
                == lib.aussm_b200_complex_workspace_bytes(shape[0], shape[1], shape[2], 16384, 1))
        six = run()
    finally:
        _lib.set_option("window_steps", 0)
    for p, q in zip(one, six):
        scale = float(p.abs().max()) + 1e-30
        assert float((p - q).abs().max()) <= 2e-5 * scale


def test_gradient_of_the_state_record_is_honoured():
    """hidden_states is a differentiable output: a loss on the recorded states reaches every input."""
    shape = (1, 4, 8, 64)
    inp = _rand(21, *shape)
    g = torch.Generator().manual_seed(3)
    gh = torch.randn(1, 4, 8, 64 // 16 + 1, 2, generator=g)
    leaves = [a.clone().requires_grad_(True) for a in _op_args(inp, "complex")]
    y, states = torch.ops.extension_cpp.ssm_adaptive_complex(*leaves)
    (states * gh.cuda()).sum().backward()
    # oracle: states of the loop recurrence at steps 16 k - 1
    a64 = [a.detach().double().cpu().requires_grad_(True) for a in leaves]
    u, dt, xr, xt, Br, Bt, Cr, Ct, D, z = a64
    A = torch.einsum("pijr,brt->pbijt", torch.stack([xr, xt]), u)
    lam = torch.polar(torch.exp(A[0]), A[1])
    Bc = torch.polar(Br, Bt)
    drive = dt * torch.nn.functional.silu(u)
    h = torch.zeros(1, 4, 8, dtype=torch.complex128)
    recs = [h]
    for t in range(64):
        h = lam[..., t] * h + drive[:, :, t, None] * Bc[:, None, :, t]
        if t % 16 == 15:
            recs.append(h)
    rec = torch.view_as_real(torch.stack(recs, dim=-1))                  # (1, 4, 8, 5, 2)
    (rec * gh.double()).sum().backward()
    assert_parity("states", states, rec.detach(), scaled_tol=1e-5)
    for i in (0, 1, 2, 3, 4, 5):                                         # u, dt, x_rho, x_theta, B_r, B_theta
        assert_parity(f"grad of input {i} from the state record", leaves[i].grad, a64[i].grad,
                      atol=1e-5 * float(a64[i].grad.abs().max()) + 1e-9, rtol=1e-3, scaled_tol=1e-4)
